"""Checkpoint files on the GPU: a run that is saved, rebuilt from other weights, restored and continued
ends bit for bit where the uninterrupted run ends (fp32 and bf16; captured graph)."""
import numpy as np
import pytest

from axis_b200 import checkpoint as C
from axis_b200.compile import CompiledTransformer
from oracle import step_numpy as O

pytestmark = pytest.mark.gpu
CFG = dict(vocab_size=96, dim=64, n_layers=2, n_heads=4, n_kv_heads=2, mlp_hidden=96, tie_embeddings=True)


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_resume_from_file_is_bit_exact(tmp_path, dtype):
    B, T = 2, 32
    rng = np.random.default_rng(3)
    batches = [O.make_batch(rng, CFG["vocab_size"], B, T, 0.1) for _ in range(4)]
    ct = CompiledTransformer(None, CFG, O.init_weights(CFG, seed=1), B, T, dtype=dtype, max_grad_norm=1.0)
    ct.capture()
    for x, y in batches[:2]:
        ct.replay_step(x, y)
    path = str(tmp_path / "step2.npz")
    C.save(path, ct, step=2, meta={"dtype": dtype})
    for x, y in batches[2:]:
        ct.replay_step(x, y)
    want = ct.state_dict()
    ct.eng.shutdown()

    ct2 = CompiledTransformer(None, CFG, O.init_weights(CFG, seed=99), B, T, dtype=dtype, max_grad_norm=1.0)
    hdr = C.load(path, ct2)
    assert hdr["step"] == 2 and hdr["meta"] == {"dtype": dtype} and hdr["optimizer"]["t"] == 2
    ct2.capture()
    for x, y in batches[2:]:
        ct2.replay_step(x, y)
    got = ct2.state_dict()
    assert set(got) == set(want)
    for k in want:
        assert np.array_equal(got[k], want[k]), k
    assert ct2.eng.device_status() == 0
    ct2.eng.shutdown()
