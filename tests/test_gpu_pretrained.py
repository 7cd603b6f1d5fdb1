"""Checkpoint fast load on the GPU: bf16 safetensors bytes go to the device as stored, the [out,in] -> [in,out]
layout change and the widening to fp32 masters run on the device (TRANSPOSE_BF16 / CAST); weights and the first
steps equal those of the same weights handed over as fp32 arrays (axis/pretrained.py:88-153 semantics)."""
import numpy as np
import pytest

from axis_b200 import engine as E
from axis_b200.compile import CompiledTransformer
from axis_b200.engine import Engine, op
from axis_b200.pretrained import compile_pretrained
from oracle import step_numpy as O
from tests.test_pretrained_cpu import CFG, make_checkpoint

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(1, 1), (5, 3), (32, 32), (33, 65), (40, 32), (257, 130), (1536, 512)])
@pytest.mark.parametrize("dt", [0, 1])
def test_transpose_op(rows, cols, dt):
    eng = Engine()
    try:
        rng = np.random.default_rng(rows * cols)
        bits = rng.integers(0, 1 << 16, (rows, cols), dtype=np.uint16)
        bits[(bits & 0x7F80) == 0x7F80] = 0x3F80            # no NaN / inf patterns
        a = eng.alloc(rows * cols, 2)
        c = eng.alloc(rows * cols + 8, 2 if dt else 4)
        eng.upload_raw(a, bits)
        eng.run([op(E.TRANSPOSE_BF16, a=a, c=c, m=rows, n=cols, dt=dt)])
        if dt:
            assert np.array_equal(eng.download_raw(c, (cols, rows), np.uint16), bits.T)
        else:
            assert np.array_equal(eng.download(c, (cols, rows)), E.bf16_bits_to_f32(bits.T.copy()).reshape(cols, rows))
        with pytest.raises(RuntimeError):
            eng.run([op(E.TRANSPOSE_BF16, a=a, c=a, m=rows, n=cols, dt=1)])
        assert eng.device_status() == 0
    finally:
        eng.shutdown()


@pytest.mark.parametrize("dtype,lora", [("bf16", 0), ("fp32", 0), ("bf16", 4)])
def test_pretrained_step_equals_the_step_of_the_converted_weights(tmp_path, dtype, lora):
    cfg = dict(CFG, tie_embeddings=(lora == 0))
    expect = make_checkpoint(str(tmp_path), cfg, "BF16", 2)
    kw = dict(lora_r=lora, lora_alpha=8.0, lora_targets=("q_proj", "v_proj", "down_proj")) if lora else {}
    rng = np.random.default_rng(3)
    batches = [O.make_batch(rng, cfg["vocab_size"], 2, 16, 0.1) for _ in range(3)]

    ct = compile_pretrained(str(tmp_path), 2, 16, dtype=dtype, max_grad_norm=1.0, **kw)
    if not lora:
        got = ct.get_weights()
        assert set(got) == set(expect)
        for nm in expect:
            assert np.array_equal(got[nm], expect[nm]), nm
    else:
        for nm, w in expect.items():
            assert np.array_equal(E.bf16_bits_to_f32(ct.eng.download_raw(ct.pb[nm], w.size, np.uint16)).reshape(w.shape), w), nm
    la = [ct.step(*b) for b in batches]
    wa = ct.get_weights()
    assert ct.eng.device_status() == 0
    ref = CompiledTransformer(None, dict(cfg, rope_theta=50000.0), expect, 2, 16, dtype=dtype, eps=1e-6,
                              max_grad_norm=1.0, **kw)
    lb = [ref.step(*b) for b in batches]
    wb = ref.get_weights()
    assert la == lb                  # small shapes: every kernel on the path sums in a fixed order
    for nm in wa:
        assert np.array_equal(wa[nm], wb[nm]), nm
