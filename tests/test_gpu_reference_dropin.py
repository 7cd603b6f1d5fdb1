"""The drop-in claim, witnessed by the reference's own code: its unmodified `axis.engine.Engine` and
`axis.compile.CompiledTransformer` (axis/engine.py:78-100, axis/compile.py:28-36, 547-615) load THIS
repository's libaxeng.so through `lib_path=` and run the reference's canonical parity fixture
(engine/modal_compile_test.py:41-71, engine/modal_bf16_test.py:70-110): the 32 reference op kinds, its
buffer plan, its per-tensor optimizer ops, eager and captured.  The comparison value is the reference's own
numpy autograd (imported from the same staged copy).  fp32: loss 1e-6, gradients 1e-5 (the reference's own gate
is 1e-4 / 1e-3).  bf16: loss 1e-3, gradients 4e-2 — the reference's lowering rounds to bf16 at more points than
this build's fused plan (separate rotary, permute, residual-add and cast passes), so its plan lands a little
above the 2e-2 that the fused plan is held to elsewhere; the reference's own gate for it is 5e-2 / 1.5e-1.

The reference tree does not exist on a GPU box; `python oracle/build_ref.py <reference checkout>` stages a
copy of its Python package (and builds its own engine) under the git-ignored oracle/_ref/.  Without that
directory the tests skip."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "axis")), reason="oracle/_ref/axis not staged")]


@pytest.fixture(scope="module")
def ref():
    """The reference's modules, the canonical fixture and its eager loss / gradients."""
    sys.path.insert(0, REF)
    try:
        import axis
        from axis import nn
        from axis.compile import CompiledTransformer
        from axis.tensor import Tensor
    finally:
        sys.path.remove(REF)
    V, B, T, D, H, KV, MLP, L = 500, 2, 32, 128, 4, 2, 256, 3
    axis.manual_seed(0)
    model = nn.Transformer(vocab_size=V, dim=D, n_layers=L, n_heads=H, n_kv_heads=KV, mlp_hidden=MLP,
                           max_seq_len=T, tie_embeddings=True)
    weights = {n: p.data.copy() for n, p in model.named_parameters()}
    rng = np.random.default_rng(0)
    toks = rng.integers(0, V, size=(B, T + 1)).astype(np.int64)
    inp, tgt = toks[:, :-1], toks[:, 1:]
    loss_t = model.loss(Tensor(inp), Tensor(tgt))
    loss_t.backward()
    grads = {n: p.grad.copy() for n, p in model.named_parameters()}
    cfg = dict(vocab_size=V, dim=D, n_layers=L, n_heads=H, n_kv_heads=KV, mlp_hidden=MLP, tie_embeddings=True)
    return dict(CT=CompiledTransformer, cfg=cfg, weights=weights, B=B, T=T, inp=inp, tgt=tgt,
                loss=float(loss_t.data), grads=grads)


def _our_lib():
    from axis_b200._build import engine_lib
    return engine_lib()


def _worst(got, want):
    return max((float(np.abs(got[n] - g).max() / (np.abs(g).max() + 1e-9)), n) for n, g in want.items())


@pytest.mark.parametrize("dtype,loss_tol,grad_tol", [("fp32", 1e-6, 1e-5), ("bf16", 1e-3, 4e-2)])
def test_reference_python_drives_this_library(ref, dtype, loss_tol, grad_tol):
    ct = ref["CT"](_our_lib(), ref["cfg"], ref["weights"], ref["B"], ref["T"], tf32=False, dtype=dtype)
    assert ct.eng.lib._name == _our_lib()
    loss = ct.step(ref["inp"], ref["tgt"], t=1)
    assert abs(loss - ref["loss"]) <= loss_tol * abs(ref["loss"]) + 1e-6, (loss, ref["loss"])
    worst = _worst(ct.grads(), ref["grads"])
    assert worst[0] <= grad_tol, worst


def test_reference_python_capture_and_replay_on_this_library(ref):
    """The reference's graph path (capture / replay_step, axis/compile.py:560-573) on this library: three
    replayed steps track three eager steps of a second instance.  Not bit for bit: the reference's own op kinds
    that its plan uses here sum with fp32 atomics (row losses in CE, EMBED_BWD, L2ACC), as in its own engine."""
    a = ref["CT"](_our_lib(), ref["cfg"], ref["weights"], ref["B"], ref["T"], tf32=False, max_grad_norm=1.0)
    eager = [a.step(ref["inp"], ref["tgt"]) for _ in range(3)]
    wa = a.get_weights()
    b = ref["CT"](_our_lib(), ref["cfg"], ref["weights"], ref["B"], ref["T"], tf32=False, max_grad_norm=1.0)
    b.capture()
    replayed = [b.replay_step(ref["inp"], ref["tgt"]) for _ in range(3)]
    assert np.allclose(replayed, eager, rtol=2e-6, atol=0)
    wb = b.get_weights()
    for n in wa:
        assert np.abs(wa[n] - wb[n]).max() <= 5e-6, n       # atomic summation order differs from run to run
    assert eager[2] < eager[0]
