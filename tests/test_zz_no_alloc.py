"""The allocation-free RMSNorm backward (`eng_rmsnorm_bwd_noalloc`) against the
regular op (`RMSNORM_BWD_ACC` through `eng_run_plan`), which takes its scratch
from a caller-allocated buffer.

The entry point exists for callers that cannot allocate device memory at the
point of the call — during CUDA-graph stream capture, under a fixed memory
budget, or inside latency-critical loops — so its dw partials live in a static
device array inside the library.  The test drives it through the C ABI with
raw device pointers (taken from torch tensors here, which stand in for a
caller's own memory), twice in a row on different data, and compares dx and dw
with the regular op on the same inputs.  The file name makes pytest collect it
last, so a failure here cannot hide results of the other GPU tests."""
import ctypes

import numpy as np
import pytest

from axis_b200 import engine as E
from axis_b200.engine import Engine, op
from oracle import step_numpy as O

pytestmark = pytest.mark.gpu


def _regular(eng, x, w, g, res, dt, rows, dim):
    """dx, dw from the existing entry point (engine buffers + caller-provided scratch)."""
    def put(a):
        i = eng.alloc(a.size, 2 if dt else 4)
        eng.upload_bf16(i, a) if dt else eng.upload(i, a)
        return i
    ix, iw, ig, ir = put(x), put(w), put(g), put(res)
    idx, idw, iscr = eng.alloc(rows * dim, 2 if dt else 4), eng.alloc(dim), eng.alloc(296 * dim)
    eng.run([op(E.RMSNORM_BWD_ACC, a=ix, b=iw, d=ig, c=idx, tb=ir, sa=idw, sb=iscr, m=rows, n=dim, dt=dt, alpha=1e-5)])
    dx = eng.download_bf16(idx, (rows, dim)) if dt else eng.download(idx, (rows, dim))
    return dx, eng.download(idw, dim)


@pytest.mark.parametrize("dt", [0, 1])
def test_noalloc_matches_regular_entry_point_twice(dt):
    torch = pytest.importorskip("torch")
    eng = Engine()
    eng.alloc(4)
    fn = eng.lib.eng_rmsnorm_bwd_noalloc
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    tdt = torch.bfloat16 if dt else torch.float32
    rnd = lambda rng, sh: (E.bf16_bits_to_f32(E.f32_to_bf16_bits(rng.standard_normal(sh).astype(np.float32)))
                           if dt else rng.standard_normal(sh).astype(np.float32))
    for call, (rows, dim) in enumerate([(300, 1536), (77, 256)]):       # two calls in a row share the static scratch
        rng = np.random.default_rng(10 + call)
        x, w, g, res = rnd(rng, (rows, dim)), rnd(rng, dim), rnd(rng, (rows, dim)), rnd(rng, (rows, dim))
        dx_ref, dw_ref = _regular(eng, x, w, g, res, dt, rows, dim)
        dev = lambda a: torch.from_numpy(a).to("cuda", dtype=tdt).contiguous()
        tx, tw, tg, tr = dev(x), dev(w), dev(g), dev(res)
        tdx = torch.empty((rows, dim), device="cuda", dtype=tdt)
        tdw = torch.empty(dim, device="cuda", dtype=torch.float32)
        torch.cuda.synchronize()
        stream = torch.cuda.current_stream().cuda_stream
        rc = fn(tx.data_ptr(), tw.data_ptr(), tg.data_ptr(), tr.data_ptr(), tdx.data_ptr(), tdw.data_ptr(),
                rows, dim, dt, 1e-5, ctypes.c_void_p(stream))
        assert rc == 0
        torch.cuda.synchronize()
        dx = tdx.float().cpu().numpy()
        dw = tdw.cpu().numpy()
        tol = 1.2e-2 if dt else 2e-5
        assert np.abs(dx - dx_ref).max() <= tol * (np.abs(dx_ref).max() + 1e-6)
        assert np.abs(dw - dw_ref).max() <= tol * (np.abs(dw_ref).max() + 1e-6)
        # and against the CPU oracle's RMSNorm backward (plus the residual that the op adds to dx)
        _, inv = O.rmsnorm_fwd(x, w, 1e-5)
        dx_o, dw_o = O.rmsnorm_bwd(x, w, inv, g)
        assert np.abs(dx - (dx_o + res)).max() <= tol * (np.abs(dx_o + res).max() + 1e-6)
        assert np.abs(dw - dw_o).max() <= tol * (np.abs(dw_o).max() + 1e-6)
    # an empty batch: the column sums are zero and are written as such, dx is left alone
    tdw.fill_(7.0)
    torch.cuda.synchronize()
    assert fn(tx.data_ptr(), tw.data_ptr(), tg.data_ptr(), None, tdx.data_ptr(), tdw.data_ptr(), 0, dim, dt, 1e-5,
              ctypes.c_void_p(stream)) == 0
    torch.cuda.synchronize()
    assert float(tdw.abs().max()) == 0.0
    # sizes beyond the built-in scratch are refused, not truncated
    assert fn(tx.data_ptr(), tw.data_ptr(), tg.data_ptr(), None, tdx.data_ptr(), None, 1, 8193, dt, 1e-5, None) == 201
    assert fn(None, tw.data_ptr(), tg.data_ptr(), None, tdx.data_ptr(), None, 1, 64, dt, 1e-5, None) == 202
    eng.shutdown()
