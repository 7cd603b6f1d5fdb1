"""The C-ABI library without a GPU: it loads, exports every entry point that
include/axeng.h declares, keeps the reference's struct layout and op numbering,
and fails loudly (no CPU fallback) when no CUDA device is present."""
import ctypes
import os
import re

import numpy as np
import pytest

from axis_b200 import engine as E
from axis_b200._build import engine_lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    return ctypes.CDLL(engine_lib())


def test_exports_match_header(lib):
    src = open(os.path.join(ROOT, "include", "axeng.h")).read()
    names = sorted(set(re.findall(r"\b(eng_[a-z0-9_]+)\s*\(", src)))
    assert len(names) >= 12
    for n in ("eng_init", "eng_alloc", "eng_has_flash", "eng_nccl_id", "eng_nccl_init", "eng_upload",
              "eng_download", "eng_run_plan", "eng_capture_plan", "eng_replay", "eng_sync", "eng_set_tf32"):
        assert n in names                      # the reference's twelve (axis/engine.py:81-100)
    for n in names:
        assert hasattr(lib, n), n


def test_struct_and_kind_numbering_match_reference():
    assert ctypes.sizeof(E._EngOp) == 80
    assert [f[0] for f in E._EngOp._fields_] == ["kind", "a", "b", "c", "d", "m", "n", "k", "batch", "tb",
                                                  "sa", "sb", "sc", "dt", "oa", "ob", "oc", "alpha", "beta", "gamma"]
    assert (E.GEMM, E.ADAMW, E.GEMM_SB, E.ROPE, E.CE, E.FLASH, E.FLASH_BWD, E.ALLREDUCE, E.BROADCAST) == \
        (0, 5, 8, 10, 20, 23, 25, 26, 31)
    src = open(os.path.join(ROOT, "include", "axeng.h")).read()
    for name, val in re.findall(r"ENG_([A-Z0-9_]+) = (\d+)", src):
        if name in E.KIND_NAMES:
            assert E.KIND_NAMES.index(name) == int(val), name
    o = E.op(E.GEMM_SB, a=1, b=2, c=3, m=4, n=5, k=6, tb=1, dt=2, alpha=0.5)
    pp = E.PackedPlan([o])
    raw = E._EngOp.from_buffer_copy(pp.arr.tobytes())
    assert (raw.kind, raw.a, raw.b, raw.c, raw.d, raw.m, raw.n, raw.k, raw.tb, raw.dt, raw.alpha) == \
        (8, 1, 2, 3, -1, 4, 5, 6, 1, 2, 0.5)


def test_bf16_conversion_is_round_to_nearest_even():
    a = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.3895314e38, 0.0], dtype=np.float32)
    b = E.bf16_bits_to_f32(E.f32_to_bf16_bits(a))
    assert b[0] == 1.0 and b[1] == 1.0 and b[2] == 1.015625 and b[3] == -2.5 and b[5] == 0.0


def _have_gpu():
    try:
        cu = ctypes.CDLL("libcuda.so.1")
        n = ctypes.c_int(0)
        return cu.cuInit(0) == 0 and cu.cuDeviceGetCount(ctypes.byref(n)) == 0 and n.value > 0
    except OSError:
        return False


@pytest.mark.skipif(_have_gpu(), reason="checks the no-device behaviour")
def test_no_device_means_loud_failure(lib):
    lib.eng_last_error.restype = ctypes.c_char_p
    assert lib.eng_init() != 0
    assert b"CUDA" in lib.eng_last_error()
    with pytest.raises(RuntimeError, match="engine init failed"):
        E.Engine()
