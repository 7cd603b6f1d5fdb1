"""Build libaxeng.so in-tree with nvcc for sm_100a.

    python -m axis_b200._build            # build if sources changed
    python -m axis_b200._build --force

The library lands in axis_b200/_lib/libaxeng.so, next to the object files.
`engine_lib()` returns its path (building on first use when a compiler is
available), or the path in $AXIS_ENGINE_LIB when that is set — the same
override the reference's axis/_build.py:84-89 honours.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "_lib_prof" if os.environ.get("AXENG_BUILD_PROF") else "_lib")
LIB = os.path.join(LIBDIR, "libaxeng.so")
SOURCES = ["axeng.cu", "elementwise.cu", "norm.cu", "loss.cu", "optim.cu", "gemm_simt.cu",
           "gemm_tc.cu", "gemm_tc2.cu", "attn_simt.cu", "attn_tc.cu", "attn_tc128.cu", "lora.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC"]
if os.environ.get("AXENG_BUILD_PROF"):      # instrumented build: in-kernel cycle stamps of the GEMM / attention kernels
    NVCC_FLAGS.append("-DAXENG_PROF")


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.isabs(c) and os.path.exists(c) or not os.path.isabs(c)):
            return c
    return "nvcc"


def _nccl_paths():
    """Include and library directory of the NCCL that PyTorch itself loads (the
    `nvidia.nccl` wheel), so that a process importing both torch and this engine
    ends up with one NCCL; the system NCCL is the fallback."""
    try:
        import importlib.util
        spec = importlib.util.find_spec("nvidia.nccl")
        if spec and spec.submodule_search_locations:
            base = list(spec.submodule_search_locations)[0]
            inc, lib = os.path.join(base, "include"), os.path.join(base, "lib")
            if os.path.exists(os.path.join(inc, "nccl.h")) and os.path.exists(os.path.join(lib, "libnccl.so.2")):
                return inc, lib
    except (ImportError, ValueError):
        pass
    return None, None


def _digest() -> str:
    h = hashlib.sha256()
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for fn in sorted(os.listdir(root)):
            if fn.endswith((".cu", ".cuh", ".h")):
                with open(os.path.join(root, fn), "rb") as f:
                    h.update(fn.encode()); h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    stamp = os.path.join(LIBDIR, "build.sha256")
    dig = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read() == dig:
        return LIB
    nvcc = _nvcc()
    nccl_inc, nccl_lib = _nccl_paths()
    inc_flags = ["-I", nccl_inc] if nccl_inc else []

    def compile_one(src):
        obj = os.path.join(LIBDIR, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *inc_flags, "-Xptxas", "-v" if verbose else "-warn-spills", "-c",
               os.path.join(CSRC, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    if nccl_lib:
        nccl_link = ["-L", nccl_lib, "-l:libnccl.so.2", "-Xlinker", f"-rpath={nccl_lib}"]
    else:
        nccl_link = ["-lnccl"]
    link = [nvcc, "-shared", "-o", LIB, *objs, *nccl_link, "-cudart", "static"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(stamp, "w") as f:
        f.write(dig)
    return LIB


def engine_lib() -> str:
    env = os.environ.get("AXIS_ENGINE_LIB")
    if env:
        return env
    if os.path.exists(LIB):
        stamp = os.path.join(LIBDIR, "build.sha256")
        try:
            if open(stamp).read() == _digest():
                return LIB
        except OSError:
            pass
    try:
        return build()
    except (RuntimeError, FileNotFoundError) as e:
        if os.path.exists(LIB):
            return LIB
        raise RuntimeError(f"libaxeng.so is not built and cannot be built here: {e}")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
