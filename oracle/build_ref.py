"""Build the reference's own engine and stage its Python package, for comparison runs on a GPU box.

    python oracle/build_ref.py /path/to/reference

Outputs go to oracle/_ref/ only (git-ignored; it travels to the GPU box with the other built files):

    oracle/_ref/libaxeng_ref.so   the reference's axis/_csrc/runtime.cu compiled from where it lies, for sm_100a,
                                  with the flags of its own recipe (axis/_build.py:52-80: nvcc -O3 --shared
                                  -Xcompiler -fPIC ... -lcublas, without NCCL)
    oracle/_ref/axis/             a copy of the reference's Python package, so that its unmodified
                                  axis.engine.Engine / axis.compile.CompiledTransformer can be imported there
                                  (the reference tree itself does not exist on the GPU box)

This is test and measurement infrastructure: tests/test_gpu_reference_dropin.py drives THIS repository's
libaxeng.so with the reference's own Python, and opbench.py --lib times the reference's kernels as the
kernel-to-beat.  Nothing in axis_b200/ imports or loads anything from here.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def build(ref_root: str) -> str:
    src = os.path.join(ref_root, "axis", "_csrc", "runtime.cu")
    if not os.path.exists(src):
        raise FileNotFoundError(src)
    os.makedirs(OUT, exist_ok=True)
    lib = os.path.join(OUT, "libaxeng_ref.so")
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O3", "-arch=sm_100a", "--shared", "-Xcompiler", "-fPIC", src, "-lcublas", "-o", lib]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("reference engine build failed:\n" + r.stderr[-3000:])
    pkg = os.path.join(OUT, "axis")
    if os.path.isdir(pkg):
        shutil.rmtree(pkg)
    shutil.copytree(os.path.join(ref_root, "axis"), pkg,
                    ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "_csrc"))
    for root, dirs, files in os.walk(pkg):          # the source tree may be read-only; the copy must be replaceable
        for n in dirs + files:
            q = os.path.join(root, n)
            os.chmod(q, os.stat(q).st_mode | 0o200)
    os.chmod(pkg, os.stat(pkg).st_mode | 0o200)
    return lib


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python oracle/build_ref.py <path to a checkout of the reference repository>")
    print(build(sys.argv[1]))
