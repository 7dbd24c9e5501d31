"""Build ``libmoda_b200.so`` in-tree with nvcc for sm_100a.

    python -m moda_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (no torch, no pybind); it is rebuilt when
any file under ``moda_b200/csrc`` or ``include/`` is newer than the ``.so``.

``build_wait_test()`` compiles the same sources with ``-DMODA_WAIT_TEST`` into
``libmoda_b200_waittest.so``: a test-only build in which the tcgen05 forwards and the dq /
dk/dv kernels withhold one barrier arrival and every bounded wait gives up after about a
millisecond, so that the wait-expiry teardown path can be exercised on a GPU without hanging it.  The
product never loads that file.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libmoda_b200.so")
OUT_WAIT_TEST = os.path.join(HERE, "libmoda_b200_waittest.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _stale(out: str = OUT) -> bool:
    if not os.path.exists(out):
        return True
    t = os.path.getmtime(out)
    deps = glob.glob(os.path.join(CSRC, "*")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(out: str, extra, force: bool, verbose: bool) -> str:
    if not force and not _stale(out):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc] + NVCC_FLAGS + list(extra) + (["-Xptxas", "-v"] if verbose else []) + ["-o", out] + sources()
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building " + os.path.basename(out))
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    return _compile(OUT, [], force, verbose)


def build_wait_test(force: bool = False, verbose: bool = False) -> str:
    return _compile(OUT_WAIT_TEST, ["-DMODA_WAIT_TEST"], force, verbose)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--wait-test" in sys.argv:
        print(build_wait_test(force="--force" in sys.argv))
