"""Build ``libmoda_b200.so`` in-tree with nvcc for sm_100a.

    python -m moda_b200.build [--force] [--verbose]

The library is a plain C-ABI shared object (no torch, no pybind); it is rebuilt when the hash
of the files under ``moda_b200/csrc`` and ``include/`` (and of the compiler flags) differs from the
one in the stamp file beside the ``.so``.  Builds are serialised by a lock file and the library is
moved into place in one piece, so the ranks of a multi-GPU launch can all call ``build()``.

``build_wait_test()`` compiles the same sources with ``-DMODA_WAIT_TEST`` into
``libmoda_b200_waittest.so``: a test-only build in which the tcgen05 forwards and the dq /
dk/dv kernels withhold one barrier arrival and every bounded wait gives up after about a
millisecond, so that the wait-expiry teardown path can be exercised on a GPU without hanging it.  The
product never loads that file.
"""
from __future__ import annotations

import fcntl
import glob
import hashlib
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


def _digest(extra) -> str:
    """Hash of everything the library is built from: sources, headers, compiler flags."""
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + list(extra)).encode())
    deps = sorted(glob.glob(os.path.join(CSRC, "*")) + glob.glob(os.path.join(ROOT, "include", "*.h")))
    for d in deps:
        if os.path.isfile(d):
            h.update(os.path.basename(d).encode())
            with open(d, "rb") as f:
                h.update(f.read())
    return h.hexdigest()


def _stale(out: str = OUT, extra=()) -> bool:
    """The library is current when the stamp beside it holds the hash of the present sources.
    File times play no part: a checkout or a copy of the tree changes them without changing a byte."""
    stamp = out + ".stamp"
    if not (os.path.exists(out) and os.path.exists(stamp)):
        return True
    with open(stamp) as f:
        return f.read().strip() != _digest(extra)


def _compile(out: str, extra, force: bool, verbose: bool) -> str:
    if not force and not _stale(out, extra):
        return out
    # One builder at a time, and the file appears in one piece: the ranks of a multi-GPU launch all
    # come here, and a library that another process is still writing must never be loaded.
    with open(out + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not _stale(out, extra):      # built by another process in the meantime
                return out
            nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
            tmp = f"{out}.tmp.{os.getpid()}"
            cmd = [nvcc] + NVCC_FLAGS + list(extra) + (["-Xptxas", "-v"] if verbose else []) + ["-o", tmp] + sources()
            res = subprocess.run(cmd, capture_output=True, text=True)
            if verbose or res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("nvcc failed building " + os.path.basename(out))
            os.replace(tmp, out)
            with open(out + ".stamp.tmp", "w") as f:
                f.write(_digest(extra) + "\n")
            os.replace(out + ".stamp.tmp", out + ".stamp")
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return out


def build(force: bool = False, verbose: bool = False) -> str:
    return _compile(OUT, [], force, verbose)


def build_wait_test(force: bool = False, verbose: bool = False) -> str:
    return _compile(OUT_WAIT_TEST, ["-DMODA_WAIT_TEST"], force, verbose)


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--wait-test" in sys.argv:
        print(build_wait_test(force="--force" in sys.argv))
