"""Installs the UNMODIFIED reference package into ``baseline/_ref`` (git-ignored).

    python baseline/install_reference.py [path to a hustvl/MoDA checkout]   (default: $MODA_REFERENCE_DIR)

The reference's Python package (``libs/moda_triton``: the ``fla`` tree with its Triton kernels) is
built into a wheel from a temporary copy (the checkout itself may be read-only) and installed with
``pip --no-index --no-deps --target baseline/_ref``; its dependencies (torch, triton, einops,
transformers) are the ones already in the environment.  Nothing of it is committed, and the product
package never imports it: the only user is ``bench.py --impl triton_baseline``, which times the
reference's Triton operators on the GPU as a reported baseline.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("MODA_REFERENCE_DIR", os.path.join(os.sep, "root", "reference"))
    src = os.path.join(ref, "libs", "moda_triton")
    if not os.path.isdir(os.path.join(src, "fla")):
        raise SystemExit(f"{src} does not hold the reference package")
    target = os.path.join(HERE, "_ref")
    with tempfile.TemporaryDirectory() as tmp:
        work = os.path.join(tmp, "moda_triton")
        shutil.copytree(src, work, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", ".git"))
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--upgrade", "--target", target, work]
        if os.path.isdir("/opt/wheelhouse"):
            cmd[5:5] = ["--find-links", "/opt/wheelhouse"]
        subprocess.run(cmd, check=True)
    print("installed into", target)


if __name__ == "__main__":
    main()
