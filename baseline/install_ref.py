"""Installs the UNMODIFIED reference package (zhengqigao/hbsattn) into baseline/_ref/ for comparison runs.

    HBSATTN_REFERENCE=<reference checkout> python baseline/install_ref.py

What it does: copies the checkout to a temporary directory (pip writes build files into the source tree
and the checkout may be read-only) and runs

    python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
        --target baseline/_ref <copy>

The reference's test/ directory (its accuracy test and speed script) is placed beside the package as
baseline/_ref/test/.  baseline/_ref/ is not tracked by git.  Nothing in hbsattn_b200/ imports it: it is used only by the comparison
legs of bench.py (the reference's Triton kernels timed on the same GPU and inputs; its unmodified PyTorch
code timed on the host cores) and by tests/test_gpu_vs_reference.py (our output against the reference's own
Triton output).  When baseline/_ref is absent those legs say so and the tests skip.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
TARGET = os.path.join(HERE, "_ref")


def reference_checkout():
    """The checkout named by HBSATTN_REFERENCE, else a directory called `reference` beside this repository."""
    cand = os.environ.get("HBSATTN_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isfile(os.path.join(cand, "hbsattn", "hbsa_interface.py")) else None


def install(force: bool = False) -> str:
    if os.path.isfile(os.path.join(TARGET, "hbsattn", "hbsa_interface.py")) and not force:
        return TARGET
    src = reference_checkout()
    if src is None:
        raise RuntimeError("no reference checkout: set HBSATTN_REFERENCE to the directory that holds hbsattn/ and setup.py")
    with tempfile.TemporaryDirectory() as tmp:
        copy = os.path.join(tmp, "ref_src")
        shutil.copytree(src, copy, ignore=shutil.ignore_patterns("__pycache__", ".git", "assets"))
        if os.path.isdir(TARGET):
            shutil.rmtree(TARGET)
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps",
               "--find-links", "/opt/wheelhouse", "--target", TARGET, copy]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("pip install of the reference failed:\n" + res.stdout[-2000:] + res.stderr[-2000:])
        # the reference's own test scripts are not part of its package; keep them beside it for the comparison tests
        shutil.copytree(os.path.join(copy, "test"), os.path.join(TARGET, "test"), ignore=shutil.ignore_patterns("__pycache__"))
    return TARGET


if __name__ == "__main__":
    print(install(force="--force" in sys.argv))
