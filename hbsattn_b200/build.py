"""Builds libhbsattn_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python hbsattn_b200/build.py [--force] [--verbose] [--strict]
    (run as a script: importing the package needs the library)

--strict also builds libhbsattn_b200_strict.so: the same sources with -DHBSA_STRICT_TCGEN05, in which the MMA
thread of the tensor-core kernel fences after every barrier it observes and waits for the P V products of a lane
to complete before the next S product overwrites their operand.  It exists to check, bit for bit, the ordering
the shipped library relies on (tests/test_gpu_strict_order.py); select it with HBSATTN_B200_LIBRARY=<path>.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libhbsattn_b200.so")
STRICT_LIB_PATH = os.path.join(PKG_DIR, "libhbsattn_b200_strict.so")
SOURCES = ["hbsa_api.cu", "hbsa_schedule.cu", "hbsa_fwd_generic.cu", "hbsa_fwd_sm100.cu",
           "hbsa_bwd_generic.cu", "hbsa_static_scratch.cu"]
HEADERS = ["hbsa_common.cuh", "sm100_ptx.cuh", os.path.join("..", "..", "include", "hbsattn_b200.h")]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; hbsattn_b200 has no CPU fallback and cannot be built without CUDA")
    return cand


def nvcc_flags(verbose: bool = False):
    flags = ["-O3", "-std=c++17", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
             "-Xcompiler", "-fPIC", "-I", os.path.join(PKG_DIR, "..", "include")]
    if verbose:
        flags += ["-Xptxas", "-v"]
    return flags


def is_stale(path: str = LIB_PATH) -> bool:
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, strict: bool = False) -> str:
    """Compile every CUDA source into hbsattn_b200/libhbsattn_b200.so (or, with strict=True, into
    libhbsattn_b200_strict.so with -DHBSA_STRICT_TCGEN05); returns the path."""
    out = STRICT_LIB_PATH if strict else LIB_PATH
    if not force and not is_stale(out):
        return out
    cmd = [_nvcc(), "-shared", "-o", out] + nvcc_flags(verbose) + (["-DHBSA_STRICT_TCGEN05"] if strict else []) + \
        [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building %s (exit %d)" % (os.path.basename(out), res.returncode))
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--strict" in sys.argv:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, strict=True))
