"""Builds ``libquest_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

    python -m quest_b200.build [--force] [--verbose]

No torch headers, no pybind: the library exports plain ``extern "C"`` functions (see
``include/quest_b200.h``) and is loaded with ctypes.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libquest_b200.so")
SOURCES = ("quantize.cu", "gemm_i4.cu")
HEADERS = (os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "tcgen05.cuh"), os.path.join(CSRC, "hadamard_quant_tc.cuh"), os.path.join(CSRC, "gemv_i4.cuh"),
           os.path.join(ROOT, "include", "quest_b200.h"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "-cudart", "static",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def up_to_date() -> bool:
    if not os.path.exists(LIB_PATH):
        return False
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, s) for s in SOURCES] + list(HEADERS) + [os.path.abspath(__file__)]
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False, out: str = LIB_PATH) -> str:
    """Compile the library.  ``trace=True`` adds the in-kernel timeline probes (a tuning build; give it another
    ``out`` path so that it never replaces the product library)."""
    if not force and not trace and up_to_date():
        return LIB_PATH
    nvcc = find_nvcc()
    cmd = [nvcc, *NVCC_FLAGS, *(["-DQB200_TRACE"] if trace else []), "-shared", "-o", out,
           *[os.path.join(CSRC, s) for s in SOURCES]]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr)
    return out


if __name__ == "__main__":
    if "--trace" in sys.argv:
        print(build(force=True, verbose="--verbose" in sys.argv, trace=True,
                    out=os.path.join(PKG_DIR, "libquest_b200_trace.so")))
    else:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
