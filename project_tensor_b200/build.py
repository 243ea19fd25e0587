"""Build libtq_sm100.so (the CUDA kernels plus their C ABI) in-tree with nvcc for sm_100a.

    python -m project_tensor_b200.build          # rebuild if a source is newer than the library
    python -m project_tensor_b200.build --force
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
SRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libtq_sm100.so")
SOURCES = ["tq_api.cu", "tq_exact.cu", "tq_score.cu", "tq_score_tc.cu", "tq_pack.cu", "tq_tensor.cu", "tq_dequant_tc.cu", "tq_score_few.cu", "tq_decode_attn.cu", "tq_score_lut.cu"]
HEADERS = [os.path.join(SRC_DIR, "tq_common.cuh"), os.path.join(SRC_DIR, "tq_ptx.cuh"),
           os.path.join(PKG_DIR, "..", "include", "tq_b200.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(SRC_DIR, s) for s in SOURCES] + HEADERS
    return any(os.path.exists(p) and os.path.getmtime(p) > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu file into one shared library; returns its path."""
    if not force and not stale():
        return LIB_PATH
    cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xcompiler", "-fPIC", "-shared", "--threads", "0"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += os.environ.get("TQ_NVCC_FLAGS", "").split()   # extra compiler flags, e.g. -DTQ_PROF for experiments
    cmd += [os.path.join(SRC_DIR, s) for s in SOURCES]
    cmd += ["-o", LIB_PATH]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
