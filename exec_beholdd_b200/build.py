"""Builds libbeholdd_b200.so in-tree with nvcc for sm_100a (no other architecture, no JIT).

Usage: python -m exec_beholdd_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libbeholdd_b200.so")

SOURCES = ["api.cu", "basic_kernels.cu", "moe.cu", "matvec_mma.cu", "matvec_decode.cu", "gemm_q8_tcgen05.cu", "matvec_decode_i8.cu", "moe_grouped_i8.cu", "moe_plan.cu", "moe_rows_f16.cu", "gemm_q8_ts.cu", "gemm_q8_persistent.cu", "gemm_q8_pair.cu", "peer.cu", "ep.cu", "layer_ops.cu", "synth_kernels.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math=false",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-shared", "-lcuda"]


def _nvcc() -> str:
    return os.environ.get("NVCC") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(PKG, "..", "include", "beholdd_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"]
    if verbose:
        flags += ["-Xptxas", "-v"]
    cmd = [_nvcc(), *flags, "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed building libbeholdd_b200.so")
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
