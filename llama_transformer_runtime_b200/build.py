"""Builds ``libpaged_attention.so`` in-tree with nvcc for sm_100a.

    python -m llama_transformer_runtime_b200.build [--verbose]

One shared library, C-ABI only (include/paged_attention.h); it links the CUDA
runtime statically-resolved symbols through nvcc's default cudart and nothing
from torch.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libpaged_attention.so")

SOURCES = ["capi.cu", "append_kernel.cu", "decode_kernel.cu", "decode_noalloc.cu", "exchange.cu", "head_gather.cu",
           "prefill_kernel.cu", "compat.cu", "compat_cxx.cu", "qkv_project.cu", "qkv_gemm.cu", "rmsnorm.cu", "ffn.cu", "sampling.cu", "embedding.cu", "block_pool.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared", "-cudart", "shared",
]


def sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "paged_attention.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(verbose: bool = False, force: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + sources()
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libpaged_attention.so")
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
