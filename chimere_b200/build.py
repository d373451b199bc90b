"""Build the CUDA library in-tree for sm_100a: chimere_b200/libchimere_b200_moe.so.

    python -m chimere_b200.build            # rebuild if sources are newer than the library
    python -m chimere_b200.build --force

nvcc cross-compiles without a GPU.  The flags are the ones the reference's build scripts use
(chimere-server/ffi/build.rs:103-160: -O3 -std=c++17 -fPIC) with the architecture replaced by
-gencode arch=compute_100a,code=sm_100a.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libchimere_b200_moe.so")
SOURCES = ["abi.cu", "gemm_i8.cu", "gemv.cu", "gemv_tiled.cu", "gguf.cpp", "kquant.cu", "pack.cu", "router.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--compiler-options", "-fPIC", "-shared"]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "chimere_b200_moe.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + r.stdout + r.stderr)
    if verbose:
        print(r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
