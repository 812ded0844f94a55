"""Builds libckl_gemm.so (the C ABI plus the ckl:: C++ entry points) in-tree.

One nvcc invocation, sm_100a only.  The output sits next to this file so it
travels with the source tree; nothing is installed into site-packages.
"""

from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libckl_gemm.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _inputs() -> list[str]:
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    deps += glob.glob(os.path.join(ROOT, "include", "*.h"))
    deps += glob.glob(os.path.join(ROOT, "include", "ckl", "*.hpp"))
    return deps


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > built for p in _inputs())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile if the library is missing or older than a source; returns its path."""
    if not force and not is_stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    # link into a scratch name and rename: a reader never sees a half-written library
    scratch = LIB + f".{os.getpid()}.partial"
    cmd = [nvcc, *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-o", scratch, *sources()]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
        print(" ".join(cmd), file=sys.stderr)
    try:
        subprocess.run(cmd, check=True)
        os.replace(scratch, LIB)
    finally:
        if os.path.exists(scratch):
            os.remove(scratch)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB)
