"""Builds libdmm.so (the CUDA library behind the C ABI in include/dmm.h) with nvcc for sm_100a.

The library is a single translation unit, csrc/dmm_api.cu, which includes the kernel
headers; the result is written next to this file so that it travels with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libdmm.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def sources():
    out = []
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".cu", ".cuh", ".h"))]
    out.append(os.path.join(HERE, "..", "include", "dmm.h"))
    return out


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(s) > t for s in sources())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library when it is missing or older than its sources; returns its path.

    Safe when several processes (one rank per GPU) import the package at once: the build runs
    under a file lock, into a temporary name that is renamed over the library only when nvcc
    succeeded, and a process that waited for the lock looks again before building."""
    if not force and not needs_build():
        return LIB
    import fcntl

    with open(LIB + ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and not needs_build():
                return LIB
            nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
            tmp = f"{LIB}.{os.getpid()}.tmp"
            cmd = [nvcc, *NVCC_FLAGS, "-o", tmp, os.path.join(CSRC, "dmm_api.cu")]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                if os.path.exists(tmp):
                    os.remove(tmp)
                raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
            os.replace(tmp, LIB)
            if verbose:
                sys.stderr.write(res.stderr)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
