"""Build recipe of the native library: one nvcc call, sm_100a only, output in-tree."""

from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SOURCES = [os.path.join(HERE, "csrc", "pi05_engine.cu"), os.path.join(HERE, "csrc", "pi05_prefill.cu")]
HEADERS = [os.path.join(HERE, "csrc", "ptx_sm100.cuh"), os.path.join(HERE, "csrc", "pi05_common.cuh"),
           os.path.join(HERE, "csrc", "pi05_chunk_kernel.cuh"),
           os.path.join(os.path.dirname(HERE), "include", "pi05_b200.h")]
LIB = os.path.join(HERE, "libpi05_b200.so")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the engine has no prebuilt or CPU fallback")


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > built for p in SOURCES + HEADERS)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the engine into ``libpi05_b200.so`` next to this file; returns its path."""
    if not force and not stale():
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS, "-o", LIB, *SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force=True, verbose=True))
