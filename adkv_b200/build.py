"""Build the C-ABI shared library ``adkv_b200/lib/libadkv_b200.so`` for sm_100a with nvcc.

The library has no dependency on torch or Python: plain ``extern "C"`` entry points declared in
``include/adkv_b200.h``.  It is built in-tree so that it travels with the source snapshot.
"""
from __future__ import annotations

import os
import shutil
from concurrent.futures import ThreadPoolExecutor
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libadkv_b200.so")
SOURCES = ["adkv_capi.cu", "adkv_encode.cu", "adkv_fused.cu", "adkv_unfused.cu", "adkv_split.cu", "adkv_wide.cu",
           "adkv_half.cu", "adkv_narrow.cu"]
HEADERS = ["adkv_device.cuh", "adkv_decode.cuh", "adkv_softmax.cuh", "adkv_half.cuh", "adkv_io.cuh", "adkv_host.h",
           "adkv_narrow.cuh",
           os.path.join("..", "..", "include", "adkv_b200.h")]
OBJ_DIR = os.path.join(PKG, "build")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libadkv_b200.so")
    return exe


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra: list[str] | None = None) -> str:
    if not force and not is_stale():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + (extra or []) + ["-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        return obj

    # the translation units are independent: compile them side by side, then link
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        objs = list(pool.map(compile_one, SOURCES))
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a"] + objs + ["-o", LIB]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.check_call(link)
    return LIB


if __name__ == "__main__":
    build(force=True, verbose=True, extra=["-Xptxas", "-v"] if "-v" in sys.argv else None)
