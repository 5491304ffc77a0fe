"""Build the reference's own CUDA extension for sm_100a into ``oracle/_ref/`` (TEST INFRASTRUCTURE).

    python oracle/build_ref.py /path/to/reference

The reference JIT-builds ``src/adkv/kernel/gemv.cpp`` + ``gemv.cu`` with
``torch.utils.cpp_extension.load(..., extra_cuda_cflags=["-O2"])`` (``src/adkv/kernel/gemv.py:8-13``).  This
recipe compiles the same two files, unmodified and where they lie in the reference checkout, with the
same preprocessor flags torch's loader passes, ``-O2`` and ``-gencode arch=compute_100a,code=sm_100a``,
straight with nvcc / g++ (the reference's own build path is not run).  Output: ``oracle/_ref/adkv_gemv.so``, a
Python extension module exporting ``forward_qk``, ``forward_ov``, ``encode_kv`` (``gemv.cpp:28-33``).  No
reference source is copied; the folder is git-ignored.

Used only by tests (to pin the packed layout and the append / self-token semantics by executing the
reference's kernels on the GPU) and by ``bench.py`` as a reported comparison.  The product never loads it.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "adkv_gemv.so")
NAME = "adkv_gemv"


def build(ref_root: str, force: bool = False, verbose: bool = False) -> str | None:
    """Returns the path of the built module, or None when the reference checkout is absent."""
    kdir = os.path.join(ref_root, "src", "adkv", "kernel")
    cu, cpp = os.path.join(kdir, "gemv.cu"), os.path.join(kdir, "gemv.cpp")
    if not (os.path.exists(cu) and os.path.exists(cpp)):
        return None
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(cu), os.path.getmtime(cpp)):
        return OUT
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT_DIR, exist_ok=True)
    inc = [f"-I{p}" for p in ce.include_paths("cuda")] + [f"-I{sysconfig.get_paths()['include']}"]
    defs = [f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    o_cu, o_cpp = os.path.join(OUT_DIR, "gemv_cu.o"), os.path.join(OUT_DIR, "gemv_cpp.o")
    cmds = [
        [nvcc, "-c", cu, "-o", o_cu, "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
         "--compiler-options", "-fPIC", *ce.COMMON_NVCC_FLAGS, *defs, *inc],
        ["g++", "-c", cpp, "-o", o_cpp, "-O2", "-std=c++17", "-fPIC", *defs, *inc],
        ["g++", "-shared", o_cu, o_cpp, "-o", OUT, *[f"-L{p}" for p in ce.library_paths("cuda")],
         "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"],
    ]
    for c in cmds:
        if verbose:
            print(" ".join(c), flush=True)
        subprocess.check_call(c)
    return OUT


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: build_ref.py /path/to/reference")
    print(build(sys.argv[1], force=True, verbose=True))
