"""Build the reference's own CUDA extension for sm_100a into ``oracle/_ref/`` (TEST INFRASTRUCTURE).

    python oracle/build_ref.py /path/to/reference

The reference JIT-builds ``src/adkv/kernel/gemv.cpp`` + ``gemv.cu`` with
``torch.utils.cpp_extension.load(..., extra_cuda_cflags=["-O2"])`` (``src/adkv/kernel/gemv.py:8-13``).  This
recipe compiles the same two files, unmodified and where they lie in the reference checkout, with the
same preprocessor flags torch's loader passes, ``-O2`` and ``-gencode arch=compute_100a,code=sm_100a``,
straight with nvcc / g++ (the reference's own build path is not run).  Output: ``oracle/_ref/adkv_gemv.so``, a
Python extension module exporting ``forward_qk``, ``forward_ov``, ``encode_kv`` (``gemv.cpp:28-33``).  No
reference source is copied; the folder is git-ignored.

The recipe also stages, byte for byte, the reference's Python files that the checkers execute -- its model
file ``src/adkv/hf/llama_adkv.py`` (the caller of the three entry points), its torch recurrence
``src/adkv/train/train_model.py`` (the CPU path) and the package ``__init__.py`` files above them -- into
``oracle/_ref/src/``.  Like the ``.so`` they are build outputs: git-ignored, never edited, and they travel with
the snapshot to the GPU box, where no reference checkout exists.  The reference's own ``adkv/kernel/gemv.py``
(which JIT-builds its extension at import) is deliberately not staged: tests register ``adkv_b200.gemv`` under
that module name instead (``adkv_b200.hf_shim``).

Used only by tests (to pin the packed layout and the append / self-token semantics by executing the
reference's kernels on the GPU, and to run the reference's unmodified model file on this library's kernels)
and by ``bench.py`` as reported comparisons (the reference's CUDA kernels, its torch CPU path).  The product
never loads any of it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "adkv_gemv.so")
NAME = "adkv_gemv"
SRC_DIR = os.path.join(OUT_DIR, "src")
# files executed by the checkers, relative to <reference>/src
STAGED = ("adkv/__init__.py", "adkv/kernel/__init__.py", "adkv/hf/llama_adkv.py", "adkv/train/__init__.py",
          "adkv/train/train_model.py")


# The reference's kernel module, kept as TEXT for the signature comparison of tests/test_boundary.py.  It is given a
# name Python cannot import: importing it would JIT-build the reference's extension.
KERNEL_MODULE_TEXT = os.path.join(OUT_DIR, "reference_kernel_module_gemv.py.txt")


def stage_python(ref_root: str) -> str | None:
    """Copy the STAGED files, unchanged, to oracle/_ref/src/.  Returns that folder, or None without a checkout."""
    src = os.path.join(ref_root, "src")
    if not os.path.exists(os.path.join(src, "adkv", "hf", "llama_adkv.py")):
        return None
    for rel in STAGED:
        a, b = os.path.join(src, rel), os.path.join(SRC_DIR, rel)
        if not os.path.exists(a):          # a package without __init__.py stays a namespace package
            continue
        os.makedirs(os.path.dirname(b), exist_ok=True)
        shutil.copyfile(a, b)
    shutil.copyfile(os.path.join(src, "adkv", "kernel", "gemv.py"), KERNEL_MODULE_TEXT)
    return SRC_DIR


def staged_src() -> str | None:
    """The folder to put on sys.path to import the staged files as ``adkv.*``, if they have been staged."""
    return SRC_DIR if os.path.exists(os.path.join(SRC_DIR, "adkv", "hf", "llama_adkv.py")) else None


def build(ref_root: str, force: bool = False, verbose: bool = False) -> str | None:
    """Returns the path of the built module, or None when the reference checkout is absent."""
    kdir = os.path.join(ref_root, "src", "adkv", "kernel")
    cu, cpp = os.path.join(kdir, "gemv.cu"), os.path.join(kdir, "gemv.cpp")
    if not (os.path.exists(cu) and os.path.exists(cpp)):
        return None
    stage_python(ref_root)
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
