"""Loader of the reference's own CUDA extension built by ``build_ref.py`` (TEST INFRASTRUCTURE).

``module()`` returns the extension module (``forward_qk``, ``forward_ov``, ``encode_kv`` with the reference's
signatures, ``src/adkv/kernel/gemv.cpp:4-26``) or ``None`` when it has not been built.  The reference's
kernels always launch on the legacy default stream (``src/adkv/kernel/gemv.cu:321, 839, 1193``).
"""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "adkv_gemv.so")
_mod = None


def available() -> bool:
    return os.path.exists(PATH)


def module():
    global _mod
    if _mod is None and available():
        import torch  # noqa: F401  (libtorch must be loaded before the extension)
        loader = importlib.machinery.ExtensionFileLoader("adkv_gemv", PATH)
        spec = importlib.util.spec_from_loader("adkv_gemv", loader)
        _mod = importlib.util.module_from_spec(spec)
        loader.exec_module(_mod)
    return _mod
