"""Make the reference's unmodified model file run on top of this package.

``src/adkv/hf/llama_adkv.py:21`` does ``from adkv.kernel.gemv import encode_kv, forward_ov, forward_qk``
and the reference's ``adkv/kernel/gemv.py`` JIT-compiles its own CUDA file at import.  ``install()``
registers :mod:`adkv_b200.gemv` under that module name *before* the reference model file is imported, so
the three names resolve to the B200 kernels and the reference's extension is never built.

``patch_mask_sizes(cls)`` lets the reference's cache class accept the ``int`` that newer transformers
releases pass to ``get_mask_sizes`` (``llama_adkv.py:76-80`` assumes a tensor).
"""
from __future__ import annotations

import importlib
import sys
import types


def install(force: bool = True):
    """Register adkv_b200.gemv as ``adkv.kernel.gemv``; returns the module."""
    from . import gemv
    for name in ("adkv", "adkv.kernel"):
        if name not in sys.modules:
            try:
                importlib.import_module(name)          # the reference checkout, if it is on sys.path
            except Exception:
                pkg = types.ModuleType(name)
                pkg.__path__ = []                      # namespace stand-in when the reference is absent
                sys.modules[name] = pkg
    if force or "adkv.kernel.gemv" not in sys.modules:
        sys.modules["adkv.kernel.gemv"] = gemv
        setattr(sys.modules["adkv.kernel"], "gemv", gemv)
    return gemv


def patch_mask_sizes(cache_layer_cls):
    """Accept an int or a tensor as ``cache_position`` in ``get_mask_sizes``."""
    def get_mask_sizes(self, cache_position):
        n = cache_position if isinstance(cache_position, int) else cache_position.shape[0]
        return self.get_seq_length() + n, 0
    cache_layer_cls.get_mask_sizes = get_mask_sizes
    return cache_layer_cls
