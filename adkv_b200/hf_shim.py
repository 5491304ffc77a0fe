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


def _reference_cuda_arithmetic():
    """A module with the three entry points bound to the arithmetic of the reference's CUDA kernels (fp16 state and
    accumulation, ``src/adkv/kernel/gemv.cu``): packed caches bit-identical to what the reference's own extension
    writes, which the fp32 recurrence of its torch code (this package's default) does not give."""
    from . import gemv
    mod = types.ModuleType("adkv.kernel.gemv")
    mod.__doc__ = "adkv_b200.gemv with half_state=True behind the reference's three entry points"

    def encode_kv(kv_cache, kv_new, kv_zp, kv_sc, kv_alpha, kv_beta, kv_t, scale_min, scale_max):
        return gemv.encode_kv(kv_cache, kv_new, kv_zp, kv_sc, kv_alpha, kv_beta, kv_t, scale_min, scale_max,
                              half_state=True)

    def forward_qk(q, k_cache, k_new, k_zp, k_sc, k_alpha, k_beta, k_t, T, scale_min, scale_max):
        return gemv.forward_qk(q, k_cache, k_new, k_zp, k_sc, k_alpha, k_beta, k_t, T, scale_min, scale_max,
                               half_state=True)

    def forward_ov(attn, v_cache, v_new, v_zp, v_sc, v_alpha, v_beta, v_t, scale_min, scale_max):
        return gemv.forward_ov(attn, v_cache, v_new, v_zp, v_sc, v_alpha, v_beta, v_t, scale_min, scale_max,
                               half_state=True)

    mod.encode_kv, mod.forward_qk, mod.forward_ov = encode_kv, forward_qk, forward_ov
    return mod


def install(force: bool = True, half_state: bool = False):
    """Register the kernels as ``adkv.kernel.gemv``; returns the registered module.

    ``half_state=False``: :mod:`adkv_b200.gemv` itself (fp32 recurrence in the order of the reference's torch code).
    ``half_state=True``: the same entry points in the arithmetic of the reference's CUDA kernels, for a deployment
    that has to reproduce, bit for bit, the caches its reference build wrote."""
    from . import gemv
    for name in ("adkv", "adkv.kernel"):
        if name not in sys.modules:
            try:
                importlib.import_module(name)          # the reference checkout, if it is on sys.path
            except Exception:
                pkg = types.ModuleType(name)
                pkg.__path__ = []                      # namespace stand-in when the reference is absent
                sys.modules[name] = pkg
    mod = _reference_cuda_arithmetic() if half_state else gemv
    if force or "adkv.kernel.gemv" not in sys.modules:
        sys.modules["adkv.kernel.gemv"] = mod
        setattr(sys.modules["adkv.kernel"], "gemv", mod)
    return sys.modules["adkv.kernel.gemv"]


def patch_mask_sizes(cache_layer_cls):
    """Accept an int or a tensor as ``cache_position`` in ``get_mask_sizes``."""
    def get_mask_sizes(self, cache_position):
        n = cache_position if isinstance(cache_position, int) else cache_position.shape[0]
        return self.get_seq_length() + n, 0
    cache_layer_cls.get_mask_sizes = get_mask_sizes
    return cache_layer_cls
