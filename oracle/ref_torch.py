"""The reference's own torch recurrence on the host cores (TEST INFRASTRUCTURE: checker and reported CPU baseline).

``oracle/build_ref.py`` stages ``src/adkv/train/train_model.py`` of the reference, unchanged, under
``oracle/_ref/src``.  This module imports it from there and drives its ``_adkv_chunk_forward``
(``train_model.py:46-86``: quantise, dequantise and advance the state token by token) the way a CPU user of the
reference gets a decode-attention result: fake-quantise K and V from their initial state, then single-query
attention over the dequantised tensors in fp32.  The function is decorated with ``torch.compile``; it is run
eagerly here (the decorator is neutralised while the module is imported) because Inductor needs a host compiler
set-up that is not part of this project and would not be bit-faithful anyway.

Nothing in the product imports this file; ``bench.py`` uses it only in its baseline legs.
"""
from __future__ import annotations

import importlib
import math
import sys
import time

from . import build_ref

_tm = None


def available() -> bool:
    return build_ref.staged_src() is not None


def module():
    """The staged ``adkv.train.train_model``, imported once with ``torch.compile`` turned into a no-op."""
    global _tm
    if _tm is not None:
        return _tm
    src = build_ref.staged_src()
    if src is None:
        raise RuntimeError("oracle/_ref/src is not staged: run oracle/build_ref.py next to a reference checkout")
    import torch
    saved_compile = torch.compile
    saved_mods = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "adkv" or k.startswith("adkv.")}

    def eager(fn=None, **_kw):
        return fn if fn is not None else (lambda f: f)

    sys.path.insert(0, src)
    try:
        torch.compile = eager
        _tm = importlib.import_module("adkv.train.train_model")
    finally:
        torch.compile = saved_compile
        sys.path.remove(src)
        for k in [k for k in sys.modules if k == "adkv" or k.startswith("adkv.")]:
            del sys.modules[k]
        sys.modules.update(saved_mods)
    return _tm


def fake_quant(x, params, bits: int, scale_min: float, scale_max: float):
    """``x [B, H, T, D]`` (any float dtype) -> dequantised fp32 ``[B, H, T, D]`` by the reference's recurrence.
    ``params``: the five ``[H, D]`` tensors (zp_init, scale_init, alpha, beta, target)."""
    import torch
    B, H, T, D = x.shape
    C = H * D
    xs = x.float().permute(0, 2, 1, 3).reshape(B, T, C).contiguous()
    zp0, s0, alpha, beta, target = (p.float().reshape(C) for p in params)
    hi, lo = 2 ** (bits - 1) - 1, -2 ** (bits - 1)
    with torch.no_grad():
        out, *_ = module()._adkv_chunk_forward(xs, zp0.expand(B, -1).contiguous(), s0.expand(B, -1).contiguous(),
                                               alpha, beta, target, hi, lo, scale_min, scale_max, False)
    return out.reshape(B, T, H, D).permute(0, 2, 1, 3)


def decode_attention(q, k, v, k_params, v_params, bits: int, scaling: float,
                     scale_min: float = math.exp(-4.0), scale_max: float = math.exp(4.0)):
    """Single-query attention over the fake-quantised K / V.  ``q [B, Hq, 1, D]``, ``k`` / ``v [B, Hkv, T, D]``
    (every token, the newest included).  Returns fp32 ``[B, Hq, D]``."""
    import torch
    kh = fake_quant(k, k_params, bits, scale_min, scale_max)
    vh = fake_quant(v, v_params, bits, scale_min, scale_max)
    G = q.shape[1] // k.shape[1]
    if G > 1:
        kh, vh = kh.repeat_interleave(G, dim=1), vh.repeat_interleave(G, dim=1)
    w = torch.softmax(torch.einsum("bhd,bhtd->bht", q[:, :, 0].float(), kh) * scaling, dim=-1)
    return torch.einsum("bht,bhtd->bhd", w, vh)


def timed(fn, repeats: int = 3):
    """(best wall-clock seconds of ``repeats`` calls, last result)."""
    best, res = float("inf"), None
    for _ in range(repeats):
        t0 = time.perf_counter()
        res = fn()
        best = min(best, time.perf_counter() - t0)
    return best, res
