"""Seeded synthetic inputs with the shapes and value distribution of the benchmark configs.

The reference measures on real Llama activations with calibrated ADKV parameters;
neither weights, checkpoints nor datasets are available offline, so these generators
stand in for them: K/V ~ N(0,1) with 4 outlier channels per head scaled x20, then
RoPE (theta 10000, HF ``rotate_half`` convention), cast to fp16.  ADKV parameters:
per-channel EMA rate ``rho ~ U(0.90, 0.999)``, ``alpha = 1 - rho`` (the reference
weights the *new* sample with alpha, ``src/adkv/train/train_model.py:77``),
``beta = 0.05`` (= 0.1 * sigmoid(0), ``train_model.py:121,133-134``),
``target = QU / 2`` (``train_model.py:124``), ``zp_init = 0``, ``scale_init = 1``
(``train_model.py:112-115``), all rounded to fp16 as the HF model stores them
(``src/adkv/hf/llama_adkv.py:302-309``).
"""
from __future__ import annotations

import math

import torch

SCALE_MIN = math.exp(-4.0)   # src/adkv/hf/llama_adkv.py:23
SCALE_MAX = math.exp(4.0)    # src/adkv/hf/llama_adkv.py:24


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def rope(x: torch.Tensor, theta: float = 10000.0, pos0: int = 0) -> torch.Tensor:
    """Rotary embedding over ``[..., T, D]`` fp32, positions ``pos0 .. pos0+T-1``."""
    T, D = x.shape[-2], x.shape[-1]
    half = D // 2
    inv = theta ** (-torch.arange(0, half, device=x.device, dtype=torch.float32) * 2.0 / D)
    pos = torch.arange(pos0, pos0 + T, device=x.device, dtype=torch.float32)
    ang = pos[:, None] * inv[None, :]
    cos = torch.cat([ang.cos(), ang.cos()], dim=-1)
    sin = torch.cat([ang.sin(), ang.sin()], dim=-1)
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rot * sin


def gen_kv(seed: int, B: int, H: int, T: int, D: int, device="cpu",
           outlier_mode: str = "scale", n_outliers: int = 4, outlier_gain: float = 20.0,
           pos0: int = 0) -> torch.Tensor:
    """``[B, H, T, D]`` fp16 post-RoPE K or V with outlier channels.

    ``outlier_mode="scale"``: the chosen channels of the N(0,1) draw are multiplied
    by ``outlier_gain`` (the literal reading of the config).  ``"persistent"``: the
    outlier channels carry a token-constant N(0,1) offset times the gain plus N(0,1)
    noise, which after RoPE drifts sinusoidally."""
    g = _gen(seed, device)
    x = torch.randn(B, H, T, D, generator=g, device=device, dtype=torch.float32)
    gsel = _gen(seed + 7919, "cpu")
    for h in range(H):
        ch = torch.randperm(D, generator=gsel)[:n_outliers].to(device)
        if outlier_mode == "scale":
            x[:, h, :, ch] *= outlier_gain
        elif outlier_mode == "persistent":
            base = torch.randn(B, 1, n_outliers, generator=g, device=device, dtype=torch.float32)
            x[:, h, :, ch] += outlier_gain * base
        else:
            raise ValueError(f"unknown outlier_mode {outlier_mode!r}")
    return rope(x, pos0=pos0).to(torch.float16)


def gen_q(seed: int, B: int, Hq: int, D: int, device="cpu") -> torch.Tensor:
    """``[B, Hq, 1, D]`` fp16 query ~ N(0,1)."""
    g = _gen(seed, device)
    return torch.randn(B, Hq, 1, D, generator=g, device=device, dtype=torch.float32).to(torch.float16)


def gen_params(seed: int, H: int, D: int, bits: int = 4, device="cpu",
               rho_lo: float = 0.90, rho_hi: float = 0.999, beta: float = 0.05):
    """The five ``[H, D]`` fp16 ADKV parameter tensors (zp_init, scale_init, alpha, beta, target)."""
    g = _gen(seed, "cpu")
    rho = rho_lo + (rho_hi - rho_lo) * torch.rand(H, D, generator=g)
    qu = (1 << (bits - 1)) - 1
    p = (torch.zeros(H, D), torch.ones(H, D), 1.0 - rho,
         torch.full((H, D), beta), torch.full((H, D), qu / 2.0))
    return tuple(t.to(torch.float16).to(device).contiguous() for t in p)
