"""CPU restatement of the arithmetic of the reference's CUDA kernels (TEST INFRASTRUCTURE, numpy).

The reference's ``gemv.cu`` keeps the recurrence in fp16 (``src/adkv/kernel/gemv.cu:150-164``), unlike its
torch / Triton path, which ``oracle/adkv_oracle.py`` restates.  Per channel, with every operation rounded
once to fp16:

    omt = 1 - beta * target          (ONE rounding: the reference's build contracts the multiply and the
                                      subtract of gemv.cu:221 into a fused multiply-add)
    q   = clamp(round_half_even((x - zp) / sc), QL, QU)     fp32 subtract and IEEE divide (gemv.cu:150-154);
                                                            NaN quotient -> 0 (float-to-int conversion)
    x^  = q * sc + zp                (gemv.cu:644-645)
    zp <- fma(alpha, q * sc, zp)     (gemv.cu:162)
    sc <- sc * fma(beta, |q|, omt)   (gemv.cu:163)           no eps guard, no clamp of the scale

fp16 operations are evaluated in float64 and rounded to float16 once, which is exact for a product or a
fused multiply-add of fp16 operands.  Packing, append slot and decode glue are those of
``oracle/adkv_oracle.py``.

Parity pin: checked on a B200 against the reference's own kernels compiled for sm_100a (``oracle/_ref``,
``tests/test_gpu_half_state.py``): codes, appended codes and final states bit for bit.
"""
from __future__ import annotations

import numpy as np

from . import adkv_oracle as orc

f16, f32, f64 = np.float16, np.float32, np.float64


def _r16(v):
    with np.errstate(over="ignore", invalid="ignore"):
        return np.asarray(v, dtype=f64).astype(f16)


class HalfState:
    """zp, sc float16 ``[B, H, D]``."""

    def __init__(self, zp, sc):
        self.zp, self.sc = zp.astype(f16).copy(), sc.astype(f16).copy()


def init_state(B, zp_init, scale_init) -> HalfState:
    H, D = zp_init.shape
    return HalfState(np.broadcast_to(zp_init.astype(f16), (B, H, D)), np.broadcast_to(scale_init.astype(f16), (B, H, D)))


def one_minus_bt(beta, target):
    return _r16(1.0 - beta.astype(f64) * target.astype(f64))


def quantize_token(x, st: HalfState, bits: int):
    """x fp16-valued ``[B,H,D]`` -> integer codes as float32 (gemv.cu:150-154)."""
    lo, hi = orc.quant_limits(bits)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        v = (x.astype(f32) - st.zp.astype(f32)) / st.sc.astype(f32)
        q = np.clip(np.rint(v), lo, hi)
    return np.where(np.isnan(v), f32(0), q).astype(f32)


def advance(q, st: HalfState, alpha, beta, omt):
    """gemv.cu:158-164."""
    with np.errstate(over="ignore", invalid="ignore"):
        qs = _r16(q.astype(f64) * st.sc.astype(f64))
        st.zp = _r16(alpha.astype(f64) * qs.astype(f64) + st.zp.astype(f64))
        g = _r16(beta.astype(f64) * np.abs(q).astype(f64) + omt.astype(f64))
        st.sc = _r16(st.sc.astype(f64) * g.astype(f64))


def dequant(q, st: HalfState):
    """gemv.cu:644-645: fp16 product, then fp16 sum."""
    with np.errstate(over="ignore", invalid="ignore"):
        return _r16(_r16(q.astype(f64) * st.sc.astype(f64)).astype(f64) + st.zp.astype(f64))


def encode_scan(x16, st: HalfState, alpha, beta, target, bits: int):
    """x16 ``[B,H,T,D]`` float16 -> codes int8 ``[B,H,T,D]``, x_hat float16; advances ``st``."""
    omt = one_minus_bt(beta.astype(f16), target.astype(f16))
    a16, b16 = alpha.astype(f16), beta.astype(f16)
    B, H, T, D = x16.shape
    codes = np.zeros((B, H, T, D), np.int8)
    xhat = np.zeros((B, H, T, D), f16)
    for t in range(T):
        q = quantize_token(x16[:, :, t], st, bits)
        codes[:, :, t] = q.astype(np.int8)
        xhat[:, :, t] = dequant(q, st)
        advance(q, st, a16, b16, omt)
    return codes, xhat


def decode_scan(codes, st: HalfState, alpha, beta, target):
    omt = one_minus_bt(beta.astype(f16), target.astype(f16))
    a16, b16 = alpha.astype(f16), beta.astype(f16)
    B, H, T, D = codes.shape
    xhat = np.zeros((B, H, T, D), f16)
    for t in range(T):
        q = codes[:, :, t].astype(f32)
        xhat[:, :, t] = dequant(q, st)
        advance(q, st, a16, b16, omt)
    return xhat


def encode_kv(cache, x16, params, bits: int = 4):
    """Prefill into a packed cache (in place); returns (cache, final state)."""
    zp0, s0, alpha, beta, target = params
    st = init_state(x16.shape[0], zp0, s0)
    codes, _ = encode_scan(x16, st, alpha, beta, target, bits)
    T = x16.shape[2]
    if T:
        ns = orc.n_super_for(T, bits)
        cache[:, :, :ns] = orc.pack_codes(codes, bits)[:, :, :ns]
    return cache, st


def decode_attn(q16, k_cache, v_cache, k_new, v_new, kparams, vparams, T: int, scaling: float, bits: int = 4,
                mask=None):
    """One decode step: replay both caches (tokens [0,T)), append the new token at T (in place), attention over
    T+1 tokens in float64.  q16 ``[B,Hq,D]``, k_new / v_new ``[B,Hkv,D]`` float16.  Returns ``[B,Hq,D]`` float32
    and the unscaled logits ``[B,Hq,T+1]``."""
    B, Hq, D = q16.shape
    Hkv = k_cache.shape[1]
    G = Hq // Hkv
    xs = []
    for cache, x_new, params in ((k_cache, k_new, kparams), (v_cache, v_new, vparams)):
        zp0, s0, alpha, beta, target = params
        st = init_state(B, zp0, s0)
        codes = orc.unpack_codes(cache, T, bits) if T else np.zeros((B, Hkv, 0, D), np.int8)
        xhat = decode_scan(codes, st, alpha, beta, target)
        qn = quantize_token(x_new, st, bits)
        with np.errstate(over="ignore", invalid="ignore"):
            xn = _r16(qn.astype(f64) * st.sc.astype(f64) + st.zp.astype(f64))       # fused (gemv.cu:796, 1155)
        orc.pack_codes(qn.astype(np.int8)[:, :, None, :], bits, out=cache, t_start=T)
        xs.append(np.concatenate([xhat, xn[:, :, None]], axis=2).astype(f64))
    kx, vx = xs
    qf = q16.astype(f64).reshape(B, Hkv, G, D)
    logits = np.einsum("bhgd,bhtd->bhgt", qf, kx)
    z = logits * scaling
    if mask is not None:
        z = z + np.asarray(mask, f64).reshape(B, 1, 1, T + 1)
    w = orc.softmax(z)
    out = np.einsum("bhgt,bhtd->bhgd", w, vx)
    return out.reshape(B, Hq, D).astype(f32), logits.reshape(B, Hq, T + 1)
