"""CPU restatement of the ADKV hot path (TEST INFRASTRUCTURE, not product code).

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
reference arm may import this module, and only as the checker.  The product
package never imports it.

What is restated, and from where in the reference project:

* the fp32 recurrence (zero point / scale tracking, quantise, dequantise):
  ``src/adkv/train/train_model.py:6-22`` (``IntQuantSTE.forward``) and
  ``src/adkv/train/train_model.py:70-81`` (the loop body of
  ``_adkv_chunk_forward``); the Triton evaluation kernel evaluates the same
  operations in the same order (``src/adkv/hf/llama_adkv_eval.py:87-97``).
* the packed 4-bit cache layout: ``src/adkv/kernel/gemv.cu:266-305`` (writer)
  and ``src/adkv/kernel/gemv.cu:502-510`` (diagram).  The 2-bit layout has no
  counterpart in the reference; it is defined here (16 tokens per 32-bit word,
  code stored as ``q + 2``) and keeps the same tile shape.
* decode-step semantics (append with the state left by token ``T-1``, self
  logit / self value from the *dequantised* new token, ``T + 1`` weights):
  ``src/adkv/kernel/gemv.cu:744-814`` and ``:1105-1159``; the glue between the
  two GEMVs (scaling, additive mask, fp32 softmax):
  ``src/adkv/hf/llama_adkv.py:263-276``.

Parity pin: the reference ships no golden vectors or tests.  The recurrence
here is pinned against outputs of the reference's own torch code executed on
CPU (``tests/golden/make_golden.py`` imports it and writes the fixtures that
``tests/test_oracle_golden.py`` checks).  Layout and decode semantics have no
executable CPU counterpart in the reference and follow the cited lines.

All arithmetic on the recurrence is numpy float32, one IEEE operation per
numpy call, so no fused multiply-add can be introduced.
"""
from __future__ import annotations

import math

import numpy as np

F32 = np.float32
EPS = F32(1e-8)                      # train_model.py:9
SCALE_MIN = math.exp(-4.0)           # llama_adkv.py:23
SCALE_MAX = math.exp(4.0)            # llama_adkv.py:24


def quant_limits(bits: int) -> tuple[int, int]:
    """(lower, upper) code limits: train_model.py:96-97."""
    return -(1 << (bits - 1)), (1 << (bits - 1)) - 1


def tokens_per_word(bits: int) -> int:
    return 32 // bits


def n_super_for(tokens: int, bits: int = 4) -> int:
    """Supergroups (one 32-bit word per channel) needed for ``tokens`` tokens.

    4-bit: llama_adkv.py:83-85 (8 tokens per supergroup)."""
    tpw = tokens_per_word(bits)
    return (tokens + tpw - 1) // tpw


class State:
    """Per-(batch, head, channel) running zero point and scale, float32."""

    def __init__(self, zp: np.ndarray, s: np.ndarray):
        self.zp = np.ascontiguousarray(zp, dtype=F32)
        self.s = np.ascontiguousarray(s, dtype=F32)

    def copy(self) -> "State":
        return State(self.zp.copy(), self.s.copy())


def init_state(B: int, zp_init: np.ndarray, scale_init: np.ndarray) -> State:
    """Broadcast the ``[H, D]`` initial values over the batch (train_model.py:163-164)."""
    H, D = zp_init.shape
    zp = np.broadcast_to(zp_init.astype(F32), (B, H, D)).copy()
    s = np.broadcast_to(scale_init.astype(F32), (B, H, D)).copy()
    return State(zp, s)


def quantize_token(x: np.ndarray, st: State, bits: int) -> tuple[np.ndarray, np.ndarray]:
    """Codes and dequantised residual of one token against the current state.

    train_model.py:72 and :8-17.  ``x`` is ``[B, H, D]`` float32."""
    lo, hi = quant_limits(bits)
    residual = x - st.zp
    sc_safe = np.maximum(st.s, EPS)
    q = np.clip(np.rint(residual / sc_safe), F32(lo), F32(hi)).astype(F32)
    residual_hat = q * sc_safe
    return q, residual_hat


def advance_state(q: np.ndarray, residual_hat: np.ndarray, st: State,
                  alpha: np.ndarray, beta: np.ndarray, target: np.ndarray,
                  scale_min: float, scale_max: float) -> None:
    """State update from the code alone (train_model.py:77-81), in place."""
    st.zp = st.zp + alpha * residual_hat
    error = np.abs(q) - target
    st.s = np.clip(st.s + st.s * beta * error, F32(scale_min), F32(scale_max)).astype(F32)


def dequant_step(q: np.ndarray, st: State, alpha, beta, target, scale_min, scale_max) -> np.ndarray:
    """Decoder side of one token: rebuild x_hat from the code and advance."""
    sc_safe = np.maximum(st.s, EPS)
    residual_hat = q * sc_safe
    x_hat = residual_hat + st.zp                       # train_model.py:74
    advance_state(q, residual_hat, st, alpha, beta, target, scale_min, scale_max)
    return x_hat


def encode_scan(x: np.ndarray, st: State, alpha, beta, target, bits: int,
                scale_min: float = SCALE_MIN, scale_max: float = SCALE_MAX,
                want_xhat: bool = True):
    """Quantise ``x [B, H, T, D]`` token by token starting from ``st`` (advanced in place).

    Returns ``(codes int8 [B,H,T,D], x_hat float32 [B,H,T,D] or None)``."""
    x = np.asarray(x, dtype=F32)
    B, H, T, D = x.shape
    alpha = alpha.astype(F32); beta = beta.astype(F32); target = target.astype(F32)
    codes = np.empty((B, H, T, D), dtype=np.int8)
    xhat = np.empty((B, H, T, D), dtype=F32) if want_xhat else None
    for t in range(T):
        q, rh = quantize_token(x[:, :, t, :], st, bits)
        codes[:, :, t, :] = q.astype(np.int8)
        if want_xhat:
            xhat[:, :, t, :] = rh + st.zp
        advance_state(q, rh, st, alpha, beta, target, scale_min, scale_max)
    return codes, xhat


def decode_scan(codes: np.ndarray, st: State, alpha, beta, target,
                scale_min: float = SCALE_MIN, scale_max: float = SCALE_MAX) -> np.ndarray:
    """Replay ``codes [B,H,T,D]`` from ``st`` (advanced in place); returns x_hat float32."""
    B, H, T, D = codes.shape
    alpha = alpha.astype(F32); beta = beta.astype(F32); target = target.astype(F32)
    xhat = np.empty((B, H, T, D), dtype=F32)
    for t in range(T):
        q = codes[:, :, t, :].astype(F32)
        xhat[:, :, t, :] = dequant_step(q, st, alpha, beta, target, scale_min, scale_max)
    return xhat


# --------------------------------------------------------------------------- layout


def cache_shape(B: int, H: int, n_super: int, D: int) -> tuple[int, ...]:
    """llama_adkv.py:87-94."""
    return (B, H, n_super, D // 4, 4, 4)


def cache_words(cache: np.ndarray) -> np.ndarray:
    """View the uint8 tile ``[B,H,ns,D/4,4,4]`` as little-endian words ``[B,H,ns,D]``.

    Word ``(sg, c)`` holds the codes of channel ``c`` for the tokens of supergroup
    ``sg``: channel ``4*cg + ch`` is 32-bit lane ``ch`` of the 16-byte vector
    ``cg`` and byte ``br`` of it is bits ``8*br .. 8*br+7`` (gemv.cu:266-305)."""
    B, H, ns, ncg, four, four2 = cache.shape
    assert four == 4 and four2 == 4 and cache.dtype == np.uint8
    return np.ascontiguousarray(cache).view("<u4").reshape(B, H, ns, ncg * 4)


def pack_codes(codes: np.ndarray, bits: int, n_super_cap: int | None = None,
               out: np.ndarray | None = None, t_start: int = 0) -> np.ndarray:
    """Pack ``codes int8 [B,H,T,D]`` for tokens ``t_start .. t_start+T-1``.

    Token ``t`` of a channel sits in word ``t // tpw`` at bit ``bits * (t % tpw)``
    as ``code - lower_limit`` (4-bit: nibble ``q + 8``, even token = low nibble
    of byte ``(t % 8) // 2``, gemv.cu:266-295).  With ``out`` given, only the bit
    fields of the packed tokens are replaced (the append's read-modify-write,
    gemv.cu:100-145); otherwise a zero-filled tile is created."""
    B, H, T, D = codes.shape
    lo, _ = quant_limits(bits)
    tpw = tokens_per_word(bits)
    need = n_super_for(t_start + T, bits)
    if out is None:
        ns = need if n_super_cap is None else n_super_cap
        out = np.zeros(cache_shape(B, H, ns, D), dtype=np.uint8)
    assert out.shape[2] >= need, "cache capacity too small"
    words = cache_words(out).copy()
    field = np.uint32((1 << bits) - 1)
    for t in range(T):
        tt = t_start + t
        sg, j = divmod(tt, tpw)
        sh = np.uint32(bits * j)
        val = (codes[:, :, t, :].astype(np.int32) - lo).astype(np.uint32) & field
        words[:, :, sg, :] = (words[:, :, sg, :] & ~(field << sh)) | (val << sh)
    out[...] = words.view(np.uint8).reshape(out.shape)
    return out


def unpack_codes(cache: np.ndarray, T: int, bits: int) -> np.ndarray:
    """Inverse of :func:`pack_codes` for tokens ``0 .. T-1`` -> int8 ``[B,H,T,D]``."""
    lo, _ = quant_limits(bits)
    tpw = tokens_per_word(bits)
    words = cache_words(cache)
    B, H, ns, D = words.shape
    codes = np.empty((B, H, T, D), dtype=np.int8)
    field = np.uint32((1 << bits) - 1)
    for t in range(T):
        sg, j = divmod(t, tpw)
        codes[:, :, t, :] = (((words[:, :, sg, :] >> np.uint32(bits * j)) & field).astype(np.int32) + lo).astype(np.int8)
    return codes


# --------------------------------------------------------------------------- entry points


def _params32(p):
    return tuple(np.asarray(a, dtype=F32) for a in p)


def encode_kv(cache: np.ndarray, x: np.ndarray, params, bits: int = 4,
              scale_min: float = SCALE_MIN, scale_max: float = SCALE_MAX):
    """Oracle of ``encode_kv`` (gemv.cu:368-414 semantics, fp32 arithmetic).

    ``x [B,H,T,D]`` (fp16 values), ``params`` = (zp_init, scale_init, alpha, beta,
    target), each ``[H,D]``.  Overwrites supergroups ``0 .. ceil(T/tpw)-1`` of
    ``cache`` (unused fields of the last one are zero, gemv.cu:243, 300-305).
    Returns ``(cache, tail_state)``."""
    zp0, s0, alpha, beta, target = _params32(params)
    x = np.asarray(x, dtype=F32)
    B, H, T, D = x.shape
    st = init_state(B, zp0, s0)
    codes, _ = encode_scan(x, st, alpha, beta, target, bits, scale_min, scale_max, want_xhat=False)
    need = n_super_for(T, bits)
    fresh = pack_codes(codes, bits, n_super_cap=need)
    cache[:, :, :need] = fresh
    return cache, st


def replay(cache: np.ndarray, T: int, params, bits: int,
           scale_min: float = SCALE_MIN, scale_max: float = SCALE_MAX):
    """Dequantise tokens ``0..T-1`` of a packed cache; returns ``(x_hat, state after T-1)``."""
    zp0, s0, alpha, beta, target = _params32(params)
    B = cache.shape[0]
    st = init_state(B, zp0, s0)
    codes = unpack_codes(cache, T, bits)
    xhat = decode_scan(codes, st, alpha, beta, target, scale_min, scale_max)
    return xhat, st


def append_token(cache: np.ndarray, x_new: np.ndarray, st: State, T: int, params, bits: int,
                 scale_min: float = SCALE_MIN, scale_max: float = SCALE_MAX) -> np.ndarray:
    """Quantise ``x_new [B,H,D]`` with ``st`` (state after token ``T-1``), write it as
    token ``T`` (gemv.cu:744-764), advance ``st`` and return the dequantised token."""
    _, _, alpha, beta, target = _params32(params)
    x_new = np.asarray(x_new, dtype=F32)
    q, rh = quantize_token(x_new, st, bits)
    x_hat = rh + st.zp
    pack_codes(q.astype(np.int8)[:, :, None, :], bits, out=cache, t_start=T)
    advance_state(q, rh, st, alpha, beta, target, scale_min, scale_max)
    return x_hat


def forward_qk(q: np.ndarray, k_cache: np.ndarray, k_new: np.ndarray, params, T: int,
               bits: int = 4, scale_min: float = SCALE_MIN, scale_max: float = SCALE_MAX) -> np.ndarray:
    """Oracle of ``forward_qk`` (gemv.cu:883-939): unscaled logits ``[B,Hq,T+1]`` float64.

    ``q [B,Hq,D]``, ``k_new [B,Hkv,D]``; q head ``h`` reads KV head ``h // (Hq/Hkv)``.
    Appends ``k_new`` in place as token ``T``; the last logit uses the dequantised
    new token (gemv.cu:766-814)."""
    q = np.asarray(q, dtype=F32)
    B, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    G = Hq // Hkv
    khat, st = replay(k_cache, T, params, bits, scale_min, scale_max)
    knew_hat = append_token(k_cache, k_new, st, T, params, bits, scale_min, scale_max)
    kall = np.concatenate([khat, knew_hat[:, :, None, :]], axis=2).astype(np.float64)  # [B,Hkv,T+1,D]
    kall = np.repeat(kall, G, axis=1)
    return np.einsum("bhd,bhtd->bht", q.astype(np.float64), kall)


def forward_ov(attn: np.ndarray, v_cache: np.ndarray, v_new: np.ndarray, params,
               bits: int = 4, scale_min: float = SCALE_MIN, scale_max: float = SCALE_MAX) -> np.ndarray:
    """Oracle of ``forward_ov`` (gemv.cu:1233-1288): ``[B,Hq,D]`` float64.

    ``attn [B,Hq,T+1]``; appends ``v_new`` in place as token ``T``."""
    attn = np.asarray(attn, dtype=np.float64)
    B, Hq, Tp1 = attn.shape
    T = Tp1 - 1
    Hkv = v_cache.shape[1]
    G = Hq // Hkv
    vhat, st = replay(v_cache, T, params, bits, scale_min, scale_max)
    vnew_hat = append_token(v_cache, v_new, st, T, params, bits, scale_min, scale_max)
    vall = np.concatenate([vhat, vnew_hat[:, :, None, :]], axis=2).astype(np.float64)
    vall = np.repeat(vall, G, axis=1)
    return np.einsum("bht,bhtd->bhd", attn, vall)


def softmax(x: np.ndarray) -> np.ndarray:
    m = x.max(axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    e = np.exp(x - m)
    return e / e.sum(axis=-1, keepdims=True)


def decode_attn(q, k_cache, v_cache, k_new, v_new, k_params, v_params, T: int, scaling: float,
                mask: np.ndarray | None = None, bits: int = 4,
                scale_min: float = SCALE_MIN, scale_max: float = SCALE_MAX) -> np.ndarray:
    """One decode step as the caller composes it (llama_adkv.py:263-276), without the
    intermediate fp16 roundings: logits * scaling (+ mask ``[B,1|Hq,T+1]``), softmax,
    weighted sum of dequantised values.  Appends to both caches.  ``[B,Hq,D]`` float64."""
    logits = forward_qk(q, k_cache, k_new, k_params, T, bits, scale_min, scale_max) * float(scaling)
    if mask is not None:
        logits = logits + np.asarray(mask, dtype=np.float64)
    w = softmax(logits)
    return forward_ov(w, v_cache, v_new, v_params, bits, scale_min, scale_max)


def dense_attn(q, k, v, scaling: float) -> np.ndarray:
    """Unquantised single-query attention over ``k, v [B,H,T,D]`` (config-1 comparison)."""
    logits = np.einsum("bhd,bhtd->bht", q.astype(np.float64), k.astype(np.float64)) * scaling
    return np.einsum("bht,bhtd->bhd", softmax(logits), v.astype(np.float64))
