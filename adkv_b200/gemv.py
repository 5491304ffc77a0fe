"""Host-side mirror of the reference's kernel module ``adkv.kernel.gemv``.

``encode_kv``, ``forward_qk`` and ``forward_ov`` keep the reference's names, positional
arguments, in-place semantics and error behaviour (``src/adkv/kernel/gemv.py:16-132``; argument
checks of ``src/adkv/kernel/gemv.cu:375-398, 892-912, 1241-1266``), so the reference's model file
``src/adkv/hf/llama_adkv.py`` runs on top of this module unchanged (see ``adkv_b200.hf_shim``).
They call hand-written sm_100a kernels through the C ABI of ``libadkv_b200.so`` on the current
torch CUDA stream.  Keyword-only extensions: ``bits`` (4 or 2), ``fast`` (contracted replay), ``half_state`` (the
fp16-state arithmetic of the reference's CUDA kernels instead of the fp32 recurrence: bit-compatible caches),
grouped-query heads (``q`` may have a multiple of the cache's heads).

``decode_attn`` is the fused decode step (q.K^T, scaling, mask, softmax, P.V and both appends in one
launch) that replaces the three-call sequence of ``src/adkv/hf/llama_adkv.py:263-276``.
``append_kv`` appends one token from a persisted tail state without replaying the cache.

Arithmetic is the reference's fp32 torch/Triton recurrence
(``src/adkv/train/train_model.py:70-81``), not the fp16 arithmetic of the reference's CUDA file;
``scale_min`` / ``scale_max`` are honoured.
"""
from __future__ import annotations

import collections
import ctypes

import torch

from . import _lib

__all__ = ["encode_kv", "forward_qk", "forward_ov", "decode_attn", "append_kv", "encode_kv_pair",
           "append_kv_pair", "n_super_for", "alloc_ckpt", "ckpt_capacity", "decode_scratch_bytes",
           "decode_attn_varlen", "decode_attn_static", "encode_kv_layers", "append_kv_layers", "LayerSet"]


def n_super_for(tokens: int, bits: int = 4) -> int:
    """Supergroups (words per channel) that hold ``tokens`` tokens."""
    tpw = 32 // bits
    return (tokens + tpw - 1) // tpw


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(t: torch.Tensor) -> ctypes.c_void_p:
    """The caller's current CUDA stream on the tensor's device, as the C ABI takes it."""
    if _raw_stream is not None:     # the handle itself, without building a torch.cuda.Stream object per call
        return ctypes.c_void_p(_raw_stream(t.device.index))
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


class _on_device:
    """``torch.cuda.device(dev)`` that costs nothing when ``dev`` is already current (the usual case)."""
    __slots__ = ("ctx",)

    def __init__(self, dev: torch.device):
        self.ctx = None if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        return False


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


# Parameter tensors are the same five buffers call after call (one set per layer and tensor): the checked
# ``adkv_params`` struct is remembered per set of device addresses.  An entry holds five integers and a small ctypes
# struct, never a tensor, so nothing is kept alive; a buffer that is freed and whose address is later reused by another
# tensor of the same dtype and size yields the very same struct, which is then just as right.  Least recently used
# entries are dropped one at a time.
_PARAM_CACHE: "collections.OrderedDict" = collections.OrderedDict()
_PARAM_CACHE_MAX = 512


def _params(names, tensors, H, D, device):
    """(adkv_params struct, tensors that must outlive the call) for five [H, D] float16 parameter tensors."""
    if all(t.is_contiguous() for t in tensors):
        key = (H, D, device, tuple((t.data_ptr(), t.dtype, t.numel(), t.device) for t in tensors))
        hit = _PARAM_CACHE.get(key)
        if hit is not None:
            _PARAM_CACHE.move_to_end(key)
            return hit, tensors
    else:
        key = None
    for n, t in zip(names, tensors):
        _require(t.dtype == torch.float16, f"{n} must be float16")
        _require(t.is_cuda and t.device == device, f"{n} must be on the cache's CUDA device")
        _require(t.numel() == H * D, f"{n} must have {H} x {D} elements")
    keep = [t.contiguous() for t in tensors]
    p = _lib.Params(*[t.data_ptr() for t in keep])
    if key is not None:
        _PARAM_CACHE[key] = p
        if len(_PARAM_CACHE) > _PARAM_CACHE_MAX:
            _PARAM_CACHE.popitem(last=False)
    return p, keep


def _cache_dims(cache: torch.Tensor, name: str):
    _require(cache.dtype == torch.uint8, f"{name} must be uint8")
    _require(cache.is_cuda, f"{name} must be a CUDA tensor (adkv_b200 has no CPU path)")
    _require(cache.dim() == 6 and cache.shape[4] == 4 and cache.shape[5] == 4,
             f"{name} must be [B, nh, n_super_cap, DIM/4, 4, 4]")
    return cache.shape[0], cache.shape[1], cache.shape[2], cache.shape[3] * 4


def encode_kv(kv_cache, kv_new, kv_zp, kv_sc, kv_alpha, kv_beta, kv_t, scale_min, scale_max, *,
              bits: int = 4, tail: torch.Tensor | None = None, t_start: int = 0, half_state: bool = False):
    """Prefill: quantise tokens ``[t_start, t_start+T)`` into the packed cache, in place.

    Same contract as the reference's ``encode_kv`` (``src/adkv/kernel/gemv.py:100-132``) for
    ``t_start == 0``.  ``tail`` (float32 ``[B, nh, 2, DIM]``) optionally receives the state after the
    last token and, for ``t_start > 0``, supplies the state to continue from.  ``half_state`` selects the
    arithmetic of the reference's CUDA kernels (fp16 state: codes equal to theirs bit for bit) instead of the
    fp32 definition.  Returns ``kv_cache``."""
    _require(kv_new.dtype == torch.float16, "kv_new must be float16")
    B, H, n_super_cap, D = _cache_dims(kv_cache, "kv_cache")
    _require(kv_cache.is_contiguous(), "kv_cache must be contiguous (written in place)")
    _require(kv_new.dim() == 4, "kv_new must be [B, nh, T, DIM]")
    _require(kv_new.shape[3] == D, "kv_cache channel groups do not match kv_new head dim")
    _require(kv_new.shape[0] == B and kv_new.shape[1] == H, "kv_new batch/heads do not match kv_cache")
    T = kv_new.shape[2]
    need = n_super_for(t_start + T, bits)
    _require(need <= n_super_cap,
             f"kv_cache capacity too small: need {need} supergroups for {t_start + T} tokens, have {n_super_cap}")
    p, keep = _params(("kv_zp", "kv_sc", "kv_alpha", "kv_beta", "kv_t"),
                      (kv_zp, kv_sc, kv_alpha, kv_beta, kv_t), H, D, kv_cache.device)
    x = kv_new.contiguous()
    if tail is not None:
        _require(tail.dtype == torch.float32 and tail.is_contiguous() and tail.shape == (B, H, 2, D),
                 "tail must be contiguous float32 [B, nh, 2, DIM]")
    with _on_device(kv_cache.device):
        if half_state:
            rc = _lib.load().adkv_encode_kv_flags(kv_cache.data_ptr(), x.data_ptr(), ctypes.addressof(p),
                                                  None if tail is None else tail.data_ptr(), None, None, None, None,
                                                  None, None, 0, 0, B, H, T, D, n_super_cap, bits, t_start, scale_min,
                                                  scale_max, _lib.FLAG_HALF_STATE, _stream(kv_cache))
        else:
            rc = _lib.load().adkv_encode(kv_cache.data_ptr(), x.data_ptr(), ctypes.addressof(p),
                                         None if tail is None else tail.data_ptr(), B, H, T, D, n_super_cap, bits,
                                         t_start, scale_min, scale_max, _stream(kv_cache))
    _lib.check(rc, "encode_kv")
    return kv_cache


def ckpt_capacity(tokens: int, interval: int) -> int:
    """Checkpoints a cache of ``tokens`` tokens can reach (entry k = state before token (k+1)*interval)."""
    return tokens // interval


def alloc_ckpt(B: int, H: int, D: int, capacity_tokens: int, interval: int, device) -> torch.Tensor:
    """Checkpoint tensor ``[B, H, n_ckpt_cap, 2, D]`` float32 for caches of up to ``capacity_tokens`` tokens."""
    return torch.zeros((B, H, max(1, ckpt_capacity(capacity_tokens, interval)), 2, D), dtype=torch.float32,
                       device=device)


def _ckpt_args(k_ckpt, v_ckpt, interval, B, H, D):
    _require(k_ckpt is not None and v_ckpt is not None, "both checkpoint tensors are needed")
    _require(interval > 0 and interval % 32 == 0, "checkpoint interval must be a positive multiple of 32")
    for c in (k_ckpt, v_ckpt):
        _require(c.dtype == torch.float32 and c.is_contiguous() and c.dim() == 5 and c.shape[0] == B and
                 c.shape[1] == H and c.shape[3] == 2 and c.shape[4] == D and c.shape[2] == k_ckpt.shape[2],
                 "checkpoints must be contiguous float32 [B, nh, n_ckpt_cap, 2, DIM]")
    return k_ckpt.data_ptr(), v_ckpt.data_ptr(), interval, k_ckpt.shape[2]


def _tail_ptr(tail, B, H, D):
    if tail is None:
        return None
    _require(tail.dtype == torch.float32 and tail.is_contiguous() and tail.shape == (B, H, 2, D),
             "tail must be contiguous float32 [B, nh, 2, DIM]")
    return tail.data_ptr()


def encode_kv_pair(k_cache, k_new, k_params, v_cache, v_new, v_params, scale_min, scale_max, *, bits: int = 4,
                   k_tail=None, v_tail=None, t_start: int = 0, k_ckpt=None, v_ckpt=None, ckpt_interval: int = 0,
                   half_state: bool = False):
    """``encode_kv`` for the K and V tensors of one layer in a single launch (same contract each;
    replaces the two calls of ``src/adkv/hf/llama_adkv.py:144-153``).  With ``k_ckpt`` / ``v_ckpt`` /
    ``ckpt_interval`` every state checkpoint reached is written as well (see :func:`alloc_ckpt`)."""
    _require(k_new.dtype == torch.float16 and v_new.dtype == torch.float16, "kv_new must be float16")
    B, H, n_super_cap, D = _cache_dims(k_cache, "kv_cache")
    _require(tuple(v_cache.shape) == tuple(k_cache.shape) and v_cache.dtype == torch.uint8 and v_cache.is_cuda,
             "v_cache must match k_cache")
    _require(k_cache.is_contiguous() and v_cache.is_contiguous(), "kv_cache must be contiguous (written in place)")
    _require(k_new.dim() == 4 and k_new.shape == v_new.shape, "k_new / v_new must both be [B, nh, T, DIM]")
    _require(k_new.shape[0] == B and k_new.shape[1] == H and k_new.shape[3] == D,
             "kv_cache channel groups do not match kv_new head dim")
    T = k_new.shape[2]
    need = n_super_for(t_start + T, bits)
    _require(need <= n_super_cap,
             f"kv_cache capacity too small: need {need} supergroups for {t_start + T} tokens, have {n_super_cap}")
    names = ("kv_zp", "kv_sc", "kv_alpha", "kv_beta", "kv_t")
    kp, keep_k = _params(names, tuple(k_params), H, D, k_cache.device)
    vp, keep_v = _params(names, tuple(v_params), H, D, k_cache.device)
    xk, xv = k_new.contiguous(), v_new.contiguous()
    with _on_device(k_cache.device):
        if half_state:
            kc, vc, iv, cap = _ckpt_args(k_ckpt, v_ckpt, ckpt_interval, B, H, D) if ckpt_interval else (None, None, 0, 0)
            rc = _lib.load().adkv_encode_kv_flags(k_cache.data_ptr(), xk.data_ptr(), ctypes.addressof(kp),
                                                  _tail_ptr(k_tail, B, H, D), kc, v_cache.data_ptr(), xv.data_ptr(),
                                                  ctypes.addressof(vp), _tail_ptr(v_tail, B, H, D), vc, iv, cap, B, H, T,
                                                  D, n_super_cap, bits, t_start, scale_min, scale_max,
                                                  _lib.FLAG_HALF_STATE, _stream(k_cache))
        elif ckpt_interval:
            kc, vc, iv, cap = _ckpt_args(k_ckpt, v_ckpt, ckpt_interval, B, H, D)
            rc = _lib.load().adkv_encode_kv_ckpt(k_cache.data_ptr(), xk.data_ptr(), ctypes.addressof(kp),
                                                 _tail_ptr(k_tail, B, H, D), kc, v_cache.data_ptr(), xv.data_ptr(),
                                                 ctypes.addressof(vp), _tail_ptr(v_tail, B, H, D), vc, iv, cap,
                                                 B, H, T, D, n_super_cap, bits, t_start, scale_min, scale_max,
                                                 _stream(k_cache))
        else:
            rc = _lib.load().adkv_encode_kv(k_cache.data_ptr(), xk.data_ptr(), ctypes.addressof(kp),
                                            _tail_ptr(k_tail, B, H, D), v_cache.data_ptr(), xv.data_ptr(),
                                            ctypes.addressof(vp), _tail_ptr(v_tail, B, H, D), B, H, T, D,
                                            n_super_cap, bits, t_start, scale_min, scale_max, _stream(k_cache))
    _lib.check(rc, "encode_kv_pair")
    return k_cache, v_cache


def append_kv_pair(k_cache, k_new, k_params, k_tail, v_cache, v_new, v_params, v_tail, T: int, scale_min, scale_max,
                   *, bits: int = 4, k_ckpt=None, v_ckpt=None, ckpt_interval: int = 0, half_state: bool = False):
    """``append_kv`` for K and V of one layer in a single launch (optionally maintaining state checkpoints)."""
    B, H, n_super_cap, D = _cache_dims(k_cache, "cache")
    _require(tuple(v_cache.shape) == tuple(k_cache.shape) and v_cache.dtype == torch.uint8 and v_cache.is_cuda,
             "v_cache must match k_cache")
    _require(k_cache.is_contiguous() and v_cache.is_contiguous(), "cache must be contiguous (appended in place)")
    _require(k_new.dtype == torch.float16 and v_new.dtype == torch.float16, "x_new must be float16")
    _require(k_new.numel() == B * H * D and v_new.numel() == B * H * D, "x_new must be [B, nh, 1, DIM]")
    _require(T >= 0, "T must be non-negative")
    _require(T // (32 // bits) < n_super_cap, f"cache has no free supergroup to append token {T}")
    _require(k_tail is not None and v_tail is not None, "append needs both tail states")
    names = ("zp", "sc", "alpha", "beta", "target")
    kp, keep_k = _params(names, tuple(k_params), H, D, k_cache.device)
    vp, keep_v = _params(names, tuple(v_params), H, D, k_cache.device)
    xk, xv = k_new.contiguous(), v_new.contiguous()
    with _on_device(k_cache.device):
        if half_state:
            kc, vc, iv, cap = _ckpt_args(k_ckpt, v_ckpt, ckpt_interval, B, H, D) if ckpt_interval else (None, None, 0, 0)
            rc = _lib.load().adkv_append_kv_flags(k_cache.data_ptr(), xk.data_ptr(), ctypes.addressof(kp),
                                                  _tail_ptr(k_tail, B, H, D), kc, v_cache.data_ptr(), xv.data_ptr(),
                                                  ctypes.addressof(vp), _tail_ptr(v_tail, B, H, D), vc, iv, cap, B, H, T,
                                                  D, n_super_cap, bits, scale_min, scale_max, _lib.FLAG_HALF_STATE,
                                                  _stream(k_cache))
        elif ckpt_interval:
            kc, vc, iv, cap = _ckpt_args(k_ckpt, v_ckpt, ckpt_interval, B, H, D)
            rc = _lib.load().adkv_append_kv_ckpt(k_cache.data_ptr(), xk.data_ptr(), ctypes.addressof(kp),
                                                 _tail_ptr(k_tail, B, H, D), kc, v_cache.data_ptr(), xv.data_ptr(),
                                                 ctypes.addressof(vp), _tail_ptr(v_tail, B, H, D), vc, iv, cap,
                                                 B, H, T, D, n_super_cap, bits, scale_min, scale_max,
                                                 _stream(k_cache))
        else:
            rc = _lib.load().adkv_append_kv(k_cache.data_ptr(), xk.data_ptr(), ctypes.addressof(kp),
                                            _tail_ptr(k_tail, B, H, D), v_cache.data_ptr(), xv.data_ptr(),
                                            ctypes.addressof(vp), _tail_ptr(v_tail, B, H, D), B, H, T, D,
                                            n_super_cap, bits, scale_min, scale_max, _stream(k_cache))
    _lib.check(rc, "append_kv_pair")
    return k_cache, v_cache


class LayerSet:
    """The packed caches, parameters and tail states of several layers, bound once for the layered calls.

    ``layers``: one tuple ``(k_cache, k_params, k_tail, v_cache, v_params, v_tail)`` per layer; all layers share
    shapes.  Building the descriptor array (argument checks, pointer extraction) is what a per-layer call pays
    on every step; a ``LayerSet`` pays it once, and :func:`encode_kv_layers` / :func:`append_kv_layers` then only
    fill in the pointers of the new tokens.  The caches and tails must stay the tensors they were bound with."""

    def __init__(self, layers, bits: int = 4):
        layers = list(layers)
        _require(len(layers) > 0, "a LayerSet needs at least one layer")
        kc0 = layers[0][0]
        self.B, self.H, self.n_super_cap, self.D = _cache_dims(kc0, "k_cache")
        self.bits, self.device, self.n = bits, kc0.device, len(layers)
        self._keep = []
        self.desc = (_lib.LayerKV * self.n)()
        names = ("zp", "sc", "alpha", "beta", "target")
        for i, (kc, kps, kt, vc, vps, vt) in enumerate(layers):
            for c in (kc, vc):
                _require(tuple(c.shape) == tuple(kc0.shape) and c.dtype == torch.uint8 and c.is_cuda and c.is_contiguous()
                         and c.device == self.device, "every cache of a LayerSet must be a contiguous uint8 tensor of one shape")
            kp, keep_k = _params(names, tuple(kps), self.H, self.D, self.device)
            vp, keep_v = _params(names, tuple(vps), self.H, self.D, self.device)
            d = self.desc[i]
            d.k_cache, d.v_cache = kc.data_ptr(), vc.data_ptr()
            d.kp, d.vp = kp, vp
            d.k_tail, d.v_tail = _tail_ptr(kt, self.B, self.H, self.D), _tail_ptr(vt, self.B, self.H, self.D)
            self._keep.append((kc, vc, kt, vt, keep_k, keep_v))

    def _bind_new(self, k_new, v_new, tokens_dims):
        """Point the descriptors at the new tokens: two lists of per-layer tensors, or two stacked tensors
        ``[n_layers, B, H, ...]``."""
        _require(len(k_new) == self.n and len(v_new) == self.n, "one K and one V tensor per layer")
        keep = []
        for i in range(self.n):
            for x in (k_new[i], v_new[i]):
                _require(x.dtype == torch.float16 and x.is_cuda, "new tokens must be float16 CUDA tensors")
            xk, xv = k_new[i].contiguous(), v_new[i].contiguous()
            _require(xk.numel() == tokens_dims and xv.numel() == tokens_dims, "new tokens have the wrong shape")
            self.desc[i].k, self.desc[i].v = xk.data_ptr(), xv.data_ptr()
            keep.append((xk, xv))
        return keep


def encode_kv_layers(layer_set: LayerSet, k_new, v_new, scale_min, scale_max, *, t_start: int = 0):
    """:func:`encode_kv_pair` for every layer of ``layer_set`` in as few launches as possible (K and V of 8 layers
    each).  ``k_new`` / ``v_new``: per layer ``[B, nh, T, DIM]`` float16 (lists, or tensors stacked along a leading
    layer axis).  For callers that hold the fp16 K/V of many layers at once."""
    ls = layer_set
    T = k_new[0].shape[2]
    need = n_super_for(t_start + T, ls.bits)
    _require(need <= ls.n_super_cap, f"kv_cache capacity too small: need {need} supergroups, have {ls.n_super_cap}")
    keep = ls._bind_new(k_new, v_new, ls.B * ls.H * T * ls.D)
    with _on_device(ls.device):
        rc = _lib.load().adkv_encode_kv_layers(ctypes.addressof(ls.desc), ls.n, ls.B, ls.H, T, ls.D, ls.n_super_cap,
                                               ls.bits, t_start, scale_min, scale_max,
                                               ctypes.c_void_p(_raw_stream(ls.device.index)) if _raw_stream else
                                               ctypes.c_void_p(torch.cuda.current_stream(ls.device).cuda_stream))
    _lib.check(rc, "encode_kv_layers")
    del keep


def append_kv_layers(layer_set: LayerSet, k_new, v_new, T: int, scale_min, scale_max):
    """:func:`append_kv_pair` for every layer of ``layer_set``: token ``T`` of every layer is quantised from that
    layer's tail states, which advance.  ``k_new`` / ``v_new``: per layer ``[B, nh, 1, DIM]`` float16 (lists or a
    tensor stacked along a leading layer axis, e.g. one ``[n_layers, B, nh, DIM]`` buffer the layers wrote into)."""
    ls = layer_set
    _require(T >= 0 and T // (32 // ls.bits) < ls.n_super_cap, f"cache has no free supergroup to append token {T}")
    _require(all(ls.desc[i].k_tail and ls.desc[i].v_tail for i in range(ls.n)), "append needs the tail states")
    keep = ls._bind_new(k_new, v_new, ls.B * ls.H * ls.D)
    with _on_device(ls.device):
        rc = _lib.load().adkv_append_kv_layers(ctypes.addressof(ls.desc), ls.n, ls.B, ls.H, T, ls.D, ls.n_super_cap,
                                               ls.bits, scale_min, scale_max,
                                               ctypes.c_void_p(_raw_stream(ls.device.index)) if _raw_stream else
                                               ctypes.c_void_p(torch.cuda.current_stream(ls.device).cuda_stream))
    _lib.check(rc, "append_kv_layers")
    del keep


def append_kv(cache, x_new, zp, sc, alpha, beta, target, tail, T: int, scale_min, scale_max, *, bits: int = 4,
              half_state: bool = False):
    """Quantise ``x_new [B, nh, 1, DIM]`` with the persisted ``tail`` state (after token ``T-1``),
    write it as token ``T`` and advance ``tail`` in place.  Returns ``cache``."""
    B, H, n_super_cap, D = _cache_dims(cache, "cache")
    _require(cache.is_contiguous(), "cache must be contiguous (appended in place)")
    _require(x_new.dtype == torch.float16, "x_new must be float16")
    _require(x_new.numel() == B * H * D, "x_new must be [B, nh, 1, DIM]")
    _require(T >= 0, "T must be non-negative")
    _require(T // (32 // bits) < n_super_cap, f"cache has no free supergroup to append token {T}")
    _require(tail.dtype == torch.float32 and tail.is_contiguous() and tail.shape == (B, H, 2, D),
             "tail must be contiguous float32 [B, nh, 2, DIM]")
    p, keep = _params(("zp", "sc", "alpha", "beta", "target"), (zp, sc, alpha, beta, target), H, D, cache.device)
    x = x_new.contiguous()
    with _on_device(cache.device):
        if half_state:
            rc = _lib.load().adkv_append_kv_flags(cache.data_ptr(), x.data_ptr(), ctypes.addressof(p), tail.data_ptr(),
                                                  None, None, None, None, None, None, 0, 0, B, H, T, D, n_super_cap,
                                                  bits, scale_min, scale_max, _lib.FLAG_HALF_STATE, _stream(cache))
        else:
            rc = _lib.load().adkv_append(cache.data_ptr(), x.data_ptr(), ctypes.addressof(p), tail.data_ptr(),
                                         B, H, T, D, n_super_cap, bits, scale_min, scale_max, _stream(cache))
    _lib.check(rc, "append_kv")
    return cache


def forward_qk(q, k_cache, k_new, k_zp, k_sc, k_alpha, k_beta, k_t, T: int, scale_min, scale_max, *,
               bits: int = 4, fast: bool = False, half_state: bool = False):
    """Decode-phase q.K^T over the packed cache; appends ``k_new`` as token ``T`` in place.

    Same contract as the reference's ``forward_qk`` (``src/adkv/kernel/gemv.py:16-55``): returns
    ``[B, nh_q, T + 1]`` float16 unscaled logits whose last entry is the logit of the appended token
    computed from its dequantised code."""
    _require(q.dtype == torch.float16, "q must be float16")
    _require(k_new.dtype == torch.float16, "k_new must be float16")
    B, Hkv, n_super_cap, D = _cache_dims(k_cache, "k_cache")
    _require(k_cache.is_contiguous(), "k_cache must be contiguous (appended in place)")
    _require(q.dim() == 4 and q.shape[2] == 1, "q must be [B, nh, 1, DIM]")
    _require(D == q.shape[3], "q head dimension does not match k_cache")
    _require(q.shape[0] == B, "q batch does not match k_cache")
    Hq = q.shape[1]
    _require(Hq % Hkv == 0, "q heads must be a multiple of the cache's heads")
    _require(k_new.numel() == B * Hkv * D, "k_new must be [B, nh, 1, DIM]")
    _require(T >= 0, "T must be non-negative")
    _require(T // (32 // bits) < n_super_cap, f"k_cache has no free supergroup to append token {T}")
    p, keep = _params(("k_zp", "k_sc", "k_alpha", "k_beta", "k_t"), (k_zp, k_sc, k_alpha, k_beta, k_t),
                      Hkv, D, k_cache.device)
    qc, kn = q.contiguous(), k_new.contiguous()
    o = torch.empty((B, Hq, T + 1), dtype=torch.float16, device=k_cache.device)
    with _on_device(k_cache.device):
        rc = _lib.load().adkv_forward_qk(qc.data_ptr(), k_cache.data_ptr(), kn.data_ptr(), ctypes.addressof(p),
                                         o.data_ptr(), B, Hq, Hkv, T, D, n_super_cap, bits, scale_min, scale_max,
                                         _lib.flags(fast, half_state), _stream(k_cache))
    _lib.check(rc, "forward_qk")
    return o


def forward_ov(attn, v_cache, v_new, v_zp, v_sc, v_alpha, v_beta, v_t, scale_min, scale_max, *,
               bits: int = 4, fast: bool = False, half_state: bool = False):
    """Decode-phase P.V over the packed cache; appends ``v_new`` as token ``T = attn.shape[2] - 1``.

    Same contract as the reference's ``forward_ov`` (``src/adkv/kernel/gemv.py:58-97``): returns
    ``[B, nh_q, DIM]`` float16; the last weight multiplies the dequantised appended token."""
    _require(attn.dtype == torch.float16, "attn must be float16")
    _require(v_new.dtype == torch.float16, "v_new must be float16")
    B, Hkv, n_super_cap, D = _cache_dims(v_cache, "v_cache")
    _require(v_cache.is_contiguous(), "v_cache must be contiguous (appended in place)")
    _require(attn.dim() == 3 and attn.shape[0] == B, "attn must be [B, nh, T + 1]")
    _require(attn.shape[2] >= 1, "attn must contain the cached weights plus the self weight")
    Hq = attn.shape[1]
    _require(Hq % Hkv == 0, "attn heads must be a multiple of the cache's heads")
    T = attn.shape[2] - 1
    _require(D == v_new.shape[-1], "v_new head dimension does not match v_cache")
    _require(v_new.numel() == B * Hkv * D, "v_new must be [B, nh, 1, DIM]")
    _require(T // (32 // bits) < n_super_cap, f"v_cache has no free supergroup to append token {T}")
    p, keep = _params(("v_zp", "v_sc", "v_alpha", "v_beta", "v_t"), (v_zp, v_sc, v_alpha, v_beta, v_t),
                      Hkv, D, v_cache.device)
    ac, vn = attn.contiguous(), v_new.contiguous()
    o = torch.empty((B, Hq, D), dtype=torch.float16, device=v_cache.device)
    with _on_device(v_cache.device):
        rc = _lib.load().adkv_forward_ov(ac.data_ptr(), v_cache.data_ptr(), vn.data_ptr(), ctypes.addressof(p),
                                         o.data_ptr(), B, Hq, Hkv, T, D, n_super_cap, bits, scale_min, scale_max,
                                         _lib.flags(fast, half_state), _stream(v_cache))
    _lib.check(rc, "forward_ov")
    return o


def decode_scratch_bytes(B: int, Hq: int, Hkv: int, T: int, interval: int) -> int:
    """Scratch bytes the checkpointed decode step needs for a cache of ``T`` tokens."""
    n = _lib.load().adkv_decode_attn_ckpt_scratch_bytes(B, Hq, Hkv, T, interval)
    _lib.check(min(n, 0), "decode_scratch_bytes")
    return n


def _tails(k_tail, v_tail, B, H, D, half_state):
    """Device pointers of the two tail states of a decode step (both or neither)."""
    _require((k_tail is None) == (v_tail is None), "k_tail and v_tail go together")
    _require(k_tail is None or not half_state, "tail states are for the fp32 arithmetic (half_state replays exactly)")
    return _tail_ptr(k_tail, B, H, D), _tail_ptr(v_tail, B, H, D)


def _fast_default(fast, k_tail) -> bool:
    """Contracted replay unless the caller says otherwise, as soon as a tail state keeps the stored codes exact."""
    return (k_tail is not None) if fast is None else bool(fast)


def decode_attn(q, k_cache, v_cache, k_new, v_new, k_params, v_params, T: int, scaling: float,
                scale_min, scale_max, *, mask: torch.Tensor | None = None, bits: int = 4, fast: bool | None = None,
                half_state: bool = False, out: torch.Tensor | None = None, k_ckpt=None, v_ckpt=None,
                ckpt_interval: int = 0, scratch: torch.Tensor | None = None, k_tail: torch.Tensor | None = None,
                v_tail: torch.Tensor | None = None, tail_keep: bool = False, split_channels: bool | None = None):
    """Fused decode step over both packed caches.

    ``q [B, nh_q, 1, DIM]``, ``k_new`` / ``v_new [B, nh_kv, 1, DIM]`` float16; ``k_params`` / ``v_params``
    the five ``[nh_kv, DIM]`` float16 tensors (zp_init, scale_init, alpha, beta, target); ``mask`` an
    additive ``[B, T+1]`` (or ``[B, 1, T+1]`` / ``[B, 1, 1, T+1]``) tensor shared by all heads.  Appends to
    both caches in place as token ``T`` and returns ``softmax(q.K^T * scaling + mask) . V`` as
    ``[B, nh_q, DIM]`` float16, the appended token included (``src/adkv/hf/llama_adkv.py:263-276``).

    ``k_tail`` / ``v_tail`` (float32 ``[B, nh_kv, 2, DIM]``, as written by :func:`encode_kv_pair` /
    :func:`append_kv_pair` or left by the previous step): the recurrence state after token ``T-1``.  The reference
    has no such state and quantises the new token with what its replay ends in (``src/adkv/kernel/gemv.cu:744-764``);
    with the tails the new token is quantised from them -- bit-identical to the encoder -- and they advance to the
    state after token ``T`` (``tail_keep=True``: left untouched, so that the same step can be repeated).  The replay
    then only feeds the attention sums, and ``fast`` defaults to True (False without tails).

    With state checkpoints (``k_ckpt``, ``v_ckpt``, ``ckpt_interval``; see :func:`alloc_ckpt`) the token axis is
    processed in independent segments; ``scratch`` (uint8/any dtype, at least :func:`decode_scratch_bytes`) is
    allocated per call when not given.

    ``split_channels``: None lets the library choose between one warp per tensor and stream and a head split
    over two warp pairs (launches with few streams); True / False force one (head dim 128, fp32 arithmetic,
    no checkpoints)."""
    _require(q.dtype == torch.float16, "q must be float16")
    _require(k_new.dtype == torch.float16 and v_new.dtype == torch.float16, "k_new / v_new must be float16")
    B, Hkv, n_super_cap, D = _cache_dims(k_cache, "k_cache")
    _require(tuple(v_cache.shape) == tuple(k_cache.shape) and v_cache.dtype == torch.uint8 and v_cache.is_cuda,
             "v_cache must match k_cache")
    _require(k_cache.is_contiguous() and v_cache.is_contiguous(), "caches must be contiguous (appended in place)")
    _require(q.dim() == 4 and q.shape[2] == 1 and q.shape[0] == B and q.shape[3] == D, "q must be [B, nh, 1, DIM]")
    Hq = q.shape[1]
    _require(Hq % Hkv == 0, "q heads must be a multiple of the cache's heads")
    _require(k_new.numel() == B * Hkv * D and v_new.numel() == B * Hkv * D, "k_new / v_new must be [B, nh, 1, DIM]")
    _require(T >= 0, "T must be non-negative")
    _require(T // (32 // bits) < n_super_cap, f"cache has no free supergroup to append token {T}")
    names = ("zp", "sc", "alpha", "beta", "t")
    kp, keep_k = _params(tuple("k_" + n for n in names), tuple(k_params), Hkv, D, k_cache.device)
    vp, keep_v = _params(tuple("v_" + n for n in names), tuple(v_params), Hkv, D, k_cache.device)
    qc, kn, vn = q.contiguous(), k_new.contiguous(), v_new.contiguous()
    mptr, mstride, mk = None, 0, None
    if mask is not None:
        _require(mask.shape[0] == B and mask.shape[-1] == T + 1 and mask.numel() == B * (T + 1),
                 "mask must be [B, T + 1], shared by all heads")
        mk = mask.reshape(B, T + 1).to(device=k_cache.device, dtype=torch.float32).contiguous()
        mptr, mstride = mk.data_ptr(), T + 1
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.float16, device=k_cache.device)
    else:
        _require(out.dtype == torch.float16 and out.is_contiguous() and out.shape == (B, Hq, D),
                 "out must be contiguous float16 [B, nh_q, DIM]")
    kt, vt = _tails(k_tail, v_tail, B, Hkv, D, half_state)
    flags = _lib.flags(_fast_default(fast, k_tail), half_state, tail_keep, split_channels)
    with _on_device(k_cache.device):
        if ckpt_interval:
            kc, vc, iv, cap = _ckpt_args(k_ckpt, v_ckpt, ckpt_interval, B, Hkv, D)
            need = decode_scratch_bytes(B, Hq, Hkv, T, iv)
            if scratch is None:
                scratch = torch.empty(need, dtype=torch.uint8, device=k_cache.device)
            _require(scratch.is_cuda and scratch.is_contiguous(), "scratch must be a contiguous CUDA tensor")
            rc = _lib.load().adkv_decode_attn_ckpt(qc.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                                   kn.data_ptr(), vn.data_ptr(), ctypes.addressof(kp),
                                                   ctypes.addressof(vp), kt, vt, kc, vc, iv, cap, mptr, mstride,
                                                   out.data_ptr(), scratch.data_ptr(),
                                                   scratch.numel() * scratch.element_size(), B, Hq, Hkv, T, D,
                                                   n_super_cap, bits, scaling, scale_min, scale_max, flags,
                                                   _stream(k_cache))
        else:
            rc = _lib.load().adkv_decode_attn(qc.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), kn.data_ptr(),
                                              vn.data_ptr(), ctypes.addressof(kp), ctypes.addressof(vp), kt, vt, mptr,
                                              mstride, out.data_ptr(), B, Hq, Hkv, T, D, n_super_cap, bits, scaling,
                                              scale_min, scale_max, flags, _stream(k_cache))
    _lib.check(rc, "decode_attn")
    return out


def decode_attn_varlen(q, k_cache, v_cache, k_new, v_new, k_params, v_params, seq_lens, scaling: float,
                       scale_min, scale_max, *, bits: int = 4, fast: bool | None = None, half_state: bool = False,
                       out: torch.Tensor | None = None, k_tail: torch.Tensor | None = None,
                       v_tail: torch.Tensor | None = None, tail_keep: bool = False):
    """Fused decode step with per-sequence lengths on the device.

    ``seq_lens`` int32 ``[B]`` CUDA tensor: sequence ``b`` attends over its ``seq_lens[b]`` cached tokens and
    appends the new token at that position (the caller advances ``seq_lens`` afterwards, on the device).
    Otherwise as :func:`decode_attn` without a mask (tail states included).  Nothing in the call depends on the lengths' values, so
    the same launch can be replayed step after step (e.g. from a captured CUDA graph)."""
    _require(q.dtype == torch.float16, "q must be float16")
    _require(k_new.dtype == torch.float16 and v_new.dtype == torch.float16, "k_new / v_new must be float16")
    B, Hkv, n_super_cap, D = _cache_dims(k_cache, "k_cache")
    _require(tuple(v_cache.shape) == tuple(k_cache.shape) and v_cache.dtype == torch.uint8 and v_cache.is_cuda,
             "v_cache must match k_cache")
    _require(k_cache.is_contiguous() and v_cache.is_contiguous(), "caches must be contiguous (appended in place)")
    _require(q.dim() == 4 and q.shape[2] == 1 and q.shape[0] == B and q.shape[3] == D, "q must be [B, nh, 1, DIM]")
    Hq = q.shape[1]
    _require(Hq % Hkv == 0, "q heads must be a multiple of the cache's heads")
    _require(k_new.numel() == B * Hkv * D and v_new.numel() == B * Hkv * D, "k_new / v_new must be [B, nh, 1, DIM]")
    _require(seq_lens.dtype == torch.int32 and seq_lens.is_cuda and seq_lens.is_contiguous() and seq_lens.numel() == B,
             "seq_lens must be a contiguous int32 CUDA tensor with one entry per sequence")
    names = ("zp", "sc", "alpha", "beta", "t")
    kp, keep_k = _params(tuple("k_" + n for n in names), tuple(k_params), Hkv, D, k_cache.device)
    vp, keep_v = _params(tuple("v_" + n for n in names), tuple(v_params), Hkv, D, k_cache.device)
    qc, kn, vn = q.contiguous(), k_new.contiguous(), v_new.contiguous()
    if out is None:
        out = torch.empty((B, Hq, D), dtype=torch.float16, device=k_cache.device)
    else:
        _require(out.dtype == torch.float16 and out.is_contiguous() and out.shape == (B, Hq, D),
                 "out must be contiguous float16 [B, nh_q, DIM]")
    kt, vt = _tails(k_tail, v_tail, B, Hkv, D, half_state)
    with _on_device(k_cache.device):
        rc = _lib.load().adkv_decode_attn_varlen(qc.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), kn.data_ptr(),
                                                 vn.data_ptr(), ctypes.addressof(kp), ctypes.addressof(vp), kt, vt,
                                                 seq_lens.data_ptr(), out.data_ptr(), B, Hq, Hkv, D, n_super_cap,
                                                 bits, scaling, scale_min, scale_max,
                                                 _lib.flags(_fast_default(fast, k_tail), half_state, tail_keep),
                                                 _stream(k_cache))
    _lib.check(rc, "decode_attn_varlen")
    return out


STATIC_SCRATCH_BYTES = 16 << 20


def decode_attn_static(q, k_cache, v_cache, k_new, v_new, k_params, v_params, T: int, scaling: float,
                       scale_min, scale_max, *, k_ckpt, v_ckpt, ckpt_interval: int, out: torch.Tensor,
                       mask: torch.Tensor | None = None, bits: int = 4, fast: bool | None = None,
                       half_state: bool = False, k_tail: torch.Tensor | None = None,
                       v_tail: torch.Tensor | None = None, tail_keep: bool = False):
    """The checkpointed decode step for a caller that must not allocate device memory.

    Same arguments and result as ``decode_attn(..., k_ckpt=, v_ckpt=, ckpt_interval=)``, except that ``out``
    is required (nothing is allocated here either) and the partial results go to a 16 MiB array built into the
    library instead of a scratch tensor.  Use it when the process has no device memory left to give -- all of
    HBM already belongs to a block pool -- or no allocator to call.  ``decode_scratch_bytes(...)`` must not
    exceed ``STATIC_SCRATCH_BYTES``, otherwise a ``RuntimeError`` names the limit.  The array is shared by
    every call on the device and keeps the previous call's contents (harmless: each call overwrites what it
    reads), so calls that could run concurrently on the GPU must be serialised by the caller.  The first call
    on a device also looks up the array's address; issue it before starting any stream capture.

    Inputs must already be contiguous float16 / float32 tensors on the cache's device (no copies are made);
    ``mask``, if given, a contiguous float32 ``[B, T+1]`` tensor."""
    B, Hkv, n_super_cap, D = _cache_dims(k_cache, "k_cache")
    Hq = q.shape[1]
    for name, t, dt in (("q", q, torch.float16), ("k_new", k_new, torch.float16), ("v_new", v_new, torch.float16),
                        ("out", out, torch.float16)):
        _require(t.dtype == dt and t.is_cuda and t.is_contiguous(), f"{name} must be a contiguous CUDA {dt} tensor")
    _require(tuple(v_cache.shape) == tuple(k_cache.shape) and v_cache.dtype == torch.uint8 and v_cache.is_cuda and
             k_cache.is_contiguous() and v_cache.is_contiguous(), "caches must be matching contiguous uint8 tensors")
    _require(q.numel() == B * Hq * D and out.numel() == B * Hq * D and Hq % Hkv == 0, "q / out must be [B, nh_q, DIM]")
    _require(k_new.numel() == B * Hkv * D and v_new.numel() == B * Hkv * D, "k_new / v_new must be [B, nh, 1, DIM]")
    _require(T >= 0 and T // (32 // bits) < n_super_cap, f"cache has no free supergroup to append token {T}")
    for name, ps in (("k", k_params), ("v", v_params)):
        for t in ps:
            _require(t.dtype == torch.float16 and t.is_cuda and t.is_contiguous() and t.numel() == Hkv * D,
                     f"{name} parameters must be contiguous float16 [nh, DIM] CUDA tensors")
    kp = _lib.Params(*[t.data_ptr() for t in k_params])
    vp = _lib.Params(*[t.data_ptr() for t in v_params])
    kc, vc, iv, cap = _ckpt_args(k_ckpt, v_ckpt, ckpt_interval, B, Hkv, D)
    mptr, mstride = None, 0
    if mask is not None:
        _require(mask.dtype == torch.float32 and mask.is_cuda and mask.is_contiguous() and
                 tuple(mask.shape) == (B, T + 1), "mask must be a contiguous float32 [B, T + 1] CUDA tensor")
        mptr, mstride = mask.data_ptr(), T + 1
    kt, vt = _tails(k_tail, v_tail, B, Hkv, D, half_state)
    with _on_device(k_cache.device):
        rc = _lib.load().adkv_decode_attn_ckpt_static(
            q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), k_new.data_ptr(), v_new.data_ptr(),
            ctypes.addressof(kp), ctypes.addressof(vp), kt, vt, kc, vc, iv, cap, mptr, mstride, out.data_ptr(),
            B, Hq, Hkv, T, D, n_super_cap, bits, scaling, scale_min, scale_max,
            _lib.flags(_fast_default(fast, k_tail), half_state, tail_keep), _stream(k_cache))
    _lib.check(rc, "decode_attn_static")
    return out


def device_status(device=None) -> int:
    """Read and clear the device status word (non-zero: a kernel gave up on a bounded wait)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    val = ctypes.c_int(0)
    with _on_device(dev):
        rc = _lib.load().adkv_device_status(ctypes.byref(val),
                                            ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _lib.check(rc, "device_status")
    return val.value
