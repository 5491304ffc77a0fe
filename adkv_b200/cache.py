"""Per-layer packed KV cache: host-side mirror of the reference's ``KVCacheLayer_ADKV``.

Same state machine, method names, argument order and errors as
``src/adkv/hf/llama_adkv.py:44-276`` (allocate on first use, grow in 64-token steps, prefill only
from token 0, decode one token at a time), on top of the B200 kernels.  Differences, all opt-in:

* ``capacity_tokens``: pre-size the buffers once instead of reallocating and copying every 64
  tokens (the reference's growth is O(T^2) bytes over a generation, ``llama_adkv.py:104-123``);
* ``fused=True`` (default): one ``decode_attn`` launch replaces ``forward_qk`` -> torch softmax ->
  ``forward_ov`` (``llama_adkv.py:263-276``); the attention weights are then not materialised and
  ``decode`` returns ``None`` in their place.  ``fused=False`` reproduces the reference's sequence;
* grouped-query attention (more query heads than KV heads), which the reference rejects
  (``llama_adkv.py:235-238``);
* ``bits`` = 4 (reference layout) or 2;
* ``half_state=True``: the fp16-state arithmetic of the reference's own CUDA kernels (``src/adkv/kernel/gemv.cu:150-164``)
  instead of the fp32 definition, so that the buffers can be exchanged with caches those kernels wrote;
* ``checkpoint_interval`` (with ``capacity_tokens``): keep recurrence-state checkpoints every that many tokens
  and decode with one warp pair per segment instead of one per sequence (long contexts, small batches).
"""
from __future__ import annotations

import torch

from . import gemv
from .synth import SCALE_MAX, SCALE_MIN

INIT_SEQ_LEN = 64   # src/adkv/hf/llama_adkv.py:40
CAP_LEN = 64        # src/adkv/hf/llama_adkv.py:41


class KVCacheLayer:
    def __init__(self, bits: int = 4, fused: bool = True, fast: bool = False, capacity_tokens: int | None = None,
                 checkpoint_interval: int = 0, half_state: bool = False):
        if bits not in (2, 4):
            raise ValueError("bits must be 2 or 4")
        if checkpoint_interval and (not capacity_tokens or not fused or checkpoint_interval % 32):
            raise ValueError("checkpoints need a fused cache with capacity_tokens and an interval that is a multiple of 32")
        self.bits, self.fused, self.fast, self.half_state = bits, fused, fast, half_state
        self._ckpt_interval = checkpoint_interval
        self._kck = self._vck = None
        self._tpw = 32 // bits
        self._capacity_tokens = capacity_tokens
        self._key_buf = None
        self._value_buf = None
        self._quant_len = 0
        self._cap_len = 0
        self._B = self._H = self._C = 0
        self._device = None

    # ------------------------------------------------------------------ bookkeeping
    def get_seq_length(self) -> int:
        return self._quant_len

    def get_mask_sizes(self, cache_position) -> tuple[int, int]:
        query_length = cache_position if isinstance(cache_position, int) else cache_position.shape[0]
        return self.get_seq_length() + query_length, 0

    @property
    def key_states(self):
        return self._key_buf

    @property
    def value_states(self):
        return self._value_buf

    def _n_super(self, tokens: int) -> int:
        return (tokens + self._tpw - 1) // self._tpw

    def _alloc(self, cap_tokens: int):
        n_super = self._n_super(cap_tokens)
        self._cap_len = n_super * self._tpw
        shape = (self._B, self._H, n_super, self._C // 4, 4, 4)
        self._key_buf = torch.zeros(shape, dtype=torch.uint8, device=self._device)
        self._value_buf = torch.zeros(shape, dtype=torch.uint8, device=self._device)
        if self._ckpt_interval and self._kck is None:
            self._kck = gemv.alloc_ckpt(self._B, self._H, self._C, self._capacity_tokens, self._ckpt_interval, self._device)
            self._vck = gemv.alloc_ckpt(self._B, self._H, self._C, self._capacity_tokens, self._ckpt_interval, self._device)

    def _ckpt_kwargs(self):
        if not self._ckpt_interval:
            return {}
        return dict(k_ckpt=self._kck, v_ckpt=self._vck, ckpt_interval=self._ckpt_interval)

    def _init_buffers(self, B: int, H: int, C: int, device):
        if C not in (128, 256, 512):
            raise ValueError(f"ADKV kernels support head_dim in (128, 256, 512), got {C}")
        if C != 128 and self._ckpt_interval:
            raise ValueError("state checkpoints are available for head_dim 128 only")
        self._B, self._H, self._C, self._device = B, H, C, device
        self._quant_len = 0
        self._alloc(max(INIT_SEQ_LEN, self._capacity_tokens or 0))

    def _cap_buffers(self, T: int):
        """Grow by CAP_LEN slots until at least ``T`` tokens fit (copying the old contents)."""
        if T <= self._cap_len:
            return
        if self._ckpt_interval:
            raise ValueError(f"checkpointed cache is sized once: {T} tokens exceed capacity_tokens {self._cap_len}")
        new_cap = self._cap_len
        while new_cap < T:
            new_cap += CAP_LEN
        old_k, old_v, old_super = self._key_buf, self._value_buf, self._key_buf.shape[2]
        self._alloc(new_cap)
        self._key_buf[:, :, :old_super].copy_(old_k)
        self._value_buf[:, :, :old_super].copy_(old_v)

    # ------------------------------------------------------------------ prefill
    def prefill(self, key_states, value_states,
                key_zp_init, key_scale_init, key_alpha, key_beta, key_quant_target,
                value_zp_init, value_scale_init, value_alpha, value_beta, value_quant_target):
        """Quantise the prompt ``[B, H, T, C]`` into the cache.  No attention is computed here."""
        B, H, T, C = key_states.shape
        if value_states.shape != key_states.shape:
            raise ValueError("key/value shapes differ")
        if self._key_buf is None:
            self._init_buffers(B, H, C, key_states.device)
        elif (B, H, C) != (self._B, self._H, self._C):
            raise ValueError("cache was created for a different (B, H, C)")
        if T == 0:
            return
        if self._quant_len != 0:
            raise NotImplementedError(
                "ADKV prefill encodes from token 0; chunked prefill is not supported by this cache object")
        self._cap_buffers(T)
        key = key_states.to(torch.float16).contiguous()
        value = value_states.to(torch.float16).contiguous()
        v = lambda t: t.view(H, C)
        gemv.encode_kv_pair(self._key_buf, key,
                            (v(key_zp_init), v(key_scale_init), v(key_alpha), v(key_beta), v(key_quant_target)),
                            self._value_buf, value,
                            (v(value_zp_init), v(value_scale_init), v(value_alpha), v(value_beta),
                             v(value_quant_target)), SCALE_MIN, SCALE_MAX, bits=self.bits,
                            half_state=self.half_state, **self._ckpt_kwargs())
        self._quant_len += T

    # ------------------------------------------------------------------ decode
    def decode(self, query_states, key_states, value_states,
               key_zp_init, key_scale_init, key_alpha, key_beta, key_quant_target,
               value_zp_init, value_scale_init, value_alpha, value_beta, value_quant_target,
               attention_mask=None, scaling: float = 1.0):
        """Attend over the cached tokens, append the new K/V, return ``(output, weights or None)``.

        ``query_states [B, Hq, 1, C]``, ``key_states`` / ``value_states [B, H, 1, C]``; a standard causal
        decode step whose softmax covers the cached tokens and the token being appended."""
        B, Hq, Tq, C = query_states.shape
        _, H, Tk, _ = key_states.shape
        if Tq != 1 or Tk != 1:
            raise ValueError("decode expects exactly one query/key/value token")
        if Hq % H != 0:
            raise ValueError("query heads must be a multiple of key/value heads")
        if self._key_buf is None:
            self._init_buffers(B, H, C, query_states.device)
        elif (B, H, C) != (self._B, self._H, self._C):
            raise ValueError("cache was created for a different (B, H, C)")
        self._cap_buffers(self._quant_len + 1)
        ctx_len = self._quant_len
        q = query_states.to(torch.float16).contiguous()
        k = key_states.to(torch.float16).contiguous()
        v = value_states.to(torch.float16).contiguous()
        hv = lambda t: t.view(H, C)
        kp = tuple(hv(t) for t in (key_zp_init, key_scale_init, key_alpha, key_beta, key_quant_target))
        vp = tuple(hv(t) for t in (value_zp_init, value_scale_init, value_alpha, value_beta, value_quant_target))
        mask = None
        if attention_mask is not None:
            mask = attention_mask[:, :, 0, :] if attention_mask.dim() == 4 else attention_mask
        if self._ckpt_interval and not (mask is None or mask.numel() == B * (ctx_len + 1)):
            raise ValueError("a checkpointed cache takes masks shared by all heads only")
        if self.fused and (mask is None or mask.numel() == B * (ctx_len + 1)):
            out = gemv.decode_attn(q, self._key_buf, self._value_buf, k, v, kp, vp, ctx_len, scaling,
                                   SCALE_MIN, SCALE_MAX, mask=mask, bits=self.bits, fast=self.fast,
                                   half_state=self.half_state, **self._ckpt_kwargs())
            weights = None
        else:
            logits = gemv.forward_qk(q, self._key_buf, k, *kp, ctx_len, SCALE_MIN, SCALE_MAX,
                                     bits=self.bits, fast=self.fast, half_state=self.half_state)
            logits = logits.float() * scaling
            if mask is not None:
                logits = logits + mask.float()
            weights = torch.softmax(logits, dim=-1).to(torch.float16)
            out = gemv.forward_ov(weights, self._value_buf, v, *vp, SCALE_MIN, SCALE_MAX,
                                  bits=self.bits, fast=self.fast, half_state=self.half_state)
        self._quant_len = ctx_len + 1
        return out.to(query_states.dtype), weights


class KVCache(list):
    """List of per-layer caches (``src/adkv/hf/llama_adkv.py:279-288``)."""

    def __init__(self, num_layers: int, **layer_kwargs):
        super().__init__(KVCacheLayer(**layer_kwargs) for _ in range(num_layers))

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self[layer_idx].get_seq_length()

    def get_mask_sizes(self, cache_position, layer_idx: int) -> tuple[int, int]:
        return self[layer_idx].get_mask_sizes(cache_position)
