"""Per-layer packed KV cache for decoding on the B200 kernels.

Takes the place of the reference's ``KVCacheLayer_ADKV`` (``src/adkv/hf/llama_adkv.py:44-276``) in an attention
module: the public surface is the same -- ``prefill`` and ``decode`` with the reference's argument order,
``get_seq_length``, ``get_mask_sizes``, ``key_states`` / ``value_states`` -- and so is what ends up in the packed
buffers, bit for bit.  What happens behind it is organised for this library's kernels rather than for the
reference's three calls:

* **Tail states.**  Next to the codes the object keeps the recurrence state after the last cached token, per
  (sequence, KV head, channel), for K and for V.  Prefill leaves it behind, every decode step consumes and
  advances it.  The reference keeps no state and has its kernels replay the cache to find it
  (``src/adkv/kernel/gemv.cu:744-764``), which ties the replay to the encoder's exact arithmetic; here the replay
  only feeds the attention sums and runs in the contracted arithmetic, while the stored codes stay exact.
  The tails also make chunked prefill possible (the reference refuses it, ``llama_adkv.py:195-197``).
* **One launch per step.**  ``decode`` is one fused kernel (q.K^T, scaling, mask, softmax, P.V, both appends)
  instead of ``forward_qk`` -> four torch kernels -> ``forward_ov`` (``llama_adkv.py:263-276``); the attention
  weights are then never materialised and ``None`` is returned in their place.  ``fused=False`` issues the
  reference's sequence instead (and then works like the reference: no tails).
* **Storage grows geometrically.**  The reference reallocates and copies every 64 tokens
  (``llama_adkv.py:104-123``: O(T^2) bytes moved over a generation); here the buffers are sized for
  ``capacity_tokens`` when the caller knows it, and otherwise doubled -- one copy per doubling, of the used
  words only.
* Options the reference does not have: grouped-query attention (``llama_adkv.py:235-238`` raises), ``bits`` 2,
  ``half_state`` (the fp16-state arithmetic of the reference's CUDA kernels, ``src/adkv/kernel/gemv.cu:150-164``,
  for caches exchanged with them), ``checkpoint_interval`` (recurrence-state checkpoints every that many tokens,
  decoded with one warp pair per segment: long contexts, few sequences).
"""
from __future__ import annotations

import torch

from . import gemv
from .synth import SCALE_MAX, SCALE_MIN

MIN_TOKENS = 64      # smallest allocation, in tokens (the reference's first allocation, llama_adkv.py:40)
HEAD_DIMS = (128, 256, 512)


class KVCacheLayer:
    def __init__(self, bits: int = 4, fused: bool = True, fast: bool | None = None,
                 capacity_tokens: int | None = None, checkpoint_interval: int = 0, half_state: bool = False):
        if bits not in (2, 4):
            raise ValueError(f"bits must be 2 or 4, not {bits}")
        if checkpoint_interval and (not fused or checkpoint_interval % 32):
            raise ValueError("state checkpoints need the fused step and an interval that is a multiple of 32")
        self.bits, self.fused, self.fast, self.half_state = bits, fused, fast, half_state
        self._tokens_per_word = 32 // bits
        self._want_tokens = int(capacity_tokens or 0)
        self._interval = int(checkpoint_interval)
        self._geom = None                     # (B, H, D, device) once the first tensors have been seen
        self._k = self._v = None              # packed codes [B, H, words, D/4, 4, 4] uint8
        self._k_tail = self._v_tail = None    # float32 [B, H, 2, D]: state after the last cached token
        self._k_ckpt = self._v_ckpt = None    # float32 [B, H, n, 2, D]: state before token (i+1)*interval
        self._scratch = None
        self._n = 0                           # cached tokens

    # ------------------------------------------------------------------ what the attention module and HF ask
    def get_seq_length(self) -> int:
        return self._n

    def get_mask_sizes(self, cache_position) -> tuple[int, int]:
        new = cache_position if isinstance(cache_position, int) else cache_position.shape[0]
        return self._n + new, 0

    @property
    def key_states(self):
        return self._k

    @property
    def value_states(self):
        return self._v

    @property
    def tails(self):
        """(k_tail, v_tail) or (None, None) when this configuration keeps none."""
        return self._k_tail, self._v_tail

    @property
    def capacity(self) -> int:
        """Tokens the current buffers hold without growing."""
        return 0 if self._k is None else self._k.shape[2] * self._tokens_per_word

    # ------------------------------------------------------------------ storage
    @property
    def _keeps_tails(self) -> bool:
        return self.fused and not self.half_state

    def _bind(self, B: int, H: int, D: int, device) -> None:
        if self._geom is None:
            if D not in HEAD_DIMS:
                raise ValueError(f"head_dim {D} is not served by the kernels (one of {HEAD_DIMS})")
            if D != 128 and self._interval:
                raise ValueError("state checkpoints are available for head_dim 128 only")
            self._geom = (B, H, D, device)
        elif (B, H, D) != self._geom[:3]:
            raise ValueError(f"this cache holds (batch, kv heads, head_dim) = {self._geom[:3]}; got a different "
                             f"shape {(B, H, D)}")

    def _reserve(self, tokens: int) -> None:
        """Make room for ``tokens`` tokens.  First call: allocate; later: double (at least) and copy what is used."""
        if tokens <= self.capacity:
            return
        B, H, D, device = self._geom
        room = max(tokens, self._want_tokens, MIN_TOKENS, 2 * self.capacity)
        words = gemv.n_super_for(room, self.bits)
        fresh = [torch.zeros((B, H, words, D // 4, 4, 4), dtype=torch.uint8, device=device) for _ in range(2)]
        if self._k is not None:
            used = gemv.n_super_for(self._n, self.bits)
            fresh[0][:, :, :used].copy_(self._k[:, :, :used])
            fresh[1][:, :, :used].copy_(self._v[:, :, :used])
        self._k, self._v = fresh
        if self._keeps_tails and self._k_tail is None:
            self._k_tail = torch.zeros((B, H, 2, D), dtype=torch.float32, device=device)
            self._v_tail = torch.zeros_like(self._k_tail)
        if self._interval:
            cap = words * self._tokens_per_word
            grown = [gemv.alloc_ckpt(B, H, D, cap, self._interval, device) for _ in range(2)]
            if self._k_ckpt is not None:
                have = self._k_ckpt.shape[2]
                grown[0][:, :, :have].copy_(self._k_ckpt)
                grown[1][:, :, :have].copy_(self._v_ckpt)
            self._k_ckpt, self._v_ckpt = grown
            self._scratch = None

    def _state_kwargs(self, Hq: int | None = None) -> dict:
        """Keyword arguments that hand tails and checkpoints to the kernels."""
        kw = {}
        if self._keeps_tails:
            kw.update(k_tail=self._k_tail, v_tail=self._v_tail)
        if self._interval:
            kw.update(k_ckpt=self._k_ckpt, v_ckpt=self._v_ckpt, ckpt_interval=self._interval)
            if Hq is not None:      # decode: partial results of the segments
                B, H, _, device = self._geom
                need = gemv.decode_scratch_bytes(B, Hq, H, self.capacity, self._interval)
                if self._scratch is None or self._scratch.numel() < need:
                    self._scratch = torch.empty(need, dtype=torch.uint8, device=device)
                kw.update(scratch=self._scratch)
        return kw

    @staticmethod
    def _per_head(params, H: int, D: int):
        return tuple(t.view(H, D) for t in params)

    # ------------------------------------------------------------------ prefill
    def prefill(self, key_states, value_states,
                key_zp_init, key_scale_init, key_alpha, key_beta, key_quant_target,
                value_zp_init, value_scale_init, value_alpha, value_beta, value_quant_target):
        """Quantise ``[B, H, T, D]`` keys and values into the cache (no attention is computed).  With tail states
        a later call continues where the previous one stopped (chunked prefill)."""
        if key_states.shape != value_states.shape:
            raise ValueError(f"keys {tuple(key_states.shape)} and values {tuple(value_states.shape)} differ in shape")
        B, H, T, D = key_states.shape
        self._bind(B, H, D, key_states.device)
        if T == 0:
            return
        if self._n and not self._keeps_tails:
            raise NotImplementedError("continuing a prefill needs the tail states, which this configuration "
                                      "(fused=False or half_state=True) does not keep")
        self._reserve(self._n + T)
        kp = self._per_head((key_zp_init, key_scale_init, key_alpha, key_beta, key_quant_target), H, D)
        vp = self._per_head((value_zp_init, value_scale_init, value_alpha, value_beta, value_quant_target), H, D)
        gemv.encode_kv_pair(self._k, key_states.to(torch.float16), kp, self._v, value_states.to(torch.float16), vp,
                            SCALE_MIN, SCALE_MAX, bits=self.bits, t_start=self._n, half_state=self.half_state,
                            **self._state_kwargs())
        self._n += T

    # ------------------------------------------------------------------ decode
    def decode(self, query_states, key_states, value_states,
               key_zp_init, key_scale_init, key_alpha, key_beta, key_quant_target,
               value_zp_init, value_scale_init, value_alpha, value_beta, value_quant_target,
               attention_mask=None, scaling: float = 1.0):
        """One causal decode step: attend over the cached tokens and the new one, append the new K/V.

        ``query_states [B, Hq, 1, D]``, ``key_states`` / ``value_states [B, H, 1, D]``.  Returns
        ``(output [B, Hq, D], weights)``; ``weights`` is None for the fused step."""
        B, Hq, Tq, D = query_states.shape
        H, Tk = key_states.shape[1], key_states.shape[2]
        if Tq != 1 or Tk != 1:
            raise ValueError(f"a decode step takes exactly one new token per sequence, not {Tq} queries / {Tk} keys")
        if Hq % H:
            raise ValueError(f"{Hq} query heads cannot share {H} key/value heads")
        self._bind(B, H, D, query_states.device)
        T = self._n
        self._reserve(T + 1)
        q, k, v = (t.to(torch.float16) for t in (query_states, key_states, value_states))
        kp = self._per_head((key_zp_init, key_scale_init, key_alpha, key_beta, key_quant_target), H, D)
        vp = self._per_head((value_zp_init, value_scale_init, value_alpha, value_beta, value_quant_target), H, D)
        mask = attention_mask
        if mask is not None and mask.dim() == 4:
            mask = mask[:, :, 0, :]
        shared_mask = mask is None or mask.numel() == B * (T + 1)
        if self._interval and not shared_mask:
            raise ValueError("a checkpointed cache takes masks shared by all heads only")
        common = dict(bits=self.bits, fast=self.fast, half_state=self.half_state)
        if self.fused and shared_mask:
            out = gemv.decode_attn(q, self._k, self._v, k, v, kp, vp, T, scaling, SCALE_MIN, SCALE_MAX, mask=mask,
                                   **common, **self._state_kwargs(Hq))
            weights = None
        else:
            if self._keeps_tails:
                # a per-head mask cannot go through the fused kernel: write the token from the tails first (that
                # also advances them); the two calls below then rewrite the same code from their own replay
                gemv.append_kv_pair(self._k, k, kp, self._k_tail, self._v, v, vp, self._v_tail, T, SCALE_MIN, SCALE_MAX,
                                    bits=self.bits)
            common["fast"] = bool(self.fast) and not self._keeps_tails     # keep the rewritten code canonical
            logits = gemv.forward_qk(q, self._k, k, *kp, T, SCALE_MIN, SCALE_MAX, **common).float() * scaling
            if mask is not None:
                logits = logits + mask.float()
            weights = torch.softmax(logits, dim=-1).to(torch.float16)
            out = gemv.forward_ov(weights, self._v, v, *vp, SCALE_MIN, SCALE_MAX, **common)
        self._n = T + 1
        return out.to(query_states.dtype), weights


class KVCache(list):
    """The per-layer caches of a model (``src/adkv/hf/llama_adkv.py:279-288``)."""

    def __init__(self, num_layers: int, **layer_kwargs):
        super().__init__(KVCacheLayer(**layer_kwargs) for _ in range(num_layers))

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self[layer_idx].get_seq_length()

    def get_mask_sizes(self, cache_position, layer_idx: int) -> tuple[int, int]:
        return self[layer_idx].get_mask_sizes(cache_position)
