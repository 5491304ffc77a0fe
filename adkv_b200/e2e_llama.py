"""End-to-end decode harness: a random-init Llama-architecture decoder on top of the ADKV kernels.

This is the caller side of the hot path for the end-to-end configuration (32 layers, d_model 4096,
32 heads, FFN 11008, fp16 weights ~ N(0, 0.02), random-token prompt, greedy generation with a 4-bit
ADKV cache), in the role of the reference's ``src/adkv/hf/llama_adkv.py`` + ``tools/perf_e2e.py``:
prefill runs dense causal attention on the prompt and quantises K/V into the packed caches
(``llama_adkv.py:358-378``), every decode step attends over the packed cache and appends the new
token (``llama_adkv.py:347-355``).  Differences that make it a B200 serving loop rather than a
port: caches are sized once for prompt + generation; one fused ``decode_attn`` launch per layer
replaces qk -> softmax -> ov; K and V of a layer are quantised in one launch; the recurrence state after the
last token is kept per layer (tail states), so every appended code comes from it bit-exactly while the replay
of the cache runs in the cheaper contracted arithmetic; and the model can be
tensor-parallel over the GPUs of a node (heads and FFN columns sharded, two NCCL all-reduces per
layer on the ``[B, d_model]`` activations, which are the only NVLink traffic -- attention itself
never leaves its GPU).

Everything except attention and quantisation is plain torch (cuBLAS GEMMs): it is plumbing around
the kernels, not part of what is measured against the roofline.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import gemv, synth


@dataclass
class LlamaShape:
    n_layers: int = 32
    d_model: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 32
    head_dim: int = 128
    ffn: int = 11008
    vocab: int = 32000
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5


def _rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope_tables(shape: LlamaShape, max_pos: int, device):
    half = shape.head_dim // 2
    inv = shape.rope_theta ** (-torch.arange(0, half, device=device, dtype=torch.float32) * 2.0 / shape.head_dim)
    ang = torch.arange(max_pos, device=device, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)     # [P, D] fp32


def _apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, H, T, D]; cos/sin [T, D] (HF rotate_half convention)."""
    half = x.shape[-1] // 2
    xf = x.float()
    rot = torch.cat([-xf[..., half:], xf[..., :half]], -1)
    return (xf * cos + rot * sin).to(x.dtype)


class ADKVLlama:
    """One tensor-parallel shard of the model with its packed KV caches."""

    def __init__(self, shape: LlamaShape, batch: int, max_tokens: int, bits: int = 4, device="cuda",
                 rank: int = 0, world: int = 1, seed: int = 0, fused: bool = True, fast: bool | None = None,
                 ckpt_interval: int = 0, half_state: bool = False, peers: list | None = None,
                 split_channels: bool | None = None):
        """``fast``: None = contracted replay wherever tail states keep the stored codes exact (the fused step in the
        fp32 arithmetic), canonical replay otherwise.  ``peers``: the other tensor-parallel shards when all of them
        live in this process (tests on one GPU); the all-reduce is then a sum over the shards' partial results, and
        the shards are stepped together with :func:`step_together`."""
        assert shape.n_heads % world == 0 and shape.n_kv_heads % world == 0 and shape.ffn % world == 0
        self.s, self.B, self.bits, self.dev = shape, batch, bits, torch.device(device)
        self.rank, self.world, self.fused, self.ckpt_interval = rank, world, fused, ckpt_interval
        self.half_state = half_state
        self.keeps_tails = fused and not half_state
        self.fast = self.keeps_tails if fast is None else fast
        self.peers = peers
        self.split_channels = split_channels      # layout of a head over warps in the eager fused step (None: automatic)
        self._marks = None                        # event recorder of profile_decode_step
        self.hq, self.hkv, self.ffn = shape.n_heads // world, shape.n_kv_heads // world, shape.ffn // world
        D, dm = shape.head_dim, shape.d_model
        g = torch.Generator(device=self.dev)
        g.manual_seed(seed)                       # same seed on every rank: replicated tensors agree

        def rnd(*sz):
            return (torch.randn(*sz, generator=g, device=self.dev, dtype=torch.float32) * 0.02).half()

        self.embed = rnd(shape.vocab, dm)
        self.lm_head = rnd(shape.vocab, dm)
        self.final_norm = torch.ones(dm, dtype=torch.float16, device=self.dev)
        self.layers = []
        h0, k0, f0 = rank * self.hq, rank * self.hkv, rank * self.ffn
        for li in range(shape.n_layers):
            # every rank draws the full-size layer from the same seed and keeps its slice, so the model is the
            # same function whatever the tensor-parallel degree
            gl = torch.Generator(device=self.dev)
            gl.manual_seed(seed * 1000 + li + 1)

            def rl(*sz):
                return (torch.randn(*sz, generator=gl, device=self.dev, dtype=torch.float32) * 0.02).half()

            wq, wk, wv = rl(shape.n_heads * D, dm), rl(shape.n_kv_heads * D, dm), rl(shape.n_kv_heads * D, dm)
            wo, wg, wu, wd = rl(dm, shape.n_heads * D), rl(shape.ffn, dm), rl(shape.ffn, dm), rl(dm, shape.ffn)
            kp = synth.gen_params(seed + 7 * li + 1, shape.n_kv_heads, D, bits, device=self.dev)
            vp = synth.gen_params(seed + 7 * li + 2, shape.n_kv_heads, D, bits, device=self.dev)
            self.layers.append(dict(
                wqkv=torch.cat([wq[h0 * D:(h0 + self.hq) * D], wk[k0 * D:(k0 + self.hkv) * D],
                                wv[k0 * D:(k0 + self.hkv) * D]]).contiguous(),
                wo=wo[:, h0 * D:(h0 + self.hq) * D].contiguous(),
                w_gate_up=torch.cat([wg[f0:f0 + self.ffn], wu[f0:f0 + self.ffn]]).contiguous(),
                w_down=wd[:, f0:f0 + self.ffn].contiguous(),
                norm1=torch.ones(dm, dtype=torch.float16, device=self.dev),
                norm2=torch.ones(dm, dtype=torch.float16, device=self.dev),
                kp=tuple(p[k0:k0 + self.hkv].contiguous() for p in kp),
                vp=tuple(p[k0:k0 + self.hkv].contiguous() for p in vp)))
            del wq, wk, wv, wo, wg, wu, wd
        ns = gemv.n_super_for(max_tokens, bits)
        for L in self.layers:
            L["kc"] = torch.zeros((batch, self.hkv, ns, D // 4, 4, 4), dtype=torch.uint8, device=self.dev)
            L["vc"] = torch.zeros_like(L["kc"])
            if self.keeps_tails:
                L["kt"] = torch.zeros((batch, self.hkv, 2, D), dtype=torch.float32, device=self.dev)
                L["vt"] = torch.zeros_like(L["kt"])
            if ckpt_interval:
                L["kck"] = gemv.alloc_ckpt(batch, self.hkv, D, max_tokens, ckpt_interval, self.dev)
                L["vck"] = gemv.alloc_ckpt(batch, self.hkv, D, max_tokens, ckpt_interval, self.dev)
        self.cos, self.sin = _rope_tables(shape, max_tokens, self.dev)
        self.T = 0
        self.scaling = D ** -0.5
        self.scratch = None
        if ckpt_interval:
            self.scratch = torch.empty(gemv.decode_scratch_bytes(batch, self.hq, self.hkv, max_tokens, ckpt_interval),
                                       dtype=torch.uint8, device=self.dev)

    # ------------------------------------------------------------------ helpers
    def _mark(self, name: str) -> None:
        """While profile_decode_step runs: a CUDA event that closes the segment `name`."""
        if self._marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def _allreduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            if self.peers is not None:      # shards of one process: summed by step_together
                raise RuntimeError("shards that share a process are stepped with step_together()")
            dist.all_reduce(x)
        self._mark("all_reduce")
        return x

    def _tails(self, L, b0=None, b1=None):
        if not self.keeps_tails:
            return {}
        return dict(k_tail=L["kt"][b0:b1], v_tail=L["vt"][b0:b1])

    def _mlp(self, L, x):
        gu = x @ L["w_gate_up"].T
        gate, up = gu[..., :self.ffn], gu[..., self.ffn:]
        return self._allreduce((F.silu(gate) * up) @ L["w_down"].T)

    def _qkv(self, L, h, T_new):
        B = h.shape[0]
        D = self.s.head_dim
        qkv = (h @ L["wqkv"].T).view(B, T_new, self.hq + 2 * self.hkv, D).transpose(1, 2)     # [B, H*, T, D]
        return qkv[:, :self.hq], qkv[:, self.hq:self.hq + self.hkv], qkv[:, self.hq + self.hkv:]

    def _ck(self, L):
        return dict(k_ckpt=L["kck"], v_ckpt=L["vck"], ckpt_interval=self.ckpt_interval) if self.ckpt_interval else {}

    # ------------------------------------------------------------------ prefill
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, batch_chunk: int = 16) -> torch.Tensor:
        """ids [B, Tp] -> next-token ids [B]; fills the caches with the quantised prompt."""
        B, Tp = ids.shape
        assert B == self.B and self.T == 0
        cos, sin = self.cos[:Tp], self.sin[:Tp]
        logits = []
        for b0 in range(0, B, batch_chunk):
            b1 = min(B, b0 + batch_chunk)
            x = self.embed[ids[b0:b1]]
            for L in self.layers:
                h = _rms_norm(x, L["norm1"], self.s.norm_eps)
                q, k, v = self._qkv(L, h, Tp)
                q, k = _apply_rope(q, cos, sin), _apply_rope(k, cos, sin)
                gemv.encode_kv_pair(L["kc"][b0:b1], k.contiguous(), L["kp"], L["vc"][b0:b1], v.contiguous(), L["vp"],
                                    synth.SCALE_MIN, synth.SCALE_MAX, bits=self.bits, half_state=self.half_state,
                                    **self._tails(L, b0, b1),
                                    **({"k_ckpt": L["kck"][b0:b1], "v_ckpt": L["vck"][b0:b1],
                                        "ckpt_interval": self.ckpt_interval} if self.ckpt_interval else {}))
                att = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.hq != self.hkv)
                x = x + self._allreduce(att.transpose(1, 2).reshape(b1 - b0, Tp, -1) @ L["wo"].T)
                x = x + self._mlp(L, _rms_norm(x, L["norm2"], self.s.norm_eps))
            last = _rms_norm(x[:, -1], self.final_norm, self.s.norm_eps)
            logits.append(last @ self.lm_head.T)
        self.T = Tp
        self.last_logits = torch.cat(logits)
        return self.last_logits.argmax(-1)

    # ------------------------------------------------------------------ the two halves of a layer, before the all-reduce
    def _attn_partial(self, L, x, T, cos, sin, seq_lens=None):
        """This shard's part of the attention block's output for one new token per sequence: [B, 1, d_model]."""
        h = _rms_norm(x, L["norm1"], self.s.norm_eps)
        q, k, v = self._qkv(L, h, 1)
        q, k = _apply_rope(q, cos, sin).contiguous(), _apply_rope(k, cos, sin).contiguous()
        v = v.contiguous()
        self._mark("norm_qkv_rope")
        smin, smax = synth.SCALE_MIN, synth.SCALE_MAX
        if seq_lens is not None:
            att = gemv.decode_attn_varlen(q, L["kc"], L["vc"], k, v, L["kp"], L["vp"], seq_lens, self.scaling, smin, smax,
                                          bits=self.bits, fast=self.fast, half_state=self.half_state, **self._tails(L))
        elif self.fused:
            att = gemv.decode_attn(q, L["kc"], L["vc"], k, v, L["kp"], L["vp"], T, self.scaling, smin, smax,
                                   bits=self.bits, fast=self.fast, half_state=self.half_state, scratch=self.scratch,
                                   split_channels=self.split_channels, **self._tails(L), **self._ck(L))
        else:   # the reference caller's three-call sequence (llama_adkv.py:263-276)
            logits = gemv.forward_qk(q, L["kc"], k, *L["kp"], T, smin, smax, bits=self.bits, fast=self.fast,
                                     half_state=self.half_state)
            w = torch.softmax(logits.float() * self.scaling, dim=-1).to(torch.float16)
            att = gemv.forward_ov(w, L["vc"], v, *L["vp"], smin, smax, bits=self.bits, fast=self.fast,
                                  half_state=self.half_state)
        self._mark("attention_kernels")
        out = att.reshape(self.B, 1, -1) @ L["wo"].T
        self._mark("o_proj")
        return out

    def _mlp_partial(self, L, x):
        gu = _rms_norm(x, L["norm2"], self.s.norm_eps) @ L["w_gate_up"].T
        out = (F.silu(gu[..., :self.ffn]) * gu[..., self.ffn:]) @ L["w_down"].T
        self._mark("norm_mlp")
        return out

    def _head(self, x):
        last = _rms_norm(x[:, 0], self.final_norm, self.s.norm_eps)
        self.last_logits = last @ self.lm_head.T
        tok = self.last_logits.argmax(-1)
        self._mark("final_norm_lm_head")
        return tok

    @torch.no_grad()
    def profile_decode_step(self, ids: torch.Tensor, steps: int = 4) -> tuple[torch.Tensor, dict]:
        """Run `steps` eager decode steps with a CUDA event after every segment of the step; returns the last
        tokens and the milliseconds per step spent in each kind of segment (device time between events, so host
        launch gaps are charged to the segment they precede; the residual additions ride with the all-reduce)."""
        totals: dict = {}
        tok = ids
        for _ in range(steps):
            self._marks = []
            start = torch.cuda.Event(enable_timing=True)
            start.record()
            tok = self.decode(tok)
            marks, self._marks = self._marks, None
            torch.cuda.synchronize(self.dev)
            prev = start
            for name, ev in marks:
                totals[name] = totals.get(name, 0.0) + prev.elapsed_time(ev)
                prev = ev
        per_step = {k: v / steps for k, v in totals.items()}
        per_step["step_total"] = sum(per_step.values())
        return tok, per_step

    # ------------------------------------------------------------------ decode, replayable
    @torch.no_grad()
    def _decode_body(self, ids: torch.Tensor) -> torch.Tensor:
        """One decode step in which nothing on the host depends on the position: the token count lives in
        ``self.seq_lens`` on the device (read by the attention kernel and the RoPE lookup, incremented at the
        end), so the recorded sequence of launches is the same for every step."""
        pos = self.seq_lens[:1].long()
        cos, sin = self.cos.index_select(0, pos), self.sin.index_select(0, pos)
        x = self.embed[ids][:, None, :]
        for L in self.layers:
            x = x + self._allreduce(self._attn_partial(L, x, None, cos, sin, seq_lens=self.seq_lens))
            x = x + self._allreduce(self._mlp_partial(L, x))
        self.seq_lens += 1
        return self._head(x)

    @torch.no_grad()
    def capture_decode(self, warmup_ids: torch.Tensor, warmup_steps: int = 3) -> torch.Tensor:
        """Run `warmup_steps` real decode steps eagerly, then record one step into a CUDA graph.
        Returns the token ids after the warm-up steps; continue with :meth:`decode_replay`.  The recorded step is
        the fused kernel with device-side lengths: the three-call sequence and checkpointed decode take the token
        count from the host and are refused here rather than silently replaced."""
        if not self.fused or self.ckpt_interval:
            raise ValueError("the replayable decode step is the fused kernel without state checkpoints "
                             "(fused=True, ckpt_interval=0)")
        self.seq_lens = torch.full((self.B,), self.T, dtype=torch.int32, device=self.dev)
        self._g_in = warmup_ids.clone()
        side = torch.cuda.Stream(device=self.dev)
        side.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(side):
            tok = self._g_in
            for _ in range(warmup_steps):
                tok = self._decode_body(tok)
            self._g_in.copy_(tok)
        torch.cuda.current_stream(self.dev).wait_stream(side)
        self.T += warmup_steps
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            self._g_out = self._decode_body(self._g_in)
        return self._g_in.clone()

    @torch.no_grad()
    def decode_replay(self, ids: torch.Tensor) -> torch.Tensor:
        self._g_in.copy_(ids)
        self._graph.replay()
        self.T += 1
        return self._g_out.clone()

    # ------------------------------------------------------------------ decode
    @torch.no_grad()
    def decode(self, ids: torch.Tensor) -> torch.Tensor:
        """ids [B] (the tokens at position T) -> next-token ids [B]; appends position T to the caches."""
        T = self.T
        cos, sin = self.cos[T:T + 1], self.sin[T:T + 1]
        x = self.embed[ids][:, None, :]                                                  # [B, 1, dm]
        for L in self.layers:
            x = x + self._allreduce(self._attn_partial(L, x, T, cos, sin))
            x = x + self._allreduce(self._mlp_partial(L, x))
        self.T = T + 1
        return self._head(x)


@torch.no_grad()
def step_together(shards: list, ids: torch.Tensor) -> torch.Tensor:
    """One decode step of tensor-parallel shards that live in one process (on one GPU): what every rank does in
    :meth:`ADKVLlama.decode`, with each all-reduce replaced by the sum of the shards' partial results.  Used to
    test the sharding (head slices of weights and ADKV parameters, caches per shard) without several GPUs."""
    T = shards[0].T
    cos, sin = shards[0].cos[T:T + 1], shards[0].sin[T:T + 1]
    x = shards[0].embed[ids][:, None, :]
    for li in range(len(shards[0].layers)):
        x = x + torch.stack([m._attn_partial(m.layers[li], x, T, cos, sin) for m in shards]).sum(0)
        x = x + torch.stack([m._mlp_partial(m.layers[li], x) for m in shards]).sum(0)
    for m in shards:
        m.T = T + 1
    tok = shards[0]._head(x)
    for m in shards[1:]:
        m.last_logits = shards[0].last_logits
    return tok


@torch.no_grad()
def prefill_together(shards: list, ids: torch.Tensor) -> torch.Tensor:
    """Prefill of co-resident shards (see :func:`step_together`)."""
    B, Tp = ids.shape
    cos, sin = shards[0].cos[:Tp], shards[0].sin[:Tp]
    x = shards[0].embed[ids]
    for li in range(len(shards[0].layers)):
        parts = []
        for m in shards:
            L = m.layers[li]
            q, k, v = m._qkv(L, _rms_norm(x, L["norm1"], m.s.norm_eps), Tp)
            q, k = _apply_rope(q, cos, sin), _apply_rope(k, cos, sin)
            gemv.encode_kv_pair(L["kc"], k.contiguous(), L["kp"], L["vc"], v.contiguous(), L["vp"], synth.SCALE_MIN,
                                synth.SCALE_MAX, bits=m.bits, half_state=m.half_state, **m._tails(L))
            att = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=m.hq != m.hkv)
            parts.append(att.transpose(1, 2).reshape(B, Tp, -1) @ L["wo"].T)
        x = x + torch.stack(parts).sum(0)
        x = x + torch.stack([m._mlp_partial(m.layers[li], x) for m in shards]).sum(0)
    for m in shards:
        m.T = Tp
    return shards[0]._head(x[:, -1:])


def run(shape: LlamaShape, batch: int, prompt: int, gen: int, bits: int = 4, fused: bool = True, fast: bool | None = None,
        ckpt_interval: int = 0, seed: int = 0, graph: bool = False, half_state: bool = False, breakdown: int = 0) -> dict:
    """Prefill a random prompt, generate `gen` tokens greedily; timings with CUDA events, max over ranks."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    model = ADKVLlama(shape, batch, prompt + gen + breakdown, bits=bits, device=dev, rank=rank, world=world, seed=seed,
                      fused=fused, fast=fast, ckpt_interval=ckpt_interval, half_state=half_state)
    g = torch.Generator(device=dev)
    g.manual_seed(seed + 99)
    ids = torch.randint(0, shape.vocab, (batch, prompt), generator=g, device=dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    ev[0].record()
    tok = model.prefill(ids)
    ev[1].record()
    out = [tok]
    if graph:
        # the warm-up steps and the capture are part of the timed decode region
        warm = min(3, gen)
        tok = model.capture_decode(tok, warm)
        out.append(tok)
        for _ in range(gen - warm):
            tok = model.decode_replay(tok)
            out.append(tok)
    else:
        for _ in range(gen):
            tok = model.decode(tok)
            out.append(tok)
    ev[2].record()
    torch.cuda.synchronize(dev)
    step_breakdown = None
    if breakdown and model.T + breakdown <= prompt + gen + breakdown:
        # extra eager steps after the timed region (the caches were sized for them)
        _, step_breakdown = model.profile_decode_step(tok, breakdown)
    t = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    prefill_ms, decode_ms = t.tolist()
    status = gemv.device_status(dev)
    toks = torch.stack(out, 1)
    return dict(rank=rank, world=world, prefill_ms=prefill_ms, decode_ms=decode_ms,
                decode_tokens_per_s=batch * gen / (decode_ms * 1e-3), ms_per_decode_step=decode_ms / gen,
                prefill_tokens_per_s=batch * prompt / (prefill_ms * 1e-3), device_status=status,
                token_checksum=int(toks.sum().item()), tokens=toks, fast=bool(model.fast),
                tail_states=model.keeps_tails, eager_step_breakdown_ms=step_breakdown)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--gen", type=int, default=512)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--bits", type=int, default=4)
    ap.add_argument("--unfused", action="store_true")
    ap.add_argument("--fast", action="store_true", help="contracted replay even without tail states")
    ap.add_argument("--exact", action="store_true", help="canonical replay even with tail states")
    ap.add_argument("--half-state", action="store_true",
                    help="the fp16-state arithmetic of the reference's CUDA kernels instead of the fp32 recurrence")
    ap.add_argument("--ckpt-interval", type=int, default=0)
    ap.add_argument("--graph", action="store_true", help="replay the decode step from a CUDA graph (device-side lengths)")
    ap.add_argument("--breakdown", type=int, default=0,
                    help="after the timed run, this many extra eager steps with CUDA events around every segment "
                         "(attention kernels, projections, MLP, all-reduces)")
    a = ap.parse_args()
    shape = LlamaShape(n_layers=a.layers)
    r = run(shape, a.batch, a.prompt, a.gen, bits=a.bits, fused=not a.unfused,
            fast=True if a.fast else (False if a.exact else None),
            ckpt_interval=a.ckpt_interval, graph=a.graph, half_state=a.half_state, breakdown=a.breakdown)
    if r["rank"] == 0:
        r.pop("tokens")
        r.update(metric="e2e_decode_tokens_per_s", config=dict(model="random-init Llama-2-7B architecture", batch=a.batch,
                 prompt=a.prompt, generate=a.gen, layers=a.layers, bits=a.bits, fused=not a.unfused,
                 replay="half" if a.half_state else ("contracted" if r["fast"] else "canonical"),
                 tail_states=r["tail_states"], tensor_parallel=r["world"],
                 cuda_graph=a.graph, data="synthetic"))
        print(json.dumps(r), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
