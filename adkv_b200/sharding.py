"""Batch x KV-head sharding of the decode path across the GPUs of one node.

Every (batch, kv head) pair is an independent stream of the packed cache: nothing in the encode
or decode kernels crosses streams, so ranks own disjoint rectangles of the (batch, kv head) grid
and the data path needs no collective.  Query heads follow their KV head.  A collective (all-gather
of the ``[B, Hq, D]`` outputs) is only needed when one rank must see the whole result.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    rank: int
    b0: int
    b1: int
    h0: int     # kv heads [h0, h1)
    h1: int

    @property
    def n_streams(self) -> int:
        return (self.b1 - self.b0) * (self.h1 - self.h0)

    def q_heads(self, group: int) -> tuple[int, int]:
        return self.h0 * group, self.h1 * group


def _split(n: int, parts: int) -> list[tuple[int, int]]:
    base, rem = divmod(n, parts)
    out, lo = [], 0
    for i in range(parts):
        hi = lo + base + (1 if i < rem else 0)
        out.append((lo, hi))
        lo = hi
    return out


def grid_for(B: int, Hkv: int, world: int) -> tuple[int, int]:
    """(batch parts, head parts) with batch parts * head parts == world.

    Prefers splitting the batch (whole sequences stay on one GPU, as the tensor-parallel projections
    around attention expect); splits KV heads only as far as the batch cannot be divided evenly."""
    best = None
    for pb in range(1, world + 1):
        if world % pb:
            continue
        ph = world // pb
        if pb > B or ph > Hkv:
            continue
        uneven = (B % pb != 0) + (Hkv % ph != 0)
        key = (uneven, ph)              # even splits first, then as few head parts as possible
        if best is None or key < best[0]:
            best = (key, (pb, ph))
    if best is None:
        raise ValueError(f"cannot place {world} ranks on a {B} x {Hkv} (batch x kv-head) grid")
    return best[1]


def plan(B: int, Hkv: int, world: int) -> list[Shard]:
    """One shard per rank; together they cover every (batch, kv head) stream exactly once."""
    pb, ph = grid_for(B, Hkv, world)
    bs, hs = _split(B, pb), _split(Hkv, ph)
    return [Shard(r, *bs[r // ph], *hs[r % ph]) for r in range(world)]


def take(shard: Shard, group: int, *, q=None, kv=None, cache=None, params=None):
    """Slice tensors to a shard: ``q [B,Hq,...]``, ``kv``/``cache [B,Hkv,...]``, ``params`` 5 x ``[Hkv,D]``."""
    out = []
    if q is not None:
        q0, q1 = shard.q_heads(group)
        out.append(q[shard.b0:shard.b1, q0:q1].contiguous())
    if kv is not None:
        out.append(kv[shard.b0:shard.b1, shard.h0:shard.h1].contiguous())
    if cache is not None:
        out.append(cache[shard.b0:shard.b1, shard.h0:shard.h1].contiguous())
    if params is not None:
        out.append(tuple(p[shard.h0:shard.h1].contiguous() for p in params))
    return out[0] if len(out) == 1 else tuple(out)
