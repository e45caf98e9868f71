"""(batch x kv-head) shards of an attention problem and their placement on GPUs.

Every kernel grid of the reference is a product over (tile, head, batch)
(adasplash/adasplash_v2.py:1287, :1314, :1352, :1486, :1531) and dK/dV reduce
only over the query heads of one kv head (:1168), so one (batch item, kv head)
pair -- q (G, N, D) with G = Hq / Hkv, k and v (1, N, D) -- is a unit of work
that needs nothing from any other unit: no collective, no peer access.

A shard is that unit.  Its id is `b * Hkv + kv_head`.  Ranks get shards by
static assignment: round-robin when all sequences have the same length, longest
processing time first (weight L_b^2, the dense work of a causal sequence) when
they do not.  A shard's tensors are generated from `seed * 1000 + shard_id`,
so a shard holds the same data whichever rank owns it and however many ranks
there are.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch


@dataclass(frozen=True)
class Shard:
    shard_id: int
    b: int
    kv_head: int
    length: int   # valid rows of the sequence (N without varlen)

    @property
    def weight(self) -> int:
        return self.length * self.length


def enumerate_shards(B: int, Hkv: int, N: int, lens: Optional[Sequence[int]] = None) -> List[Shard]:
    """All B * Hkv shards in id order."""
    if lens is not None and len(lens) != B:
        raise ValueError(f"lens has {len(lens)} entries for B={B}")
    return [Shard(b * Hkv + h, b, h, int(lens[b]) if lens is not None else N)
            for b in range(B) for h in range(Hkv)]


def assign(shards: Sequence[Shard], world: int) -> List[List[Shard]]:
    """Static placement of shards on `world` ranks; returns one list per rank.

    Equal lengths: round-robin in id order (rank r gets ids r, r + world, ...), which for
    B * Hkv divisible by world gives every rank the same number of shards.  Unequal lengths:
    longest processing time first on weight L^2 -- shards in decreasing weight (ties by id),
    each to the rank with the least load so far (ties by rank).  The heaviest rank then carries
    at most the mean load plus one shard's weight.
    """
    if world < 1:
        raise ValueError("world must be >= 1")
    out: List[List[Shard]] = [[] for _ in range(world)]
    if len({s.length for s in shards}) <= 1:
        for i, s in enumerate(sorted(shards, key=lambda s: s.shard_id)):
            out[i % world].append(s)
        return out
    load = [0] * world
    for s in sorted(shards, key=lambda s: (-s.weight, s.shard_id)):
        r = min(range(world), key=lambda i: (load[i], i))
        out[r].append(s)
        load[r] += s.weight
    for lst in out:
        lst.sort(key=lambda s: s.shard_id)
    return out


def loads(assignment: Sequence[Sequence[Shard]]) -> List[int]:
    return [sum(s.weight for s in lst) for lst in assignment]


def shard_seed(seed: int, shard_id: int) -> int:
    return seed * 1000 + shard_id


def make_shard_inputs(shard: Shard, G: int, N: int, D: int, seed: int, scale: float,
                      dtype=torch.bfloat16, device="cpu"):
    """q (1,G,N,D), k, v (1,1,N,D) = N(0,1) * scale and dO (1,G,N,D) = N(0,1), zero on the rows at
    or beyond the shard's length, drawn on `device` from the shard's own seed."""
    g = torch.Generator(device=device).manual_seed(shard_seed(seed, shard.shard_id))

    def rn(shape, s):
        return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * s).to(dtype)
    q = rn((1, G, N, D), scale)
    k = rn((1, 1, N, D), scale)
    v = rn((1, 1, N, D), scale)
    do = rn((1, G, N, D), 1.0)
    if shard.length < N:
        do[:, :, shard.length:] = 0
    return q, k, v, do


def make_rank_batch(my_shards: Sequence[Shard], G: int, N: int, D: int, seed: int, scale: float,
                    dtype=torch.bfloat16, device="cpu"):
    """The shards of one rank as one attention problem: batch item i = shard i, Hq = G, Hkv = 1.
    Returns q, k, v, dO and the int32 lengths (None when every shard is full length)."""
    if not my_shards:
        return None
    parts = [make_shard_inputs(s, G, N, D, seed, scale, dtype, device) for s in my_shards]
    q, k, v, do = (torch.cat([p[i] for p in parts], dim=0).contiguous() for i in range(4))
    lens = [s.length for s in my_shards]
    varlen = None
    if any(l < N for l in lens):
        varlen = torch.tensor(lens, dtype=torch.int32, device=device)
    return q, k, v, do, varlen
