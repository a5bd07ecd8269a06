"""Head-shard planning for multi-GPU attention.

Every (batch, query head) pair is independent and a KV head is shared only by its own ``Hq/Hkv`` query heads,
so the path shards with no collective: rank ``r`` of ``world`` gets a contiguous range of whole KV groups.  When
there are fewer KV groups than ranks the batch is split next.  The optional all-gather of the output
(``aidn_sdpa_args.gather_output``) needs equal, consecutive head shards, which ``plan`` produces whenever
``Hkv % world == 0``.

The reference has no counterpart: its multi-device code (``Engines/MultiGpuManager.cs``, ``Engines/Distributed``)
never touches attention.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass(frozen=True)
class Shard:
    rank: int
    head_begin: int   # first q head
    head_count: int   # q heads (whole KV groups)
    batch_begin: int
    batch_count: int

    @property
    def empty(self) -> bool:
        return self.head_count == 0 or self.batch_count == 0


def plan(world: int, batch: int, num_q_heads: int, num_kv_heads: int) -> List[Shard]:
    """Partition ``batch x kv groups`` over ``world`` ranks: heads first (K/V never duplicated), then batch."""
    if world <= 0 or batch <= 0 or num_q_heads <= 0 or num_kv_heads <= 0:
        raise ValueError("world, batch and head counts must be positive")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be a multiple of num_kv_heads")
    group = num_q_heads // num_kv_heads
    shards: List[Shard] = []
    if num_kv_heads >= world:
        base, extra = divmod(num_kv_heads, world)
        start = 0
        for r in range(world):
            n = base + (1 if r < extra else 0)
            shards.append(Shard(r, start * group, n * group, 0, batch))
            start += n
        return shards
    # fewer KV groups than ranks: `per` ranks share one KV group and split the batch among themselves
    per = world // num_kv_heads
    for r in range(world):
        g, j = divmod(r, per)
        if g >= num_kv_heads:            # leftover ranks when world is not a multiple of num_kv_heads
            shards.append(Shard(r, 0, 0, 0, 0))
            continue
        b0 = (batch * j) // per
        b1 = (batch * (j + 1)) // per
        shards.append(Shard(r, g * group, group, b0, b1 - b0))
    return shards


def gatherable(shards: List[Shard]) -> bool:
    """True when the shards are equal consecutive head ranges over the whole batch (what the in-place
    all-gather of the output requires)."""
    if not shards:
        return False
    n = shards[0].head_count
    return all(s.head_count == n and s.head_begin == s.rank * n and s.batch_begin == 0
               and s.batch_count == shards[0].batch_count and n > 0 for s in shards)
