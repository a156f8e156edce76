"""KV-head partitioning of the decode path over the GPUs of one node.

The reference is single-GPU (its kernels map query head ``hq`` to kv head ``hq // (Hq // Hkv)``,
csrc/kernels/gqa_decode.cu:96-97).  Attention and eviction are independent per (sequence, kv head), so
rank ``r`` of ``g`` owns a contiguous slice of kv heads together with the query heads of those groups;
nothing is read from a peer and the attention kernels need no collective.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    kv_heads: range   # global kv-head indices owned by this rank
    q_heads: range    # global query-head indices owned by this rank

    @property
    def n_kv(self) -> int:
        return len(self.kv_heads)

    @property
    def n_q(self) -> int:
        return len(self.q_heads)


def shard_heads(Hq: int, Hkv: int, world: int, rank: int) -> HeadShard:
    """Contiguous kv-head slice of ``rank`` and the query heads that attend to it."""
    if Hq <= 0 or Hkv <= 0 or Hq % Hkv:
        raise ValueError(f"Hq={Hq} must be a positive multiple of Hkv={Hkv}")
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if Hkv % world:
        raise ValueError(f"{Hkv} kv-heads cannot be split evenly over {world} ranks")
    per = Hkv // world
    group = Hq // Hkv
    kv = range(rank * per, (rank + 1) * per)
    return HeadShard(rank, world, kv, range(kv.start * group, kv.stop * group))


def shard_columns(n: int, world: int, rank: int) -> range:
    """Contiguous slice of ``n`` columns (MLP intermediate channels) owned by ``rank``."""
    if n % world:
        raise ValueError(f"{n} columns cannot be split evenly over {world} ranks")
    per = n // world
    return range(rank * per, (rank + 1) * per)
