"""Head-group sharding of the attention path across ranks.

Every (batch, KV-head group) of the op is independent: query head h reads KV
head h // (Hq/Hkv) (src/e1_rope_publication_v1.py:616) and nothing is reduced
across heads.  Rank r of P therefore owns the contiguous KV heads
[r*Hkv/P, (r+1)*Hkv/P) together with their query heads, runs the unmodified
single-GPU operator on that slice, and no collective is needed on the data
path.  Gamma vectors and rotary tables are replicated.  An all-gather of the
output along the head dimension is offered for callers that need the full
tensor on every rank; it is not part of the timed operator.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    kv_lo: int
    kv_hi: int
    q_lo: int
    q_hi: int

    @property
    def n_kv(self) -> int:
        return self.kv_hi - self.kv_lo

    @property
    def n_q(self) -> int:
        return self.q_hi - self.q_lo


def head_shard(hq: int, hkv: int, rank: int, world: int) -> HeadShard:
    """The slice of heads rank ``rank`` of ``world`` owns (whole GQA groups)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    if hkv < 1 or hq % hkv:
        raise ValueError("Hq must be a multiple of Hkv")
    if hkv % world:
        raise ValueError(f"{hkv} KV heads do not split evenly over {world} ranks")
    g = hq // hkv
    per = hkv // world
    return HeadShard(rank, world, rank * per, (rank + 1) * per, rank * per * g, (rank + 1) * per * g)


def shard_inputs(q, k, v, sh: HeadShard, contiguous: bool = True):
    """Slice full q/k/v [B,H,S,D] down to the heads of ``sh``.  With
    ``contiguous=False`` the batch-strided views are returned (the kernels
    take explicit strides); the benchmark materialises contiguous shards."""
    qs, ks, vs = q[:, sh.q_lo:sh.q_hi], k[:, sh.kv_lo:sh.kv_hi], v[:, sh.kv_lo:sh.kv_hi]
    if contiguous:
        qs, ks, vs = qs.contiguous(), ks.contiguous(), vs.contiguous()
    return qs, ks, vs


def gather_heads(out_local: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather per-rank outputs [B,Hq/P,S,D] into [B,Hq,S,D] on every rank
    (NCCL over NVLink on GPUs, gloo on CPU)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if world == 1:
        return out_local
    parts = [torch.empty_like(out_local) for _ in range(world)]
    dist.all_gather(parts, out_local.contiguous(), group=group)
    return torch.cat(parts, dim=1)
