"""Head sharding by KV group across the GPUs of one node.

Every stage of the path is independent per head except the sharing state, so a rank that owns
the query heads of a contiguous range of KV heads needs two small exchanges per layer:

* before the election: every head's query-aware divergence (one fp32 per head), so that all
  ranks replay the same ascending-head election and agree on the pivots;
* after the pivot update: the summary of each pivot elected in this layer (pooled vertical and
  slash profiles, pattern bitmap, vs_ratio) from its owner to everyone.

Both are NCCL all-gathers of fixed size issued every layer, so no rank ever has to read a
device flag on the host.  Remote data lands in local HBM through NCCL before any kernel
reads it; no kernel touches peer memory.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def kv_group_shard(num_q_heads: int, num_kv_heads: int, rank: int, world: int) -> Tuple[int, int, int, int]:
    """(q_head_begin, q_head_end, kv_head_begin, kv_head_end) owned by ``rank``."""
    if num_kv_heads % world:
        raise ValueError(f"{num_kv_heads} KV heads cannot be split into {world} whole groups")
    per = num_kv_heads // world
    g = num_q_heads // num_kv_heads
    return rank * per * g, (rank + 1) * per * g, rank * per, (rank + 1) * per


class HeadShardExchange:
    def __init__(self, head_begin: int, head_end: int, group=None):
        self.h0, self.h1 = head_begin, head_end
        self.group = group
        self.world = dist.get_world_size(group)
        self.launches = 0

    def gather_heads(self, local: torch.Tensor) -> torch.Tensor:
        """All ranks' per-head values in global head order (equal shard sizes)."""
        out = torch.empty(self.world * local.numel(), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=self.group)
        return out

    def share_new_pivots(self, sharing, layer: int) -> None:
        st = sharing.state
        if st is None or st.n_slots == 0:
            return
        f = st.field
        head, lay = f("pivot_head"), f("pivot_layer")
        mine = (lay == layer) & (head >= self.h0) & (head < self.h1)          # [S] bool
        s = st.n_slots
        fl = [f("vs_ratio").view(torch.int32).view(s, 1), f("pivot_vertical").view(torch.int32),
              f("pivot_slash").view(torch.int32), f("pattern").reshape(s, -1)]
        packed = torch.cat([mine.to(torch.int32).view(s, 1)] + fl, dim=1)
        packed = torch.where(mine.view(s, 1), packed, torch.zeros_like(packed))
        gathered = torch.empty(self.world, *packed.shape, dtype=packed.dtype, device=packed.device)
        dist.all_gather_into_tensor(gathered, packed, group=self.group)
        merged = gathered.sum(0)                     # at most one rank contributes per slot
        new = merged[:, 0] > 0
        nb = st.nb
        o = 1
        upd = [("vs_ratio", 1), ("pivot_vertical", nb), ("pivot_slash", nb), ("pattern", fl[3].shape[1])]
        for name, width in upd:
            dst = f(name).view(torch.int32).reshape(s, -1)
            dst.copy_(torch.where(new.view(s, 1), merged[:, o:o + width], dst))
            o += width
        f("pattern_ready").copy_(torch.where(new, torch.ones_like(lay), f("pattern_ready")))
