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


SUMMARY_FIELDS = ("vs_ratio", "pivot_vertical", "pivot_slash", "pattern")


def pack_pivot_summaries(state, layer: int, h0: int, h1: int) -> torch.Tensor:
    """int32 ``[S, 1 + widths]``: for every slot whose pivot was elected in ``layer`` among heads
    ``[h0, h1)`` a leading 1 and the summary fields' raw bits, zeros elsewhere."""
    f = state.field
    s = max(state.n_slots, 1)
    mine = (f("pivot_layer") == layer) & (f("pivot_head") >= h0) & (f("pivot_head") < h1)
    cols = [mine.to(torch.int32).view(s, 1)] + [f(n).view(torch.int32).reshape(s, -1) for n in SUMMARY_FIELDS]
    packed = torch.cat(cols, dim=1)
    return torch.where(mine.view(s, 1), packed, torch.zeros_like(packed))


def merge_pivot_summaries(state, gathered: torch.Tensor) -> None:
    """Install the summaries of ``gathered [ranks, S, width]`` (at most one rank contributes per
    slot) into the local state and mark those patterns ready."""
    f = state.field
    s = max(state.n_slots, 1)
    merged = gathered.sum(0)
    new = merged[:, 0] > 0
    o = 1
    for name in SUMMARY_FIELDS:
        dst = f(name).view(torch.int32).reshape(s, -1)
        width = dst.shape[1]
        dst.copy_(torch.where(new.view(s, 1), merged[:, o:o + width], dst))
        o += width
    ready = f("pattern_ready")
    ready.copy_(torch.where(new, torch.ones_like(ready), ready))


class HeadShardExchange:
    def __init__(self, head_begin: int, head_end: int, group=None):
        self.h0, self.h1 = head_begin, head_end
        self.group = group
        self.world = dist.get_world_size(group)
        self._buffers = None

    def gather_heads(self, local: torch.Tensor) -> torch.Tensor:
        """All ranks' per-head values in global head order (equal shard sizes)."""
        out = torch.empty(self.world * local.numel(), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=self.group)
        return out

    def share_new_pivots(self, sharing, layer: int) -> None:
        st = sharing.state
        if st is None or st.n_slots == 0:
            return
        from . import native
        if isinstance(st, native.SharingStateBuffer):
            # device state: one pack kernel, the all-gather, one merge kernel; buffers are reused
            key = (st.n_slots, st.nb, st.buf.device)
            if self._buffers is None or self._buffers[0] != key:
                width = native.load().spf_pivot_summary_width(st.nb)
                packed = torch.empty(st.n_slots, width, dtype=torch.int32, device=st.buf.device)
                flat = torch.empty(self.world, st.n_slots, width, dtype=torch.int32, device=st.buf.device)
                self._buffers = (key, packed, flat)
            _, packed, flat = self._buffers
            native.pack_pivot_summaries(st, layer, self.h0, self.h1, out=packed)
            dist.all_gather_into_tensor(flat.view(-1), packed.view(-1), group=self.group)
            native.merge_pivot_summaries(st, flat)
            return
        # any other state object exposing field(): the same exchange in torch ops (tests of the
        # exchange logic on CPU process groups)
        packed = pack_pivot_summaries(st, layer, self.h0, self.h1)
        flat = torch.empty(self.world * packed.numel(), dtype=packed.dtype, device=packed.device)
        dist.all_gather_into_tensor(flat, packed.reshape(-1), group=self.group)
        merge_pivot_summaries(st, flat.view(self.world, *packed.shape))
