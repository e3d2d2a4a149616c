"""Pattern selection and cross-head sharing state, device resident.

Host-side mirror of ``AttentionSharing`` (attn/attention_sharing.py:35-384): same
construction from a lookup file, ``reset_state``, ``find_cluster_id``,
``get_active_blocks`` and ``update_pivotal_attns``.  The dictionaries of tensors the
reference keeps per cluster live in one device buffer, decisions are device flags and
patterns are bitmaps, so a layer's selection runs without a host synchronisation.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Tuple

import torch

from . import native


class BlockPattern:
    """Selected blocks of one layer: ``bitmap[H][nb][nbw]`` plus per-head flags."""

    def __init__(self, bitmap, flags, slot_of_head, nb, nv, ns, info=None):
        self.bitmap = bitmap
        self.flags = flags
        self.slot_of_head = slot_of_head
        self.num_blocks = nb
        self.nv, self.ns = nv, ns
        self.info = info or {}

    @property
    def use_dense(self) -> torch.Tensor:
        """bool ``[1,H]``: heads elected pivot in this layer (the reference's ``use_dense``)."""
        return ((self.flags & native.HEAD_PIVOT) != 0)[None]

    def to_index_lists(self) -> List[List[torch.Tensor]]:
        """The reference's format: ``[batch][head] ->`` sorted unique int64 flat indices."""
        return [native.bitmap_to_sets(self.bitmap)]

    def visited_blocks(self) -> torch.Tensor:
        return native.bitmap_row_counts(self.bitmap)[1]


def load_lookup(file_path: str) -> Tuple[Dict[str, list], set]:
    """Read a head-cluster lookup (reference JSON layout or the compact table)."""
    if not os.path.exists(file_path):
        raise FileNotFoundError(f"Sharing lookup file not found: {file_path}")
    with open(file_path, "r") as f:
        info = json.load(f)
    if info.get("format") == "spf-cluster-table-v1":
        from .clusters.convert_lookup import from_table
        info = from_table(info)
    return info["clusters"], set(info["shared_clusters"])


class AttentionSharing:
    def __init__(self, sharing_lookup_path: str, head_range: Optional[Tuple[int, int]] = None,
                 exchange=None):
        """``head_range=(h0, h1)`` makes this instance own query heads ``[h0, h1)`` of a larger
        model (one KV-group shard per GPU); ``exchange`` then provides the two small
        collectives (see ``shareprefill_b200.sharded``)."""
        self.sharing_lookup_path = sharing_lookup_path
        self.clusters, self.shared_clusters = self.load_clusters(sharing_lookup_path)
        self._cluster_of: Dict[Tuple[int, int], str] = {}
        for cid, pairs in self.clusters.items():
            for layer, head in pairs:
                self._cluster_of.setdefault((int(layer), int(head)), cid)
        # slot = position of a shared cluster in a fixed order
        self.slot_ids: List[str] = [c for c in self.clusters.keys() if c in self.shared_clusters]
        self._slot_index = {c: i for i, c in enumerate(self.slot_ids)}
        self.head_range = head_range
        self.exchange = exchange
        self._slot_tables: Dict[Tuple[int, int, str], torch.Tensor] = {}
        self._layer_shares: Dict[Tuple[int, int], bool] = {}
        self._state: Optional[native.SharingStateBuffer] = None
        self._qa_scores: Optional[torch.Tensor] = None
        self._needs_reset = True
        self.last_pattern: Optional[BlockPattern] = None
        self.on_stage = None   # optional callable(stage_name), e.g. to record CUDA events

    def _mark(self, stage: str):
        if self.on_stage is not None:
            self.on_stage(stage)

    # ---- lookup
    @staticmethod
    def load_clusters(file_path: str):
        return load_lookup(file_path)

    def find_cluster_id(self, layer: int, head: int) -> Optional[str]:
        return self._cluster_of.get((int(layer), int(head)))

    def _slot_table(self, layer: int, num_heads: int, device) -> torch.Tensor:
        key = (int(layer), num_heads, str(device))
        t = self._slot_tables.get(key)
        if t is None:
            slots = []
            for h in range(num_heads):
                cid = self.find_cluster_id(layer, h)
                if cid is None:
                    # the reference fails on such a head as soon as it is not query-aware
                    # (attention_sharing.py:83-84); here the lookup is checked up front
                    raise TypeError(f"(layer {layer}, head {h}) is missing from the sharing lookup "
                                    f"{self.sharing_lookup_path}")
                slots.append(self._slot_index.get(cid, -1))
            t = torch.tensor(slots, dtype=torch.int32, device=device)
            self._slot_tables[key] = t
            self._layer_shares[(int(layer), num_heads)] = any(x >= 0 for x in slots)
        return t

    def layer_can_share(self, layer: int, num_heads: int) -> bool:
        """Does any head of this layer belong to a shared cluster?  Known from the lookup alone, so
        the host may skip the pivot passes and the pivot exchange of layers where it is False."""
        return self._layer_shares.get((int(layer), num_heads), True)

    # ---- state
    def reset_state(self):
        """Forget all pivots; called before every forward (shareprefill_patch.py:156-160)."""
        self._needs_reset = True
        self.last_pattern = None

    def _ensure_state(self, nb: int, device) -> native.SharingStateBuffer:
        st = self._state
        if st is None or st.nb != nb or st.buf.device != device:
            st = native.SharingStateBuffer(len(self.slot_ids), nb, device)
            self._state = st
            self._needs_reset = False
        elif self._needs_reset:
            st.reset()
            self._needs_reset = False
        return st

    @property
    def state(self) -> Optional[native.SharingStateBuffer]:
        return self._state

    # ---- selection
    def get_active_blocks(
        self,
        q: torch.Tensor,
        k: torch.Tensor,
        layer_idx: int,
        num_heads: int,
        block_size: int,
        min_budget: int,
        max_budget: int,
        pattern_threshold: float = 0.9,
        similarity_threshold: float = 0.5,
        fallback_threshold: float = 0.9,
        queryaware_threshold: float = 0.1,
        gqa_interleave: bool = False,
        stage_inputs: Optional[dict] = None,
    ):
        """Select the blocks each head visits (attn/attention_sharing.py:105-366).

        ``q`` is ``[1,N,H,D]`` (or ``[N,H,D]``), ``k`` ``[1,N,Hkv,D]`` with the UN-repeated KV
        heads; ``min_budget`` / ``max_budget`` are in blocks, as the reference passes them.
        Returns ``(BlockPattern, use_dense[1,H])``.

        ``stage_inputs`` (tests) replaces computed intermediates by given tensors:
        ``vertical``/``slash`` ``[H,N]``, ``avg_qk`` ``[H,nb]``, ``qa_scores`` ``[H,nb,nb]``.
        """
        ctx = self.profile_heads(q, k, layer_idx, num_heads, block_size, min_budget, max_budget,
                                 pattern_threshold, gqa_interleave, stage_inputs)
        return self.select_blocks(ctx, self._all_heads_divergence(ctx), similarity_threshold,
                                  fallback_threshold, queryaware_threshold)

    def _all_heads_divergence(self, ctx: dict) -> torch.Tensor:
        """Every head's query-aware divergence, as the election needs it.  With the heads sharded, the
        other ranks' values come through the exchange - but only in layers where some head belongs
        to a shared cluster: elsewhere no pivot can be elected, a head's flags depend on its own
        divergence alone, and the collective (a synchronisation point of all ranks) is skipped; the
        entries of the other ranks' heads are then NaN, which the election reads as "nothing to do"."""
        local = ctx["jsd_qa"]
        if self.exchange is None:
            return local
        if self.layer_can_share(ctx["layer"], ctx["num_heads"]):
            return self.exchange.gather_heads(local)
        full = torch.full((ctx["num_heads"],), float("nan"), dtype=local.dtype, device=local.device)
        full[ctx["h0"]:ctx["h0"] + local.numel()] = local
        return full

    def profile_heads(self, q, k, layer_idx, num_heads, block_size, min_budget, max_budget,
                      pattern_threshold=0.9, gqa_interleave=False, stage_inputs=None) -> dict:
        """First half of ``get_active_blocks``: everything that is independent per head (pooling,
        last-block profile, budgets, pooled last-row estimate, divergences).  The returned context
        carries ``jsd_qa`` - the one per-head value every rank needs from every other rank."""
        if gqa_interleave:
            raise NotImplementedError("gqa_interleave=True is not supported by the B200 kernels")
        if q.dim() == 4:
            if q.shape[0] != 1:
                raise NotImplementedError("the sharing state assumes batch size 1")
            q, k = q[0], k[0]
        n, h, d = q.shape
        nb = native.num_blocks(n, block_size)
        dev = q.device
        state = self._ensure_state(nb, dev)
        h0 = 0 if self.head_range is None else self.head_range[0]
        slot_all = self._slot_table(layer_idx, num_heads, dev)
        slot_local = slot_all[h0:h0 + h] if (h0 or h != num_heads) else slot_all
        si = stage_inputs or {}

        avg_q, avg_k = native.pool_qk(q, k, block_size)
        self._mark("pool")
        if "vertical" in si:
            vertical, slash = si["vertical"], si["slash"]
        else:
            vertical, slash = native.lastblock_profile(q, k, block_size)
        self._mark("profile")
        max_blocks = min(int(max_budget), nb)
        nv, ns, vpool, spool = native.profile_budgets(vertical, slash, block_size, pattern_threshold,
                                                      min_budget, max_blocks)
        avg_qk = si["avg_qk"] if "avg_qk" in si else native.pooled_last_row(q, avg_k, block_size)
        jsd_qa, jsd_v, jsd_s = native.classify_heads(avg_qk, vpool, spool, slot_local, state)
        return dict(layer=layer_idx, nb=nb, h0=h0, state=state, num_heads=num_heads, slot_all=slot_all, slot_local=slot_local,
                    avg_q=avg_q, avg_k=avg_k, vertical=vertical, slash=slash, nv=nv, ns=ns, vpool=vpool,
                    spool=spool, avg_qk=avg_qk, jsd_qa=jsd_qa, jsd_v=jsd_v, jsd_s=jsd_s,
                    min_blocks=min_budget, pattern_threshold=pattern_threshold,
                    qa_scores=si.get("qa_scores"))

    def select_blocks(self, ctx: dict, jsd_qa_all: torch.Tensor, similarity_threshold=0.5,
                      fallback_threshold=0.9, queryaware_threshold=0.1):
        """Second half: election / sharing over ALL heads' divergences, then this instance's
        heads' patterns.  Returns ``(BlockPattern, use_dense[1,H])``."""
        state = ctx["state"]
        nv, ns, vpool, spool = ctx["nv"], ctx["ns"], ctx["vpool"], ctx["spool"]
        flags = native.elect_and_share(jsd_qa_all, ctx["slot_all"], ctx["h0"], ctx["jsd_v"], ctx["jsd_s"],
                                       vpool, spool, state, ctx["layer"], queryaware_threshold,
                                       similarity_threshold, fallback_threshold, ctx["min_blocks"], nv, ns)
        bitmap = native.build_vs_bitmap(vpool, spool, nv, ns, flags, ctx["slot_local"], state)
        scores = ctx["qa_scores"]
        if scores is None:
            # one buffer per shape, reused by every layer and never cleared: only the rows of query-aware
            # heads are written (in full) and read
            nb_, h_ = ctx["nb"], ctx["avg_q"].shape[1]
            buf = self._qa_scores
            if buf is None or buf.shape != (h_, nb_, nb_) or buf.device != ctx["avg_q"].device:
                buf = torch.empty(h_, nb_, nb_, dtype=torch.float32, device=ctx["avg_q"].device)
                self._qa_scores = buf
            scores = native.query_aware_scores(ctx["avg_q"], ctx["avg_k"], flags, scores=buf)
        native.query_aware_select(scores, flags, ctx["pattern_threshold"], bitmap)
        pat = BlockPattern(bitmap, flags, ctx["slot_local"], ctx["nb"], nv, ns,
                           info={"can_share": self.layer_can_share(ctx["layer"], ctx["num_heads"]),
                                 **{k_: ctx[k_] for k_ in ("vertical", "slash", "vpool", "spool", "avg_qk",
                                                        "avg_k", "avg_q", "jsd_qa", "jsd_v", "jsd_s")}})
        self.last_pattern = pat
        self._mark("select")
        return pat, pat.use_dense

    def update_pivotal_attns(self, layer_idx, avg_attn, use_dense, pattern_threshold=0.9):
        """Build the shared pattern of every head elected pivot in this layer from its
        block-mass matrix (attn/attention_sharing.py:94-103).  The matrix was written into the
        state by the attention kernel; ``avg_attn`` / ``use_dense`` are accepted for signature
        compatibility and ignored."""
        pat = self.last_pattern
        if pat is not None and self._state is not None and self.slot_ids and pat.info.get("can_share", True):
            native.update_pivots(pat.flags, pat.slot_of_head, self._state, pattern_threshold)
            if self.exchange is not None:
                self.exchange.share_new_pivots(self, layer_idx)
        self._mark("pivot_update")
