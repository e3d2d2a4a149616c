"""CPU oracle for the sparse-prefill attention path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module: only ``tests/``, the
smoke check and the CPU-baseline / reference arm of ``bench.py`` use it, and
only as the checker.  It restates, with torch CPU ops, what the reference
computes between the Hugging Face attention interface and the attention output:

* selection  - shareprefill/attn/attention_sharing.py:105-366 (``get_active_blocks``)
* helpers    - shareprefill/attn/utils.py:26-128
* attention  - shareprefill/attn/shareprefill_attn.py:331-471 (the Triton kernel's
               arithmetic) and :226-269 (CSR offsets)
* pivot state- shareprefill/attn/attention_sharing.py:94-103 (``update_pivotal_attns``)

Pinning.  The reference has no tests and no golden vectors of its own, so the oracle is
pinned against outputs of the reference's code itself:
* selection: the reference's ``get_active_blocks`` / ``update_pivotal_attns`` / helpers imported
  and run on CPU (``tests/golden/make_golden.py`` -> ``tests/golden/*.npz``): every block set,
  flag, pivot pattern and vs_ratio is reproduced exactly;
* attention, CSR offsets, pooling: the reference's Triton kernels run unmodified on a B200
  (``tests/golden/make_golden_triton.py`` -> ``tests/golden/triton_kernels.npz``): attention
  outputs agree within the path's bf16 tolerance (max-abs 2e-2 / mean-abs 2e-3), block-mass
  matrices within 2e-3, CSR offsets exactly; the pooled means differ from the Triton kernel's
  by its bf16 reduction-tree rounding (this restatement sums in fp32).

The arithmetic follows torch CPU semantics the reference inherits: ``cumsum`` on
fp32 accumulates in fp64 and rounds every prefix to fp32; comparisons against a
Python float are made in fp32; sort/topk tie order is unspecified (callers keep
test data tie-free at the decision boundaries).

Layout here is token-major and batch-free: q ``[N,H,D]``, k/v ``[N,Hkv,D]``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

INT32_MAX = 2**31 - 1


# --------------------------------------------------------------------------- helpers

def sqrt_jsd(p: torch.Tensor, q: torch.Tensor) -> torch.Tensor:
    """Square root of the Jensen-Shannon divergence along the last dim (utils.py:26-30).

    Exact zeros give 0*log(0) = NaN, which makes every ``<`` test false; kept on purpose.
    """
    m = (p + q) / 2
    a = (p * torch.log(p / m)).sum(-1)
    b = (q * torch.log(q / m)).sum(-1)
    return torch.sqrt(0.5 * a + 0.5 * b)


def block_sum_pool(x: torch.Tensor, bs: int) -> torch.Tensor:
    """Sum groups of ``bs`` along the last dim, zero padded (utils.py:33-44)."""
    n = x.shape[-1]
    pad = -(-n // bs) * bs - n
    x = torch.nn.functional.pad(x, (0, pad), value=0)
    return x.reshape(*x.shape[:-1], -1, bs).sum(-1)


def cover_count(x: torch.Tensor, thr: float) -> torch.Tensor:
    """Elements needed to cover ``thr``, crossing element included (utils.py:47-50)."""
    s = torch.sort(x, dim=-1, descending=True).values
    c = torch.cumsum(s, dim=-1)
    return (c <= thr).sum(-1) + 1


def cover_indices_global(x: torch.Tensor, thr: float) -> torch.Tensor:
    """Indices whose sorted prefix sum stays <= thr, crossing one excluded (utils.py:53-57).

    Returns the unique kept indices plus index 0 (the reference pads with 0).
    """
    s, idx = torch.sort(x, dim=-1, descending=True)
    c = torch.cumsum(s, dim=-1)
    kept = idx[c <= thr]
    return torch.unique(torch.cat((kept, kept.new_zeros(1))))


def cover_indices_rows(x: torch.Tensor, thr: float) -> torch.Tensor:
    """Per-row cover sets, crossing element included, as flat indices (utils.py:60-76).

    A row whose prefix sums never reach ``thr`` keeps one element (argmax of an
    all-false mask is 0).  Index 0 is always present (padding value).
    """
    rows, cols = x.shape
    s, idx = torch.sort(x, dim=-1, descending=True)
    c = torch.cumsum(s, dim=-1)
    keep_n = (c >= thr).float().argmax(dim=-1) + 1
    pos = torch.arange(cols)[None, :]
    flat = idx + torch.arange(rows)[:, None] * cols
    flat = torch.where(pos < keep_n[:, None], flat, torch.zeros_like(flat))
    return torch.unique(flat.reshape(-1))


def antidiagonal_sums(p: torch.Tensor) -> torch.Tensor:
    """``out[..., j] = sum_i p[..., i, j - (n-1) + i]`` (utils.py:79-86).

    With the ``n`` query rows being the last ``n`` tokens of an ``m``-token
    sequence, ``out[m-1-d]`` collects the mass at query-key distance ``d``.
    """
    n, m = p.shape[-2], p.shape[-1]
    padded = torch.nn.functional.pad(p, (n - 1, 0), value=0)
    out = torch.zeros(*p.shape[:-2], m, dtype=p.dtype)
    for i in range(n):
        out += padded[..., i, i:i + m]
    return out


def vs_multiset(v_idx: torch.Tensor, s_idx: torch.Tensor, nb: int) -> torch.Tensor:
    """Flat block indices of a vertical/slash pattern, duplicates and 0-padding kept
    (utils.py:99-128).  ``v_idx`` are column blocks, ``s_idx`` block distances."""
    r = torch.arange(nb)[:, None]
    vert = r * nb + v_idx[None, :]
    vert = torch.where(r >= v_idx[None, :], vert, torch.zeros_like(vert)).reshape(-1)
    sl = (r + s_idx[None, :]) * nb + r
    sl = torch.where(sl < nb * nb, sl, torch.zeros_like(sl)).reshape(-1)
    return torch.cat((sl, vert))


def block_mean_pool(x: torch.Tensor, bs: int) -> torch.Tensor:
    """Mean over token blocks of ``x[N,H,D]`` -> ``[nb,H,D]`` in x's dtype; the last,
    partial block divides by its true length (utils.py:171,186-187,217).

    The Triton kernel reduces in the input dtype with an unspecified tree order;
    this restatement accumulates in fp32 and rounds once.
    """
    n, h, d = x.shape
    nb = -(-n // bs)
    pad = nb * bs - n
    xf = torch.nn.functional.pad(x.float(), (0, 0, 0, 0, 0, pad))
    s = xf.reshape(nb, bs, h, d).sum(1)
    cnt = torch.full((nb, 1, 1), float(bs))
    cnt[-1] = bs - pad
    return (s / cnt).to(x.dtype)


# --------------------------------------------------------------------------- stages

def last_block_profile(q: torch.Tensor, k: torch.Tensor, bs: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Vertical and slash profiles of the last query block (attention_sharing.py:127-167).

    Returns ``vertical[H,N]`` (mean over the block's queries of the softmax) and
    ``slash[H,N]`` (mean over queries of the mass on each anti-diagonal), fp32.
    The logits are rounded to the input dtype before the fp32 softmax, as the
    reference's einsum does.
    """
    n, h, d = q.shape
    g = h // k.shape[1]
    lq = q[-bs:] / math.sqrt(d)
    rows = lq.shape[0]
    vertical = torch.empty(h, n, dtype=torch.float32)
    slash = torch.empty(h, n, dtype=torch.float32)
    i = torch.arange(rows)
    for hh in range(h):
        logits = (lq[:, hh, :] @ k[:, hh // g, :].T)
        tail = logits[:, -bs:]
        tail.masked_fill_(~(i[:, None] >= i[None, :])[-tail.shape[0]:, -tail.shape[1]:], float("-inf"))
        p = torch.softmax(logits, dim=-1, dtype=torch.float32)
        slash[hh] = antidiagonal_sums(p) / rows
        vertical[hh] = p.mean(-2)
    return vertical, slash


def block_budgets(vertical: torch.Tensor, slash: torch.Tensor, bs: int, thr: float,
                  min_blocks: int, max_blocks: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-head vertical / slash budgets in blocks (attention_sharing.py:169-176)."""
    nv = cover_count(vertical, thr) // bs + 1
    ns = cover_count(slash, thr) // bs + 1
    nv = nv.clamp(min=min_blocks).clamp(max=max_blocks)
    ns = ns.clamp(min=min_blocks).clamp(max=max_blocks)
    # the reference applies "< min -> min" then "> max -> max": max wins when min > max
    return nv, ns


def pooled_last_row(q: torch.Tensor, avg_k: torch.Tensor, bs: int) -> torch.Tensor:
    """softmax over blocks of mean(last queries / sqrt(D)) . avg_k (attention_sharing.py:197-200).

    ``avg_k`` is ``[nb,Hkv,D]``; returns ``[H,nb]`` fp32.
    """
    n, h, d = q.shape
    g = h // avg_k.shape[1]
    lq = (q[-bs:] / math.sqrt(d)).mean(0, keepdim=True)  # [1,H,D] in q's dtype
    out = torch.empty(h, avg_k.shape[0], dtype=torch.float32)
    for hh in range(h):
        logits = lq[:, hh, :] @ avg_k[:, hh // g, :].T
        out[hh] = torch.softmax(logits[0], dim=-1, dtype=torch.float32)
    return out


def query_aware_scores(q_h: torch.Tensor, avg_k_h: torch.Tensor, bs: int) -> torch.Tensor:
    """Causal block-level softmax of pooled Q . pooled K for one head, flattened
    ``[nb*nb]`` fp32 (attention_sharing.py:350-360).  ``q_h`` is ``[N,D]``."""
    n, d = q_h.shape
    nb = -(-n // bs)
    pad = nb * bs - n
    avg_q = torch.nn.functional.pad(q_h, (0, 0, 0, pad), value=0).view(nb, bs, d).mean(1)
    avg_q[-1, :] = avg_q[-1, :] * bs / (bs - pad)
    logits = (avg_q / math.sqrt(d)) @ avg_k_h.T
    logits.masked_fill_(~torch.tril(torch.ones(nb, nb, dtype=torch.bool)), float("-inf"))
    return torch.softmax(logits, dim=-1, dtype=torch.float32).view(-1)


def vs_lists(v_row: torch.Tensor, s_row: torch.Tensor, nv: int, ns: int, kv: int, ks: int):
    """Top ``kv`` vertical column blocks and top ``ks`` slash block distances of one
    head, slots beyond the head's own budgets zeroed (attention_sharing.py:306-329).
    ``v_row`` / ``s_row`` already carry the forced +inf on the sink / diagonal block."""
    nb = v_row.shape[-1]
    v_idx = v_row.topk(kv, -1).indices
    v_idx = torch.where(torch.arange(kv) < nv, v_idx, torch.zeros_like(v_idx))
    s_idx = (nb - 1) - s_row.topk(ks, -1).indices
    s_idx = torch.where(torch.arange(ks) < ns, s_idx, torch.zeros_like(s_idx))
    return v_idx, s_idx


# --------------------------------------------------------------------------- state + selection

class SharingOracle:
    """Per-forward pattern-sharing state and the block selection that uses it.

    Restates ``AttentionSharing`` (attention_sharing.py:35-384) for batch 1.
    ``lookup`` is the reference's JSON layout or a path to it.
    """

    def __init__(self, lookup):
        if isinstance(lookup, (str, os.PathLike)):
            if not os.path.exists(lookup):
                raise FileNotFoundError(f"Sharing lookup file not found: {lookup}")
            with open(lookup) as f:
                lookup = json.load(f)
        self.cluster_of: Dict[Tuple[int, int], str] = {}
        for cid, pairs in lookup["clusters"].items():
            for layer, head in pairs:
                self.cluster_of.setdefault((int(layer), int(head)), cid)
        self.shared = set(lookup["shared_clusters"])
        self.reset()

    def reset(self):
        self.pivot_head: Dict[str, int] = {}
        self.pivot_layer: Dict[str, int] = {}
        self.pivot_vertical: Dict[str, torch.Tensor] = {}
        self.pivot_slash: Dict[str, torch.Tensor] = {}
        self.pivot_vs: Dict[str, torch.Tensor] = {}
        self.pivot_attn: Dict[str, torch.Tensor] = {}
        self.pivot_pattern: Dict[str, torch.Tensor] = {}
        self.vs_ratio: Dict[str, float] = {}
        self.trace: List[dict] = []

    def cluster(self, layer: int, head: int) -> str:
        cid = self.cluster_of.get((layer, head))
        if cid is None:
            # the reference dereferences a missing dict entry here (attention_sharing.py:83-84)
            raise TypeError(f"(layer {layer}, head {head}) is not in the sharing lookup")
        return cid

    # ---- stage: everything after the pooled scores exist
    def select_from_scores(
        self,
        layer: int,
        vertical: torch.Tensor,       # [H,N] fp32
        slash: torch.Tensor,          # [H,N] fp32
        avg_qk: torch.Tensor,         # [H,nb] fp32 softmax of pooled last-row logits
        qa_scores,                    # callable h -> [nb*nb] fp32, or dict
        *,
        block_size: int,
        min_blocks: int,
        max_blocks: int,
        pattern_threshold: float,
        similarity_threshold: float,
        fallback_threshold: float,
        queryaware_threshold: float,
        heads: Optional[Sequence[int]] = None,
        vpool: Optional[torch.Tensor] = None,
        spool: Optional[torch.Tensor] = None,
    ):
        """Selection from pooled scores (attention_sharing.py:169-364).

        Returns ``(block_sets, use_dense, info)``: per head a sorted unique int64
        tensor of flat block indices ``row*nb+col``, a bool ``[H]`` marking heads
        elected pivot in this layer, and a dict of intermediates.

        ``heads`` (with ``vpool``/``spool`` ``[H,nb]`` for ALL heads): the rows of
        ``vertical``/``slash`` then belong to these heads only.  The election is replayed
        over all heads; budgets and block sets are only meaningful for ``heads`` (the
        other entries of the returned list are ``None``).
        """
        n = vertical.shape[-1]
        nb = -(-n // block_size)
        max_blocks = min(max_blocks, nb)
        nv, ns = block_budgets(vertical, slash, block_size, pattern_threshold, min_blocks, max_blocks)
        if heads is None:
            vpool = block_sum_pool(vertical, block_size)
            spool = block_sum_pool(slash, block_size)
        else:
            idx = torch.as_tensor(list(heads))
            nv_all = torch.full((avg_qk.shape[0],), min_blocks, dtype=nv.dtype)
            ns_all = nv_all.clone()
            nv_all[idx], ns_all[idx] = nv, ns
            nv, ns = nv_all, ns_all
        h = avg_qk.shape[0]
        jsd_qa = sqrt_jsd(avg_qk, vpool)
        use_qa = jsd_qa < queryaware_threshold
        use_dense = torch.zeros(h, dtype=torch.bool)
        use_share = torch.zeros(h, dtype=torch.bool)
        sets: List[torch.Tensor] = [torch.empty(0, dtype=torch.int64) for _ in range(h)]
        jsd_v = torch.full((h,), float("nan"))
        jsd_s = torch.full((h,), float("nan"))

        for hh in range(h):
            if bool(use_qa[hh]):
                continue
            cid = self.cluster(layer, hh)
            if cid not in self.shared:
                continue
            if cid not in self.pivot_head:
                # pivot election: full causal triangle, remember this head's profiles
                rr, cc = torch.tril_indices(nb, nb)
                sets[hh] = rr * nb + cc
                self.pivot_head[cid] = hh
                self.pivot_layer[cid] = layer
                use_dense[hh] = True
                self.pivot_vertical[cid] = vpool[hh].clone()
                self.pivot_slash[cid] = spool[hh].clone()
                v_w = vpool[hh].clone(); v_w[0] = float("inf")
                s_w = spool[hh].clone(); s_w[-1] = float("inf")
                v_idx, s_idx = vs_lists(v_w, s_w, int(nv[hh]), int(ns[hh]),
                                        min(int(nv[hh]), nb), min(int(ns[hh]), nb))
                self.pivot_vs[cid] = vs_multiset(v_idx, s_idx, nb)
            elif cid in self.pivot_pattern:
                jsd_v[hh] = sqrt_jsd(self.pivot_vertical[cid], vpool[hh])
                jsd_s[hh] = sqrt_jsd(self.pivot_slash[cid], spool[hh])
                if cid not in self.vs_ratio:
                    flat = self.pivot_attn[cid].reshape(-1)
                    self.vs_ratio[cid] = (flat[self.pivot_vs[cid]].sum() / flat.sum()).item()
                if (jsd_v[hh] < similarity_threshold and jsd_s[hh] < similarity_threshold
                        and self.vs_ratio[cid] < fallback_threshold):
                    sets[hh] = self.pivot_pattern[cid]
                    use_share[hh] = True

        nv = nv.clone(); ns = ns.clone()
        nv[use_qa | use_share] = min_blocks
        ns[use_qa | use_share] = min_blocks
        vpool_inf = vpool.clone(); vpool_inf[:, 0] = float("inf")
        spool_inf = spool.clone(); spool_inf[:, -1] = float("inf")
        kv = min(int(nv.max()), nb)
        ks = min(int(ns.max()), nb)
        vs_sets = []
        for hh in range(h):
            v_idx, s_idx = vs_lists(vpool_inf[hh], spool_inf[hh], int(nv[hh]), int(ns[hh]), kv, ks)
            vs = vs_multiset(v_idx, s_idx, nb)
            vs_sets.append(torch.unique(vs))
            sets[hh] = torch.unique(torch.cat((sets[hh], vs)))

        thr_sum = pattern_threshold * nb
        for hh in range(h):
            if not bool(use_qa[hh]) or (heads is not None and hh not in heads):
                continue
            sc = qa_scores[hh] if isinstance(qa_scores, dict) else qa_scores(hh)
            sets[hh] = torch.unique(torch.cat((sets[hh], cover_indices_global(sc, thr_sum))))

        if heads is not None:
            sets = [s_ if hh in heads else None for hh, s_ in enumerate(sets)]
        info = dict(nv=nv, ns=ns, vpool=vpool, spool=spool, jsd_qa=jsd_qa, use_qa=use_qa,
                    use_share=use_share, jsd_v=jsd_v, jsd_s=jsd_s, vs_sets=vs_sets)
        return sets, use_dense, info

    # ---- full selection from q/k
    def get_active_blocks(self, q, k, layer, *, block_size, min_blocks, max_blocks,
                          pattern_threshold=0.9, similarity_threshold=0.5,
                          fallback_threshold=0.9, queryaware_threshold=0.1):
        """q ``[N,H,D]``, k ``[N,Hkv,D]`` -> ``(block_sets, use_dense, info)``
        (attention_sharing.py:105-366)."""
        n, h, d = q.shape
        g = h // k.shape[1]
        vertical, slash = last_block_profile(q, k, block_size)
        avg_k = block_mean_pool(k, block_size)
        avg_qk = pooled_last_row(q, avg_k, block_size)

        def qa(hh):
            return query_aware_scores(q[:, hh, :], avg_k[:, hh // g, :], block_size)

        sets, use_dense, info = self.select_from_scores(
            layer, vertical, slash, avg_qk, qa,
            block_size=block_size, min_blocks=min_blocks, max_blocks=max_blocks,
            pattern_threshold=pattern_threshold, similarity_threshold=similarity_threshold,
            fallback_threshold=fallback_threshold, queryaware_threshold=queryaware_threshold)
        info.update(vertical=vertical, slash=slash, avg_k=avg_k, avg_qk=avg_qk)
        return sets, use_dense, info

    def update_pivots(self, layer: int, avg_attn: Dict[int, torch.Tensor], use_dense: torch.Tensor,
                      pattern_threshold: float = 0.9):
        """Store each new pivot's block-mass matrix ``[nb,nb]`` and its per-row cover
        pattern (attention_sharing.py:94-103).  ``avg_attn`` maps head -> matrix."""
        for hh in torch.nonzero(use_dense).flatten().tolist():
            cid = self.cluster(layer, hh)
            a = avg_attn[hh]
            self.pivot_attn[cid] = a
            self.pivot_pattern[cid] = cover_indices_rows(a, pattern_threshold)


# --------------------------------------------------------------------------- attention

def csr_row_offsets(sorted_idx: torch.Tensor, nb: int) -> torch.Tensor:
    """Row offsets ``[nb+1]`` of a sorted flat index list (shareprefill_attn.py:226-269)."""
    rows = torch.div(sorted_idx, nb, rounding_mode="floor")
    cnt = torch.bincount(rows[rows < nb], minlength=nb)
    return torch.cat((cnt.new_zeros(1), cnt.cumsum(0))).to(torch.int32)


def sparse_attention(q, k, v, block_sets: Sequence[torch.Tensor], use_dense, bs: int,
                     scale: Optional[float] = None, heads: Optional[Sequence[int]] = None,
                     rows: Optional[Sequence[int]] = None):
    """Block-sparse causal attention, restating the Triton kernel's arithmetic
    (shareprefill_attn.py:381-471): scores in fp32 times ``scale*log2(e)``,
    element-wise causal mask on every visited block, online softmax in base 2,
    probabilities rounded to the value dtype before P.V, fp32 accumulation,
    output rounded to the input dtype (bf16 in the reference).

    For heads flagged in ``use_dense`` a second pass writes, per visited block,
    the mean over the block's valid queries of the softmax mass landing in that
    key block (``:425-457``).

    q ``[N,H,D]``, k/v ``[N,Hkv,D]``.  Returns ``(o[N,H,D], {head: avg_attn[nb,nb]})``.
    ``heads`` / ``rows`` restrict the computation (other outputs stay zero).
    """
    n, h, d = q.shape
    g = h // k.shape[1]
    nb = -(-n // bs)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    qk_scale = scale * math.log2(math.e)
    o = torch.zeros(n, h, d, dtype=q.dtype)
    avg: Dict[int, torch.Tensor] = {}
    pos = torch.arange(n)
    for hh in (range(h) if heads is None else heads):
        idx = torch.sort(block_sets[hh]).values
        off = csr_row_offsets(idx, nb)
        qh = q[:, hh, :].float()
        kh = k[:, hh // g, :].float()
        vh = v[:, hh // g, :]
        dense = bool(use_dense[hh])
        if dense:
            avg[hh] = torch.zeros(nb, nb, dtype=torch.float32)
        for r in (range(nb) if rows is None else rows):
            r0, r1 = r * bs, min((r + 1) * bs, n)
            cols = (idx[off[r]:off[r + 1]] % nb).tolist()
            qt = qh[r0:r1]
            m_i = torch.full((r1 - r0,), float("-inf"))
            lse = torch.full((r1 - r0,), float("-inf"))
            acc = torch.zeros(r1 - r0, d, dtype=torch.float32)
            for c in cols:
                c0, c1 = c * bs, min((c + 1) * bs, n)
                s = (qt @ kh[c0:c1].T) * qk_scale
                s = s.masked_fill(pos[r0:r1, None] < pos[None, c0:c1], float("-inf"))
                m_new = torch.maximum(m_i, s.max(dim=1).values)
                p = torch.exp2(s - m_new[:, None])
                l_new = p.sum(dim=1)
                acc = acc * torch.exp2(m_i - m_new)[:, None]
                acc = acc + p.to(vh.dtype).float() @ vh[c0:c1].float()
                lse = m_new + torch.log2(torch.exp2(lse - m_new) + l_new)
                m_i = m_new
            if dense:
                for c in cols:
                    c0, c1 = c * bs, min((c + 1) * bs, n)
                    s = (qt @ kh[c0:c1].T) * qk_scale
                    s = s.masked_fill(pos[r0:r1, None] < pos[None, c0:c1], float("-inf"))
                    p = torch.exp2(s - lse[:, None])
                    avg[hh][r, c] = p.sum() / float(r1 - r0)
            o[r0:r1, hh, :] = (acc * torch.exp2(m_i - lse)[:, None]).to(q.dtype)
    return o, avg


def pivot_block_mass(q_h: torch.Tensor, k_h: torch.Tensor, bs: int, scale: Optional[float] = None) -> torch.Tensor:
    """Block-mass matrix ``[nb,nb]`` of one head that visits the full causal triangle: entry
    (r, c) is the mean over query block r's rows of the softmax mass landing in key block c
    (shareprefill_attn.py:425-457).  Same quantity as the ``use_dense`` pass of
    ``sparse_attention``, computed a query block at a time (one matrix product per row block)
    so that 32K- and 128K-token pivots finish in seconds; the row normaliser is a direct
    log-sum-exp instead of the online one (equal up to fp32 rounding).  ``q_h``/``k_h`` ``[N,D]``."""
    n, d = q_h.shape
    nb = -(-n // bs)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    qk_scale = scale * math.log2(math.e)
    qf, kf = q_h.float(), k_h.float()
    out = torch.zeros(nb, nb, dtype=torch.float32)
    pos = torch.arange(n)
    for r in range(nb):
        r0, r1 = r * bs, min((r + 1) * bs, n)
        s = (qf[r0:r1] @ kf[:r1].T) * qk_scale
        s = s.masked_fill(pos[r0:r1, None] < pos[None, :r1], float("-inf"))
        m = s.max(dim=1, keepdim=True).values
        lse = m + torch.log2(torch.exp2(s - m).sum(dim=1, keepdim=True))
        p = torch.exp2(s - lse).sum(dim=0)
        pad = (r + 1) * bs - r1
        if pad:
            p = torch.nn.functional.pad(p, (0, pad))
        out[r, :r + 1] = p.view(r + 1, bs).sum(-1) / float(r1 - r0)
    return out


def masked_dense_attention(q, k, v, block_sets, bs: int, scale: Optional[float] = None):
    """Plain fp32 softmax attention restricted to the selected blocks and the causal
    mask; an independent check on ``sparse_attention`` (no online update, no bf16 P)."""
    n, h, d = q.shape
    g = h // k.shape[1]
    nb = -(-n // bs)
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    o = torch.zeros(n, h, d, dtype=torch.float32)
    pos = torch.arange(n)
    for hh in range(h):
        bm = torch.zeros(nb * nb, dtype=torch.bool)
        bm[block_sets[hh]] = True
        mask = bm.view(nb, nb).repeat_interleave(bs, 0).repeat_interleave(bs, 1)[:n, :n]
        mask &= pos[:, None] >= pos[None, :]
        s = (q[:, hh].float() @ k[:, hh // g].float().T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        o[:, hh] = torch.softmax(s, dim=-1) @ v[:, hh // g].float()
    return o


def decode_attention(q, k, v, scale: Optional[float] = None):
    """One decode step: q ``[H,D]`` against the whole cache k/v ``[Nk,Hkv,D]``, fp32 softmax.
    The reference hands this step to flash_attn_func (attn/shareprefill_attn.py:146-153)."""
    h, d = q.shape
    g = h // k.shape[1]
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    kf = k.float().repeat_interleave(g, 1)
    vf = v.float().repeat_interleave(g, 1)
    s = torch.einsum("hd,nhd->hn", q.float(), kf) * scale
    return torch.einsum("hn,nhd->hd", torch.softmax(s, dim=-1), vf)


def sparse_prefill_layer(state: SharingOracle, q, k, v, layer: int, *, block_size=128,
                         min_budget=1024, max_budget=None, pattern_threshold=0.9,
                         similarity_threshold=0.5, fallback_threshold=0.9,
                         queryaware_threshold=0.1, scale=None):
    """One layer of the prefill path: selection, attention, pivot update
    (shareprefill_attn.py:110-144).  Returns ``(o, block_sets, use_dense, info)``."""
    min_budget = 1 if min_budget is None else min_budget
    max_budget = INT32_MAX if max_budget is None else max_budget
    sets, use_dense, info = state.get_active_blocks(
        q, k, layer, block_size=block_size,
        min_blocks=math.ceil(min_budget / block_size),
        max_blocks=math.ceil(max_budget / block_size),
        pattern_threshold=pattern_threshold, similarity_threshold=similarity_threshold,
        fallback_threshold=fallback_threshold, queryaware_threshold=queryaware_threshold)
    o, avg = sparse_attention(q, k, v, sets, use_dense, block_size, scale)
    state.update_pivots(layer, avg, use_dense, pattern_threshold)
    info["avg_attn"] = avg
    return o, sets, use_dense, info
