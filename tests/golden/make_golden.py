"""Generate golden vectors by running the reference's own selection code on CPU.

Run in a container that has the reference checkout (it cannot travel):

    python tests/golden/make_golden.py --reference <path to the reference checkout>

The reference's ``AttentionSharing.get_active_blocks`` / ``update_pivotal_attns``
(shareprefill/attn/attention_sharing.py:94-366) and their helpers
(shareprefill/attn/utils.py) run unmodified.  Three things are supplied from the
outside, none touching reference files:

* the literal device string ``"cuda"`` in ``torch.empty(..., device="cuda")`` and
  ``Tensor.to("cuda")`` is mapped to CPU while the reference runs;
* ``triton_bnhd_pool`` (a Triton kernel) is rebound to a torch block mean;
* the block-sparse attention kernel (Triton, GPU only) is replaced by the oracle's
  restatement, which is what feeds ``avg_attn`` into ``update_pivotal_attns``.
  The ``avg_attn`` matrices stored here are therefore oracle outputs, not reference
  outputs; everything else in the files is reference output.

Stage-boundary tensors are captured by wrapping the helper names inside the
``attention_sharing`` module namespace (it imports them by name, :23-32).

Two families of files are written.  The small multi-layer cases (``CASES``) keep every
intermediate of every head.  The cases at the sizes and head layouts of the benchmark
configurations (``SCALE_CASES``: 8K tokens with 8q/2kv and 28q/4kv heads, 32K tokens with
32q/8kv heads on the shipped Llama-3.1-8B lookup, 128K tokens with one KV group) keep the
reference's RESULTS for every head (block bitmaps, flags, cover counts, divergences, pooled
profiles) and its un-pooled score tensors only for the heads listed in ``score_heads``
(``None`` = every head), which bounds the file size: a head's vertical + slash profiles are
1 MiB at 128K tokens and a query-aware head's pooled score matrix 4 MiB.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import spf_oracle as orc  # noqa: E402
from oracle.reference_shim import cuda_string_to_cpu  # noqa: E402
from shareprefill_b200.workloads import AttentionWorkload, make_qkv, synthetic_lookup  # noqa: E402


def tensor_digest(*ts) -> str:
    hsh = hashlib.sha256()
    for t in ts:
        hsh.update(t.contiguous().view(torch.uint8).numpy().tobytes())
    return hsh.hexdigest()


CASES = {
    # name: (workload, lookup kwargs, layers, description)
    "peaky_share": dict(
        wl=AttentionWorkload("peaky_share", 90, 1024, 4, 2, head_dim=64, num_layers=3,
                             num_head_clusters=2, shared_rank=4, block_size=64, min_budget=128,
                             pattern_threshold=0.9, fallback_threshold=1e9, q_gain=3.0),
        lookup=dict(num_clusters=2, shared=[0, 1]),
    ),
    "peaky_default": dict(
        wl=AttentionWorkload("peaky_default", 91, 2048, 8, 2, head_dim=128, num_layers=3,
                             num_head_clusters=2, shared_rank=4, block_size=128, min_budget=256,
                             pattern_threshold=0.95, q_gain=2.5),
        lookup=dict(num_clusters=2, shared=[1]),
    ),
    "diffuse_qa": dict(
        wl=AttentionWorkload("diffuse_qa", 92, 2048, 8, 2, head_dim=128, num_layers=2,
                             num_head_clusters=2, shared_rank=4, block_size=128, min_budget=256,
                             pattern_threshold=0.95, queryaware_threshold=0.3),
        lookup=dict(num_clusters=2, shared=[0, 1]),
    ),
    "ragged_rope": dict(
        wl=AttentionWorkload("ragged_rope", 93, 1000, 6, 2, head_dim=64, num_layers=3,
                             num_head_clusters=2, shared_rank=4, block_size=64, min_budget=192,
                             rope_theta=500000.0, pattern_threshold=0.9, fallback_threshold=1e9,
                             q_gain=2.0, similarity_threshold=0.9),
        lookup=dict(num_clusters=2, shared=[0]),
    ),
}


def run_case(name, spec, refmod):
    wl: AttentionWorkload = spec["wl"]
    lookup = synthetic_lookup(wl.num_layers, wl.num_q_heads, group_size=wl.group_size, **spec["lookup"])
    lookup_path = os.path.join(HERE, f"_{name}_lookup.json")
    with open(lookup_path, "w") as f:
        json.dump(lookup, f)
    att = refmod
    ref_state = att.AttentionSharing(lookup_path)
    os.remove(lookup_path)

    bs, nb = wl.block_size, wl.num_blocks
    mb = math.ceil(wl.min_budget / bs)
    xb = math.ceil((2**31 - 1 if wl.max_budget is None else wl.max_budget) / bs)
    g = wl.group_size
    out = {"meta": json.dumps(dict(name=name, workload=wl.__dict__, lookup=lookup))}

    for layer in range(wl.num_layers):
        q, k, v = make_qkv(wl, layer, dtype=torch.bfloat16)
        out[f"L{layer}_digest"] = np.frombuffer(bytes.fromhex(tensor_digest(q, k, v)), dtype=np.uint8)
        rec = {"jsd": [], "cover_idx": [], "sumpool": []}

        real = {n: getattr(att, n) for n in
                ("square_root_js_divergence", "score_cover_idx", "torch_bhn_sumpool")}

        def jsd(p, qq):
            rec["jsd"].append((p.detach().clone(), qq.detach().clone()))
            return real["square_root_js_divergence"](p, qq)

        def cover_idx(x, score, padding_value=0):
            rec["cover_idx"].append(x.detach().clone())
            return real["score_cover_idx"](x, score, padding_value)

        def sumpool(x, ks):
            rec["sumpool"].append(x.detach().clone())
            return real["torch_bhn_sumpool"](x, ks)

        def pool(x, ks, pool_type="avg"):
            return orc.block_mean_pool(x[0], ks)[None]

        att.square_root_js_divergence = jsd
        att.score_cover_idx = cover_idx
        att.torch_bhn_sumpool = sumpool
        att.triton_bnhd_pool = pool
        try:
            with cuda_string_to_cpu():
                k_rep = k.repeat_interleave(g, dim=1)
                block_idx, use_dense = ref_state.get_active_blocks(
                    q[None].contiguous(), k_rep[None].contiguous(), layer, wl.num_q_heads, bs, mb, xb,
                    wl.pattern_threshold, wl.similarity_threshold, wl.fallback_threshold,
                    wl.queryaware_threshold, False)
        finally:
            for n, f in real.items():
                setattr(att, n, f)

        sets = [block_idx[0][h].to(torch.int64) for h in range(wl.num_q_heads)]
        use_dense = use_dense[0]
        vertical, slash = rec["sumpool"][0][0], rec["sumpool"][1][0]     # [H,N] fp32, un-pooled
        avg_qk = rec["jsd"][0][0][0]                                       # [H,nb]
        use_qa = real["square_root_js_divergence"](rec["jsd"][0][0], rec["jsd"][0][1])[0] < wl.queryaware_threshold
        qa_heads = torch.nonzero(use_qa).flatten().tolist()
        assert len(qa_heads) == len(rec["cover_idx"])

        o, avg = orc.sparse_attention(q, k, v, sets, use_dense, bs)
        avg_full = torch.zeros(1, wl.num_q_heads, nb, nb)
        for h, a in avg.items():
            avg_full[0, h] = a
        with cuda_string_to_cpu():
            ref_state.update_pivotal_attns(layer, avg_full, use_dense[None], wl.pattern_threshold)

        pre = f"L{layer}_"
        out[pre + "set_len"] = np.array([len(s) for s in sets], dtype=np.int64)
        out[pre + "set_cat"] = torch.cat(sets).numpy()
        out[pre + "use_dense"] = use_dense.numpy()
        out[pre + "use_qa"] = use_qa.numpy()
        out[pre + "vertical"] = vertical.numpy()
        out[pre + "slash"] = slash.numpy()
        out[pre + "avg_qk"] = avg_qk.numpy()
        out[pre + "qa_heads"] = np.array(qa_heads, dtype=np.int64)
        if qa_heads:
            out[pre + "qa_scores"] = torch.stack(rec["cover_idx"]).numpy()
        out[pre + "dense_heads"] = np.array(sorted(avg.keys()), dtype=np.int64)
        if avg:
            out[pre + "avg_attn"] = torch.stack([avg[h] for h in sorted(avg.keys())]).numpy()
        print(f"{name} L{layer}: dense={torch.nonzero(use_dense).flatten().tolist()} qa={qa_heads} "
              f"density={[round(len(s) / (nb * (nb + 1) / 2), 3) for s in sets]}")

    # state at the end of the forward
    for cid in lookup["shared_clusters"]:
        ph = ref_state.pivotal_heads[cid][0]
        out[f"S{cid}_pivot_head"] = np.array(-1 if ph is None else int(ph), dtype=np.int64)
        pat = ref_state.pivotal_patterns[cid][0]
        if pat is not None:
            out[f"S{cid}_pattern"] = pat.numpy()
        r = ref_state.pivotal_vs_ratio[cid][0]
        out[f"S{cid}_vs_ratio"] = np.array(float("nan") if r is None else r, dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)


SHIPPED_LOOKUP = "shareprefill/clusters/sharing_lookup/Llama-3.1-8B-Instruct_code_debug_hiera-40.0-2.json"

SCALE_CASES = {
    # 8K tokens, the 8q/2kv head layout: every head query-aware (64 blocks: the 16-byte path of the
    # query-aware cover kernel)
    "qa_8k": dict(
        wl=AttentionWorkload("qa_8k", 94, 8192, 8, 2, num_layers=2, num_head_clusters=2, shared_rank=4,
                             q_gain=0.5),
        lookup=dict(num_clusters=2, shared=[0, 1]), layers=[0, 1], score_heads=None),
    # the same layout with a query-aware threshold that splits the heads: query-aware heads, pivots and
    # shared heads in one layer stack
    "mixed_8k": dict(
        wl=AttentionWorkload("mixed_8k", 95, 8192, 8, 2, num_layers=3, num_head_clusters=2, shared_rank=4,
                             queryaware_threshold=0.17, fallback_threshold=1e9, similarity_threshold=0.9),
        lookup=dict(num_clusters=2, shared=[0, 1]), layers=[0, 1, 2], score_heads=None),
    # Qwen2.5-7B head layout: 28 query / 4 KV heads (groups of 7), min_budget 2048, RoPE theta 1e6
    "qwen_8k": dict(
        wl=AttentionWorkload("qwen_8k", 96, 8192, 28, 4, num_layers=2, rope_theta=1e6, min_budget=2048,
                             queryaware_threshold=0.18, fallback_threshold=1e9, similarity_threshold=0.9),
        lookup=dict(num_clusters=4, shared=[1, 2]), layers=[0, 1], score_heads=None),
    # Llama-3.1-8B layout at 32K tokens on the shipped lookup: layer 14 elects head 17 pivot of the shared
    # cluster "9", layer 17 tests heads 16 and 17 against it.  Scores are kept for KV group 4 (heads 16-19).
    "llama_32k": dict(
        wl=AttentionWorkload("llama_32k", 97, 32768, 32, 8, num_layers=18, rope_theta=500000.0, q_gain=2.0,
                             fallback_threshold=1e9, similarity_threshold=0.9),
        lookup="shipped", layers=[14, 17], score_heads=[16, 17, 18, 19]),
    # the same layout, diffuse inputs and a query-aware threshold that splits the heads
    "llama_32k_diffuse": dict(
        wl=AttentionWorkload("llama_32k_diffuse", 98, 32768, 32, 8, num_layers=15, rope_theta=500000.0,
                             queryaware_threshold=0.15),
        lookup="shipped", layers=[14], score_heads=[16, 17, 18, 19]),
    # Llama-3.1-70B head layout (64 query / 8 KV heads, groups of 8) at 8K tokens; scores kept for KV group 1,
    # whose first head becomes the pivot of shared cluster 1
    "llama70b_8k": dict(
        wl=AttentionWorkload("llama70b_8k", 100, 8192, 64, 8, num_layers=2, rope_theta=500000.0,
                             queryaware_threshold=0.17, fallback_threshold=1e9, similarity_threshold=0.9),
        lookup=dict(num_clusters=4, shared=[1]), layers=[0, 1], score_heads=[8, 9, 10, 11, 12, 13, 14, 15]),
    # 128K tokens, one KV group of four query heads; the threshold makes exactly one of them query-aware
    "group_128k": dict(
        wl=AttentionWorkload("group_128k", 99, 131072, 4, 1, num_layers=1, num_head_clusters=1,
                             rope_theta=500000.0, queryaware_threshold=0.13),
        lookup=dict(num_clusters=1, shared=[]), layers=[0], score_heads=None),
}


def sets_to_bitmap_np(sets, nb):
    """Per-head sorted flat indices -> uint32 ``[H][nb][ceil(nb/32)]`` bitmaps (bit c%32 of word c//32)."""
    nbw = (nb + 31) // 32
    out = np.zeros((len(sets), nb, nbw * 32), dtype=bool)
    for h, s in enumerate(sets):
        s = s.numpy()
        out[h, s // nb, s % nb] = True
    w = out.reshape(len(sets), nb, nbw, 32).astype(np.uint64) << np.arange(32, dtype=np.uint64)
    return w.sum(-1).astype(np.uint32)


def run_scale_case(name, spec, att, reference_root):
    wl: AttentionWorkload = spec["wl"]
    layers = spec["layers"]
    if spec["lookup"] == "shipped":
        lookup_path = os.path.join(reference_root, SHIPPED_LOOKUP)
        lookup_meta = "shipped"
    else:
        lookup_meta = synthetic_lookup(wl.num_layers, wl.num_q_heads, group_size=wl.group_size, **spec["lookup"])
        lookup_path = os.path.join(HERE, f"_{name}_lookup.json")
        with open(lookup_path, "w") as f:
            json.dump(lookup_meta, f)
    ref_state = att.AttentionSharing(lookup_path)
    if lookup_meta != "shipped":
        os.remove(lookup_path)

    bs, nb, H, g = wl.block_size, wl.num_blocks, wl.num_q_heads, wl.group_size
    mb = math.ceil(wl.min_budget / bs)
    xb = math.ceil((2**31 - 1 if wl.max_budget is None else wl.max_budget) / bs)
    score_heads = list(range(H)) if spec["score_heads"] is None else list(spec["score_heads"])
    out = {"meta": json.dumps(dict(name=name, workload=wl.__dict__, lookup=lookup_meta, layers=layers,
                                   score_heads=score_heads))}

    for layer in layers:
        q, k, v = make_qkv(wl, layer, dtype=torch.bfloat16)
        out[f"L{layer}_digest"] = np.frombuffer(bytes.fromhex(tensor_digest(q, k, v)), dtype=np.uint8)
        rec = {"jsd": [], "jsd_out": [], "cover_idx": [], "sumpool": [], "sumpool_out": [], "topk": []}
        names = ("square_root_js_divergence", "score_cover_idx", "torch_bhn_sumpool", "score_cover_topk")
        real = {n: getattr(att, n) for n in names}

        def jsd(p, qq):
            r = real["square_root_js_divergence"](p, qq)
            rec["jsd"].append((p.detach().clone(), qq.detach().clone()))
            rec["jsd_out"].append(r.detach().clone())
            return r

        def cover_idx(x, score, padding_value=0):
            rec["cover_idx"].append(x.detach().clone())
            return real["score_cover_idx"](x, score, padding_value)

        def sumpool(x, ks):
            r = real["torch_bhn_sumpool"](x, ks)
            rec["sumpool"].append(x.detach().clone())
            rec["sumpool_out"].append(r.detach().clone())
            return r

        def cover_topk(x, score):
            r = real["score_cover_topk"](x, score)
            rec["topk"].append(r.detach().clone())
            return r

        def pool(x, ks, pool_type="avg"):
            return orc.block_mean_pool(x[0], ks)[None]

        att.square_root_js_divergence, att.score_cover_idx = jsd, cover_idx
        att.torch_bhn_sumpool, att.score_cover_topk, att.triton_bnhd_pool = sumpool, cover_topk, pool
        try:
            with cuda_string_to_cpu():
                k_rep = k.repeat_interleave(g, dim=1)
                block_idx, use_dense = ref_state.get_active_blocks(
                    q[None].contiguous(), k_rep[None].contiguous(), layer, H, bs, mb, xb,
                    wl.pattern_threshold, wl.similarity_threshold, wl.fallback_threshold,
                    wl.queryaware_threshold, False)
        finally:
            for n, f in real.items():
                setattr(att, n, f)
        del k_rep

        sets = [block_idx[0][h].to(torch.int64) for h in range(H)]
        use_dense = use_dense[0]
        vertical, slash = rec["sumpool"][0][0], rec["sumpool"][1][0]          # [H,N] fp32, un-pooled
        vpool, spool = rec["sumpool_out"][0][0], rec["sumpool_out"][1][0]     # [H,nb]
        avg_qk = rec["jsd"][0][0][0]                                           # [H,nb]
        jsd_qa = rec["jsd_out"][0][0]                                          # [H]
        use_qa = jsd_qa < wl.queryaware_threshold
        qa_heads = torch.nonzero(use_qa).flatten().tolist()
        assert len(qa_heads) == len(rec["cover_idx"])
        # raw cover counts (score_cover_topk is called for vertical, then for slash: attention_sharing.py:169-172)
        cover_v, cover_s = rec["topk"][0][0], rec["topk"][1][0]

        dense = torch.nonzero(use_dense).flatten().tolist()
        avg_full = torch.zeros(1, H, nb, nb)
        for h in dense:
            avg_full[0, h] = orc.pivot_block_mass(q[:, h], k[:, h // g], bs)
        with cuda_string_to_cpu():
            ref_state.update_pivotal_attns(layer, avg_full, use_dense[None], wl.pattern_threshold)

        pre = f"L{layer}_"
        out[pre + "bitmap"] = sets_to_bitmap_np(sets, nb)
        out[pre + "use_dense"] = use_dense.numpy()
        out[pre + "use_qa"] = use_qa.numpy()
        out[pre + "jsd_qa"] = jsd_qa.numpy()
        out[pre + "cover_v"] = cover_v.numpy()
        out[pre + "cover_s"] = cover_s.numpy()
        out[pre + "avg_qk"] = avg_qk.numpy()
        out[pre + "vpool"] = vpool.numpy()
        out[pre + "spool"] = spool.numpy()
        out[pre + "vertical"] = vertical[score_heads].numpy()
        out[pre + "slash"] = slash[score_heads].numpy()
        out[pre + "qa_heads"] = np.array(qa_heads, dtype=np.int64)
        kept = [h for h in qa_heads if h in score_heads]
        out[pre + "qa_score_heads"] = np.array(kept, dtype=np.int64)
        if kept:
            out[pre + "qa_scores"] = torch.stack([rec["cover_idx"][qa_heads.index(h)] for h in kept]).numpy()
        out[pre + "dense_heads"] = np.array(dense, dtype=np.int64)
        if dense:
            out[pre + "avg_attn"] = avg_full[0, dense].numpy()
        tri = nb * (nb + 1) / 2
        print(f"{name} L{layer}: dense={dense} qa={qa_heads} "
              f"density={[round(len(s) / tri, 3) for s in sets]}")

    shared = sorted(ref_state.shared_clusters)
    out["shared_ids"] = np.array([int(c) for c in shared], dtype=np.int64)
    for cid in shared:
        ph = ref_state.pivotal_heads[cid][0]
        out[f"S{cid}_pivot_head"] = np.array(-1 if ph is None else int(ph), dtype=np.int64)
        pat = ref_state.pivotal_patterns[cid][0]
        if pat is not None:
            out[f"S{cid}_pattern"] = sets_to_bitmap_np([pat.to(torch.int64)], nb)[0]
        r = ref_state.pivotal_vs_ratio[cid][0]
        out[f"S{cid}_vs_ratio"] = np.array(float("nan") if r is None else r, dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)


def tie_vectors(utils):
    """Query-aware cover rule (score_cover_idx, utils.py:53-57) on pooled score matrices whose values
    repeat, so that the value at which the running sum crosses the threshold is shared by several
    blocks.  The kept set then depends on the sort's tie order; torch's CPU sort keeps equal values in
    index order (lowest first), which is the order recorded here."""
    g = torch.Generator().manual_seed(23)
    out = {}
    for nb in (64, 80, 96):
        logits = torch.randn(nb, nb, generator=g) * 1.5
        logits.masked_fill_(~torch.tril(torch.ones(nb, nb, dtype=torch.bool)), float("-inf"))
        p = torch.softmax(logits, dim=-1)
        p = torch.round(p * 256.0) / 256.0          # 8-bit values: long runs of equal scores
        for thr in (0.5, 0.9, 0.95):
            kept = utils.score_cover_idx(p.reshape(-1), thr * nb)
            out[f"tie{nb}_scores"] = p.numpy()
            out[f"tie{nb}_kept_{thr}"] = torch.unique(kept).numpy()
    np.savez_compressed(os.path.join(HERE, "qa_ties.npz"), **out)


def helper_vectors(utils):
    """Known-answer vectors for the look-alike cover rules and the other helpers."""
    g = torch.Generator().manual_seed(7)
    out = {}
    x = torch.rand(6, 333, generator=g)
    x = x ** 4
    x = x / x.sum(-1, keepdim=True)
    out["cover_x"] = x.numpy()
    for thr in (0.5, 0.9, 0.95):
        out[f"cover_topk_{thr}"] = utils.score_cover_topk(x, thr).numpy()
        out[f"cover_rows_{thr}"] = utils.score_cover_idx_each_row(x, thr).numpy()
        out[f"cover_global_{thr}"] = utils.score_cover_idx(x.reshape(-1), thr * 6).numpy()
    p = torch.rand(5, 40, generator=g); p /= p.sum(-1, keepdim=True)
    q = torch.rand(5, 40, generator=g); q /= q.sum(-1, keepdim=True)
    q[4, 3] = 0.0
    out["jsd_p"], out["jsd_q"] = p.numpy(), q.numpy()
    out["jsd"] = utils.square_root_js_divergence(p, q).numpy()
    m = torch.rand(1, 3, 16, 100, generator=g)
    out["diag_in"] = m.numpy()
    out["diag_out"] = utils.sum_all_diagonal_matrix(m).numpy()
    out["sumpool_out"] = utils.torch_bhn_sumpool(m[0], 16).numpy()
    v = torch.tensor([[[0, 3, 5]]]); s = torch.tensor([[[0, 2]]])
    out["vs_v"], out["vs_s"] = v.numpy(), s.numpy()
    out["vs_out"] = utils.combine_vertical_slash_indices(v, s, 7).numpy()
    np.savez_compressed(os.path.join(HERE, "helpers.npz"), **out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path to the reference checkout")
    ap.add_argument("--only", default=None)
    ap.add_argument("--family", default="all", choices=["all", "small", "scale"])
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import importlib
    att = importlib.import_module("shareprefill.attn.attention_sharing")
    utils = importlib.import_module("shareprefill.attn.utils")
    torch.manual_seed(0)
    if args.family in ("all", "small"):
        helper_vectors(utils)
        for name, spec in CASES.items():
            if args.only and name != args.only:
                continue
            run_case(name, spec, att)
    if args.family in ("all", "scale"):
        if not args.only:
            tie_vectors(utils)
        for name, spec in SCALE_CASES.items():
            if args.only and name != args.only:
                continue
            run_scale_case(name, spec, att, args.reference)


if __name__ == "__main__":
    main()
