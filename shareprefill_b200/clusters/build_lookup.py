"""Offline generator of a head-cluster lookup.

The reference ships only the consumer of such a file (``AttentionSharing.load_clusters`` /
``find_cluster_id``, attn/attention_sharing.py:368-384) and one instance of it
(``clusters/sharing_lookup/Llama-3.1-8B-Instruct_code_debug_hiera-40.0-2.json``: hierarchical
clustering of the heads' attention patterns on one calibration task, a distance threshold and a
minimum cluster size in the name); the program that wrote it is not part of the reference.  This
module produces files of the same layout for other models:

1. *Signatures.*  For every (layer, head) the pooled vertical and slash profiles of the last query
   block - the quantities the run-time share test compares (attention_sharing.py:271-276) - taken
   with the library's own kernels and averaged over the calibration inputs.
2. *Distances.*  Pairwise sqrt-Jensen-Shannon divergence of the vertical profiles plus that of the
   slash profiles, all pairs on the GPU (``spf_pairwise_sqrt_jsd``).
3. *Clusters.*  Average-linkage agglomerative clustering cut at ``distance_threshold``.  Every
   (layer, head) ends up in exactly one cluster (the consumer fails on a missing pair); clusters with
   at least ``min_cluster_size`` members that span more than one layer are listed as shared - a
   pivot's pattern only becomes usable in later layers (attention_sharing.py:94-103, 265-295).

    python -m shareprefill_b200.clusters.build_lookup --model <hf model dir> --prompts <text file> \\
        --out lookup.json [--distance-threshold 0.3] [--min-cluster-size 2] [--length 8192]

The calibration forward needs a CUDA device; clustering and file writing run on the host.
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, Iterable, List, Sequence, Tuple

import numpy as np
import torch

from .. import native


def head_signatures(q: torch.Tensor, k: torch.Tensor, block_size: int) -> torch.Tensor:
    """Pooled vertical and slash profiles of every head of one layer: ``[H, 2, nb]`` fp32, rows sum
    to 1.  q ``[N,H,D]``, k ``[N,Hkv,D]`` bf16 on the GPU."""
    vertical, slash = native.lastblock_profile(q, k, block_size)
    nb = native.num_blocks(q.shape[0], block_size)
    _, _, vpool, spool = native.profile_budgets(vertical, slash, block_size, 0.9, 1, nb)
    return torch.stack((vpool, spool), dim=1)


def pairwise_distance(signatures: torch.Tensor) -> torch.Tensor:
    """``[P, 2, nb]`` signatures -> ``[P, P]`` distances (vertical sqrt-JSD + slash sqrt-JSD),
    symmetric, zero diagonal; a NaN divergence (an exact zero in a profile) counts as the maximum."""
    lib = native.load()
    p, two, nb = signatures.shape
    assert two == 2
    sig = signatures.to(torch.float32).contiguous()
    out = torch.zeros(p, p, dtype=torch.float32, device=sig.device)
    for part in range(2):
        x = sig[:, part].contiguous()
        d = torch.empty(p, p, dtype=torch.float32, device=sig.device)
        native._check(lib.spf_pairwise_sqrt_jsd(x.data_ptr(), p, nb, d.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream),
                      "spf_pairwise_sqrt_jsd")
        native._launched(1)
        out += torch.nan_to_num(d, nan=1.0)
    out = 0.5 * (out + out.T)
    out.fill_diagonal_(0.0)
    return out


def cluster_heads(distance: np.ndarray, pairs: Sequence[Tuple[int, int]], distance_threshold: float,
                  min_cluster_size: int = 2) -> dict:
    """Average-linkage clustering of the (layer, head) pairs; returns the lookup dictionary
    ``{"clusters": {id: [[layer, head], ...]}, "shared_clusters": [id, ...]}`` with ids ``"0"``, ``"1"``,
    ... in order of each cluster's first member."""
    from scipy.cluster.hierarchy import fcluster, linkage
    from scipy.spatial.distance import squareform
    n = len(pairs)
    assert distance.shape == (n, n)
    if n == 1:
        labels = np.array([1])
    else:
        z = linkage(squareform(np.asarray(distance, dtype=np.float64), checks=False), method="average")
        labels = fcluster(z, t=distance_threshold, criterion="distance")
    order: Dict[int, int] = {}
    clusters: Dict[str, List[List[int]]] = {}
    for (layer, head), lab in zip(pairs, labels):
        cid = str(order.setdefault(int(lab), len(order)))
        clusters.setdefault(cid, []).append([int(layer), int(head)])
    shared = [cid for cid, members in clusters.items()
              if len(members) >= min_cluster_size and len({m[0] for m in members}) > 1]
    return {"clusters": clusters, "shared_clusters": shared}


def build_lookup(layer_inputs: Iterable[Tuple[int, torch.Tensor, torch.Tensor]], block_size: int,
                 distance_threshold: float, min_cluster_size: int = 2) -> dict:
    """``layer_inputs`` yields ``(layer, q[N,H,D], k[N,Hkv,D])`` (possibly several times per layer, one
    per calibration input; all of one length).  Returns the lookup dictionary."""
    acc: Dict[int, torch.Tensor] = {}
    cnt: Dict[int, int] = {}
    for layer, q, k in layer_inputs:
        s = head_signatures(q, k, block_size)
        acc[layer] = s if layer not in acc else acc[layer] + s
        cnt[layer] = cnt.get(layer, 0) + 1
    layers = sorted(acc)
    sig = torch.cat([acc[layer] / cnt[layer] for layer in layers])
    pairs = [(layer, h) for layer in layers for h in range(acc[layer].shape[0])]
    dist = pairwise_distance(sig).cpu().numpy()
    return cluster_heads(dist, pairs, distance_threshold, min_cluster_size)


def write_lookup(path: str, lookup: dict) -> str:
    """Write the reference's JSON layout (attn/attention_sharing.py:368-378 reads it back)."""
    with open(path, "w") as f:
        json.dump({"clusters": lookup["clusters"], "shared_clusters": list(lookup["shared_clusters"])}, f)
    return path


def calibrate_model(model, input_ids_list: Sequence[torch.Tensor], block_size: int):
    """Run a Hugging Face decoder-only model over the calibration inputs and yield
    ``(layer, q, k)`` after RoPE for every attention layer, by registering a recording attention
    function the way ``SharePrefill`` registers its own."""
    import importlib
    records: List[Tuple[int, torch.Tensor, torch.Tensor]] = []
    attention_cls = model.model.layers[0].self_attn.__class__
    module = importlib.import_module(attention_cls.__module__)
    functions = getattr(module, "ALL_ATTENTION_FUNCTIONS")
    previous = model.config._attn_implementation

    def recorder(attn_module, query, key, value, attention_mask, **kwargs):
        records.append((attn_module.layer_idx, query[0].transpose(0, 1).contiguous(),
                        key[0].transpose(0, 1).contiguous()))
        return functions["sdpa"](attn_module, query, key, value, attention_mask, **kwargs)

    functions["spf_calibration_recorder"] = recorder
    model.config._attn_implementation = "spf_calibration_recorder"
    try:
        with torch.no_grad():
            for ids in input_ids_list:
                records.clear()
                model(ids, logits_to_keep=1)
                for rec in records:
                    yield rec
    finally:
        model.config._attn_implementation = previous
        functions.pop("spf_calibration_recorder", None)


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="Hugging Face model directory")
    ap.add_argument("--prompts", required=True, help="text file; its token stream is cut into calibration inputs")
    ap.add_argument("--out", required=True)
    ap.add_argument("--length", type=int, default=8192)
    ap.add_argument("--num-inputs", type=int, default=4)
    ap.add_argument("--block-size", type=int, default=128)
    ap.add_argument("--distance-threshold", type=float, default=0.3)
    ap.add_argument("--min-cluster-size", type=int, default=2)
    a = ap.parse_args()
    from transformers import AutoModelForCausalLM, AutoTokenizer
    tok = AutoTokenizer.from_pretrained(a.model)
    model = AutoModelForCausalLM.from_pretrained(a.model, torch_dtype=torch.bfloat16).cuda().eval()
    with open(a.prompts) as f:
        ids = tok(f.read(), return_tensors="pt").input_ids[0]
    reps = -(-a.length * a.num_inputs // ids.numel())
    ids = ids.repeat(reps)[: a.length * a.num_inputs].view(a.num_inputs, 1, a.length).cuda()
    lookup = build_lookup(calibrate_model(model, list(ids), a.block_size), a.block_size,
                          a.distance_threshold, a.min_cluster_size)
    write_lookup(a.out, lookup)
    print(f"{len(lookup['clusters'])} clusters, {len(lookup['shared_clusters'])} shared -> {a.out}")


if __name__ == "__main__":
    main()
