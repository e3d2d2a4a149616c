"""The offline head-cluster lookup generator: clustering and file layout on the CPU, signatures and
pairwise divergences on the GPU."""
import json

import numpy as np
import pytest
import torch

from shareprefill_b200.clusters import build_lookup as bl
from shareprefill_b200.sharing_state import AttentionSharing, load_lookup


def _planted_distance(labels, within=0.05, across=0.6, seed=0):
    rng = np.random.default_rng(seed)
    n = len(labels)
    d = np.where(np.equal.outer(labels, labels), within, across) + rng.uniform(0, 0.02, (n, n))
    d = 0.5 * (d + d.T)
    np.fill_diagonal(d, 0.0)
    return d


def test_clustering_recovers_planted_groups_and_round_trips(tmp_path):
    layers, heads = 3, 8
    pairs = [(layer, h) for layer in range(layers) for h in range(heads)]
    # heads 0-2 of every layer alike, heads 3-4 alike, head 5 alike only within layer 0, 6 and 7 alone
    labels = np.array([0 if h < 3 else 1 if h < 5 else 100 + 10 * layer + h for layer, h in pairs])
    lookup = bl.cluster_heads(_planted_distance(labels), pairs, distance_threshold=0.3, min_cluster_size=2)
    got = {}
    for cid, members in lookup["clusters"].items():
        for layer, h in members:
            got[(layer, h)] = cid
    assert set(got) == set(pairs), "every (layer, head) must be in exactly one cluster"
    for a in range(len(pairs)):
        for b in range(len(pairs)):
            assert (got[pairs[a]] == got[pairs[b]]) == (labels[a] == labels[b])
    # shared: the two groups that span several layers; singletons are clusters but not shared
    assert sorted(lookup["shared_clusters"]) == sorted({got[(0, 0)], got[(0, 3)]})
    path = bl.write_lookup(str(tmp_path / "lookup.json"), lookup)
    clusters, shared = load_lookup(path)
    assert clusters == lookup["clusters"] and shared == set(lookup["shared_clusters"])
    sharing = AttentionSharing(path)
    assert sharing.find_cluster_id(2, 1) == got[(2, 1)]
    assert json.load(open(path)).keys() == {"clusters", "shared_clusters"}


def test_single_layer_clusters_are_not_shared():
    pairs = [(0, h) for h in range(4)]
    lookup = bl.cluster_heads(_planted_distance(np.array([0, 0, 1, 1])), pairs, 0.3, 2)
    assert len(lookup["clusters"]) == 2 and lookup["shared_clusters"] == []


@pytest.mark.gpu
def test_pairwise_divergence_matches_torch():
    g = torch.Generator().manual_seed(1)
    sig = torch.rand(37, 2, 100, generator=g)
    sig /= sig.sum(-1, keepdim=True)
    got = bl.pairwise_distance(sig.cuda()).cpu()

    def jsd(p, q):
        m = (p + q) / 2
        return torch.sqrt(0.5 * (p * torch.log(p / m)).sum(-1) + 0.5 * (q * torch.log(q / m)).sum(-1))

    want = sum(jsd(sig[:, None, part], sig[None, :, part]) for part in range(2))
    want.fill_diagonal_(0.0)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
def test_generator_recovers_the_head_groups_planted_in_synthetic_inputs():
    """Synthetic layers whose heads come in four planted clusters (a shared low-rank component per
    cluster, the same input for every layer so that clusters span layers): heads that the generator
    puts together always belong to one planted cluster, every cluster it calls shared spans layers, and
    the file drives a sparse-prefill layer."""
    from shareprefill_b200.workloads import AttentionWorkload, make_qkv
    wl = AttentionWorkload("lookup_gen", 60, 4096, 16, 4, num_layers=3, num_head_clusters=4, shared_rank=8,
                           rope_theta=500000.0, q_gain=2.0)
    q, k, _ = make_qkv(wl, 0)                 # drawn on the CPU: the seed then names one input everywhere
    q, k = q.cuda(), k.cuda()
    lookup = bl.build_lookup(((layer, q, k) for layer in range(wl.num_layers)), wl.block_size,
                             distance_threshold=0.29, min_cluster_size=2)
    planted = lambda h: (h // wl.group_size) % wl.num_head_clusters  # noqa: E731
    seen = set()
    for cid, members in lookup["clusters"].items():
        assert len({planted(h) for _, h in members}) == 1, f"cluster {cid} mixes planted clusters"
        seen.update((layer, h) for layer, h in members)
    assert len(seen) == wl.num_layers * wl.num_q_heads
    # identical inputs in every layer: a head's copies in the three layers are at distance 0
    for cid, members in lookup["clusters"].items():
        assert {layer for layer, _ in members} == set(range(wl.num_layers))
    assert sorted(lookup["shared_clusters"]) == sorted(lookup["clusters"])
    assert len(lookup["clusters"]) < wl.num_q_heads, "no two heads were put together"
