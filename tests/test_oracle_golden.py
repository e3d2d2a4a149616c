"""The CPU oracle against vectors produced by the reference's own code (CPU run)."""
import numpy as np
import pytest
import torch

from oracle import spf_oracle as orc
from golden_cases import CASE_NAMES, GOLDEN_DIR, GoldenCase


@pytest.fixture(scope="module")
def helpers():
    return np.load(f"{GOLDEN_DIR}/helpers.npz")


def test_cover_rules(helpers):
    x = torch.from_numpy(helpers["cover_x"])
    for thr in (0.5, 0.9, 0.95):
        assert torch.equal(orc.cover_count(x, thr), torch.from_numpy(helpers[f"cover_topk_{thr}"]))
        assert torch.equal(orc.cover_indices_rows(x, thr), torch.from_numpy(helpers[f"cover_rows_{thr}"]))
        ref = torch.unique(torch.from_numpy(helpers[f"cover_global_{thr}"]))
        assert torch.equal(orc.cover_indices_global(x.reshape(-1), thr * 6), ref)


def test_cover_rules_textbook_example():
    # crossing element: included by the count rule and the per-row rule, excluded by the global rule
    x = torch.tensor([0.5, 0.3, 0.15, 0.05])
    assert int(orc.cover_count(x, 0.9)) == 3
    assert orc.cover_indices_global(x, 0.9).tolist() == [0, 1]
    assert orc.cover_indices_rows(x[None], 0.9).tolist() == [0, 1, 2]


def test_jsd_and_nan(helpers):
    p, q = torch.from_numpy(helpers["jsd_p"]), torch.from_numpy(helpers["jsd_q"])
    got = orc.sqrt_jsd(p, q)
    want = torch.from_numpy(helpers["jsd"])
    assert torch.isnan(got[4]) and torch.isnan(want[4])
    assert torch.equal(got[:4], want[:4])


def test_diagonal_and_pool(helpers):
    m = torch.from_numpy(helpers["diag_in"])
    torch.testing.assert_close(orc.antidiagonal_sums(m), torch.from_numpy(helpers["diag_out"]),
                               rtol=1e-6, atol=1e-6)
    assert torch.equal(orc.block_sum_pool(m[0], 16), torch.from_numpy(helpers["sumpool_out"]))


def test_vs_multiset(helpers):
    v = torch.from_numpy(helpers["vs_v"])[0, 0]
    s = torch.from_numpy(helpers["vs_s"])[0, 0]
    assert torch.equal(orc.vs_multiset(v, s, 7), torch.from_numpy(helpers["vs_out"])[0, 0])


@pytest.mark.parametrize("name", CASE_NAMES)
def test_selection_from_recorded_scores_is_exact(name):
    """Identical pooled scores in -> identical block sets, flags and pivot state out."""
    gc = GoldenCase(name)
    st = orc.SharingOracle(gc.lookup)
    for layer in range(gc.wl.num_layers):
        sets, use_dense, info = st.select_from_scores(
            layer, gc.t(f"L{layer}_vertical"), gc.t(f"L{layer}_slash"), gc.t(f"L{layer}_avg_qk"),
            gc.qa_scores(layer), **gc.knobs())
        assert torch.equal(use_dense, gc.t(f"L{layer}_use_dense"))
        assert torch.equal(info["use_qa"], gc.t(f"L{layer}_use_qa"))
        for h, (a, b) in enumerate(zip(sets, gc.sets(layer))):
            assert torch.equal(a, b), f"layer {layer} head {h}"
        st.update_pivots(layer, gc.avg_attn(layer), use_dense, gc.wl.pattern_threshold)
    for cid in gc.lookup["shared_clusters"]:
        ph = int(gc.z[f"S{cid}_pivot_head"])
        assert st.pivot_head.get(cid, -1) == ph
        if gc.has(f"S{cid}_pattern"):
            assert torch.equal(st.pivot_pattern[cid], gc.t(f"S{cid}_pattern"))
        r = float(gc.z[f"S{cid}_vs_ratio"])
        if r == r:
            assert st.vs_ratio[cid] == r


@pytest.mark.parametrize("name", CASE_NAMES)
def test_profiles_from_qk_match_reference(name):
    """vertical / slash / pooled last-row estimate computed by the oracle from q,k."""
    gc = GoldenCase(name)
    q, k, _ = gc.qkv(0)
    vertical, slash = orc.last_block_profile(q, k, gc.bs)
    # the bf16 GEMM's accumulation order differs between einsum and matmul: a handful of
    # logits round to the neighbouring bf16 value, hence a tolerance on the profiles
    torch.testing.assert_close(vertical, gc.t("L0_vertical"), rtol=2e-2, atol=1e-6)
    torch.testing.assert_close(slash, gc.t("L0_slash"), rtol=2e-2, atol=1e-6)
    avg_k = orc.block_mean_pool(k, gc.bs)
    torch.testing.assert_close(orc.pooled_last_row(q, avg_k, gc.bs), gc.t("L0_avg_qk"),
                               rtol=2e-2, atol=1e-6)


@pytest.mark.parametrize("name", CASE_NAMES)
def test_full_layer_stack_matches_reference_sets(name):
    """q,k,v in -> the reference's block sets out, every layer, state carried across layers."""
    gc = GoldenCase(name)
    st = orc.SharingOracle(gc.lookup)
    wl = gc.wl
    for layer in range(wl.num_layers):
        q, k, v = gc.qkv(layer)
        o, sets, use_dense, info = orc.sparse_prefill_layer(
            st, q, k, v, layer, block_size=wl.block_size, min_budget=wl.min_budget,
            max_budget=wl.max_budget, pattern_threshold=wl.pattern_threshold,
            similarity_threshold=wl.similarity_threshold, fallback_threshold=wl.fallback_threshold,
            queryaware_threshold=wl.queryaware_threshold)
        assert torch.equal(use_dense, gc.t(f"L{layer}_use_dense"))
        for h, (a, b) in enumerate(zip(sets, gc.sets(layer))):
            assert torch.equal(a, b), f"layer {layer} head {h}"


def test_sparse_attention_against_masked_dense():
    gc = GoldenCase("peaky_share")
    q, k, v = gc.qkv(1)
    sets = gc.sets(1)
    o, _ = orc.sparse_attention(q, k, v, sets, torch.zeros(4, dtype=torch.bool), gc.bs)
    ref = orc.masked_dense_attention(q, k, v, sets, gc.bs)
    err = (o.float() - ref).abs()
    assert err.max() < 2e-2 and err.mean() < 2e-3


def test_avg_attn_rows_sum_to_one():
    gc = GoldenCase("peaky_share")
    a = gc.avg_attn(0)
    for h, m in a.items():
        torch.testing.assert_close(m.sum(-1), torch.ones(gc.nb), rtol=1e-3, atol=1e-3)
        assert torch.all(torch.triu(m, 1) == 0)
