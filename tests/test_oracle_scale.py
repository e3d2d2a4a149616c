"""The CPU oracle against the reference's results at the sizes and head layouts of the benchmark
configurations (tests/golden/make_golden.py, SCALE_CASES), and the query-aware cover rule on tied
scores."""
import numpy as np
import pytest
import torch

from golden_cases import GOLDEN_DIR, SCALE_CASE_NAMES, ScaleCase
from oracle import spf_oracle as orc


def _avg_attn(gc, layer):
    if not gc.has(f"L{layer}_avg_attn"):
        return {}
    return dict(zip(gc.z[f"L{layer}_dense_heads"].tolist(), gc.t(f"L{layer}_avg_attn")))


@pytest.mark.parametrize("name", SCALE_CASE_NAMES)
def test_stage_values_are_exact(name):
    """Cover counts over the un-pooled profiles, pooled profiles and the query-aware divergence."""
    gc = ScaleCase(name)
    thr = gc.wl.pattern_threshold
    for layer in gc.layers:
        v, s = gc.t(f"L{layer}_vertical"), gc.t(f"L{layer}_slash")
        sh = gc.score_heads
        assert torch.equal(orc.cover_count(v, thr), gc.t(f"L{layer}_cover_v")[sh])
        assert torch.equal(orc.cover_count(s, thr), gc.t(f"L{layer}_cover_s")[sh])
        assert torch.equal(orc.block_sum_pool(v, gc.bs), gc.t(f"L{layer}_vpool")[sh])
        assert torch.equal(orc.block_sum_pool(s, gc.bs), gc.t(f"L{layer}_spool")[sh])
        jsd = orc.sqrt_jsd(gc.t(f"L{layer}_avg_qk"), gc.t(f"L{layer}_vpool"))
        assert torch.equal(jsd, gc.t(f"L{layer}_jsd_qa"))


@pytest.mark.parametrize("name", SCALE_CASE_NAMES)
def test_selection_from_recorded_scores_is_exact(name):
    gc = ScaleCase(name)
    st = orc.SharingOracle(gc.lookup)
    for layer in gc.layers:
        kw = {} if gc.all_scores else dict(heads=gc.score_heads, vpool=gc.t(f"L{layer}_vpool"),
                                           spool=gc.t(f"L{layer}_spool"))
        sets, use_dense, info = st.select_from_scores(
            layer, gc.t(f"L{layer}_vertical"), gc.t(f"L{layer}_slash"), gc.t(f"L{layer}_avg_qk"),
            gc.qa_scores(layer), **gc.knobs(), **kw)
        assert torch.equal(use_dense, gc.t(f"L{layer}_use_dense"))
        assert torch.equal(info["use_qa"], gc.t(f"L{layer}_use_qa"))
        want = gc.sets(layer)
        qa_sc = gc.qa_scores(layer)
        for h in gc.score_heads:
            if torch.equal(sets[h], want[h]):
                continue
            from golden_cases import same_cover_up_to_ties
            a = torch.zeros(gc.nb * gc.nb, dtype=torch.bool); a[sets[h]] = True
            b = torch.zeros(gc.nb * gc.nb, dtype=torch.bool); b[want[h]] = True
            assert h in qa_sc and same_cover_up_to_ties(a, b, qa_sc[h]), f"layer {layer} head {h}"
        st.update_pivots(layer, _avg_attn(gc, layer), use_dense, gc.wl.pattern_threshold)
    for cid in gc.shared_ids():
        assert st.pivot_head.get(cid, -1) == int(gc.z[f"S{cid}_pivot_head"])
        if gc.has(f"S{cid}_pattern"):
            from golden_cases import bitmap_to_sets_cpu
            want = bitmap_to_sets_cpu(torch.from_numpy(gc.z[f"S{cid}_pattern"].astype(np.int64))[None], gc.nb)[0]
            assert torch.equal(st.pivot_pattern[cid], want)
        r = float(gc.z[f"S{cid}_vs_ratio"])
        if r == r:
            assert st.vs_ratio[cid] == r


@pytest.mark.parametrize("name", ["qa_8k", "qwen_8k", "llama_32k"])
def test_selection_from_qkv_at_scale(name):
    """q,k in -> the reference's flags and (nearly all of) its block sets: the oracle's logits come from
    a matmul, the reference's from an einsum, and a few bf16 roundings differ between the two."""
    gc = ScaleCase(name)
    st = orc.SharingOracle(gc.lookup)
    for layer in gc.layers:
        q, k, v = gc.qkv(layer)
        sets, use_dense, info = st.get_active_blocks(q, k, layer, **gc.knobs())
        assert torch.equal(use_dense, gc.t(f"L{layer}_use_dense"))
        assert torch.equal(info["use_qa"], gc.t(f"L{layer}_use_qa"))
        want = gc.sets(layer)
        same = sum(int(torch.equal(a, b)) for a, b in zip(sets, want))
        assert same >= len(want) - 2, f"{name} layer {layer}: {same} of {len(want)} heads identical"
        g = gc.wl.group_size
        avg = {h: orc.pivot_block_mass(q[:, h], k[:, h // g], gc.bs)
               for h in torch.nonzero(use_dense).flatten().tolist()}
        st.update_pivots(layer, avg, use_dense, gc.wl.pattern_threshold)


def test_pivot_block_mass_matches_the_two_pass_restatement():
    from golden_cases import GoldenCase
    gc = GoldenCase("ragged_rope")
    q, k, v = gc.qkv(0)
    for h, m in gc.avg_attn(0).items():
        got = orc.pivot_block_mass(q[:, h], k[:, h // gc.wl.group_size], gc.bs)
        torch.testing.assert_close(got, m, rtol=1e-5, atol=1e-6)


def test_query_aware_cover_with_tied_scores():
    """Ties at the crossing value: same number of blocks as the reference, identical outside the tied
    value (the order of equal values is torch.sort's choice and may differ between builds)."""
    from golden_cases import same_cover_up_to_ties
    z = np.load(f"{GOLDEN_DIR}/qa_ties.npz")
    for nb in (64, 80, 96):
        p = torch.from_numpy(z[f"tie{nb}_scores"])
        for thr in (0.5, 0.9, 0.95):
            got = torch.zeros(nb * nb, dtype=torch.bool)
            got[orc.cover_indices_global(p.reshape(-1), thr * nb)] = True
            want = torch.zeros(nb * nb, dtype=torch.bool)
            want[torch.from_numpy(z[f"tie{nb}_kept_{thr}"])] = True
            want[0] = True
            assert same_cover_up_to_ties(got, want, p.reshape(-1))
