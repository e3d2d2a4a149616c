"""Edge cases of the CUDA path: degenerate patterns, smallest and ragged sizes, argument errors."""
import ctypes
import math

import pytest
import torch

from oracle import spf_oracle as orc
from shareprefill_b200 import native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _qkv(n, h, hkv, d, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(n, h, d, generator=g).bfloat16(), torch.randn(n, hkv, d, generator=g).bfloat16(),
            torch.randn(n, hkv, d, generator=g).bfloat16())


def _close(got, want):
    want = want.float()
    err = (got.float().cpu() - want).abs()
    bound = torch.maximum(torch.full_like(want, 2e-2), want.abs() * 2.0 ** -7)
    assert (err - bound).max().item() <= 0 and err.mean().item() <= 2e-3


@pytest.mark.parametrize("bs,d", [(128, 128), (64, 64)])
def test_rows_without_blocks_give_zeros(bs, d):
    """A head whose bitmap row is empty (never produced by the selection, but legal input) outputs
    zeros for that query block on both kernels; its neighbours are unaffected."""
    n, h = bs * 4, 2
    q, k, v = _qkv(n, h, 1, d, 1)
    nb = 4
    full = torch.tril(torch.ones(nb, nb, dtype=torch.bool))
    m0 = full.clone(); m0[2] = False                      # head 0 skips query block 2 entirely
    sets = [torch.nonzero(m0.reshape(-1)).flatten(), torch.nonzero(full.reshape(-1)).flatten()]
    out = native.sparse_attention(q.to(DEV), k.to(DEV), v.to(DEV), native.sets_to_bitmap(sets, nb, DEV), bs,
                                  1 / math.sqrt(d))
    assert float(out[2 * bs:3 * bs, 0].abs().max()) == 0.0
    want, _ = orc.sparse_attention(q, k, v, [sets[1], sets[1]], torch.zeros(2, dtype=torch.bool), bs)
    _close(out[:, 1], want[:, 1])
    _close(out[:2 * bs, 0], want[:2 * bs, 0])
    assert native.load().spf_device_timeouts() == 0


@pytest.mark.parametrize("n", [128, 129, 255, 257])
def test_smallest_and_ragged_lengths_full_path(n, tmp_path):
    """N = block_size and N just around block boundaries through the whole selection + attention."""
    import json
    from shareprefill_b200.attention import sparse_prefill_attention
    from shareprefill_b200.configuration import SharePrefillConfig
    from shareprefill_b200.sharing_state import AttentionSharing
    from shareprefill_b200.workloads import synthetic_lookup
    p = tmp_path / "l.json"
    p.write_text(json.dumps(synthetic_lookup(1, 4, 2, group_size=2)))
    cfg = SharePrefillConfig(model_name="x", sharing_lookup_path=str(p), min_budget=128)
    q, k, v = _qkv(n, 4, 2, 128, n)
    sharing = AttentionSharing(str(p))
    out, pat = sparse_prefill_attention(sharing, q.to(DEV), k.to(DEV), v.to(DEV), 0, 4, cfg, 1 / math.sqrt(128))
    sets = [s.cpu() for s in pat.to_index_lists()[0]]
    want, _ = orc.sparse_attention(q, k, v, sets, pat.use_dense[0].cpu(), 128)
    _close(out, want)
    nb = -(-n // 128)
    for s in sets:
        assert 0 in s.tolist() and (nb * nb - 1) in s.tolist()      # sink block and last diagonal block


def test_selection_with_every_head_in_one_shared_cluster(tmp_path):
    """One cluster, shared, 8 heads: exactly one pivot is elected (the first non-query-aware head),
    and it stays the pivot in the next layer."""
    import json
    from shareprefill_b200.sharing_state import AttentionSharing
    from shareprefill_b200.workloads import AttentionWorkload, make_qkv, synthetic_lookup
    wl = AttentionWorkload("one_cluster", 60, 2048, 8, 2, num_layers=2, num_head_clusters=1, q_gain=3.0)
    p = tmp_path / "l.json"
    p.write_text(json.dumps(synthetic_lookup(2, 8, 1)))
    sharing = AttentionSharing(str(p))
    for layer in range(2):
        q, k, v = (t.to(DEV) for t in make_qkv(wl, layer))
        pat, dense = sharing.get_active_blocks(q[None], k[None], layer, 8, 128, 2, 2**31 - 1, 0.95, 0.5, 1e9, 0.1)
        out = native.sparse_attention(q, k, v, pat.bitmap, 128, 1 / math.sqrt(128), pat.flags, pat.slot_of_head,
                                      sharing.state)
        sharing.update_pivotal_attns(layer, None, dense, 0.95)
        qa = (pat.flags & native.HEAD_QUERY_AWARE) != 0
        if layer == 0:
            assert int(dense.sum()) == (0 if bool(qa.all()) else 1)
            first = int(sharing.state.field("pivot_head")[0])
            if first >= 0:
                assert not bool(qa[first]) and bool(qa[:first].all())
        else:
            assert int(dense.sum()) == 0 or first < 0
    assert int(sharing.state.field("pattern_ready")[0]) == (1 if first >= 0 else 0)


def test_argument_errors_on_device_pointers():
    lib = native.load()
    q, k, v = (t.to(DEV) for t in _qkv(256, 2, 1, 128))
    out = torch.empty(256, 2, 128, dtype=torch.bfloat16, device=DEV)
    bm = torch.zeros(2, 2, 1, dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream

    def attn(qp, sn, sh, n, hq, hkv, d, bs):
        return lib.spf_sparse_attention(qp, sn, sh, k.data_ptr(), 128, 128, v.data_ptr(), 128, 128, n, hq, hkv, d, bs,
                                        0.088, bm.data_ptr(), None, None, None, 0, out.data_ptr(), st)
    assert attn(q.data_ptr(), 256, 128, 256, 2, 1, 128, 128) == 0
    assert attn(q.data_ptr() + 2, 256, 128, 256, 2, 1, 128, 128) == -3      # misaligned pointer
    assert attn(q.data_ptr(), 252, 128, 256, 2, 1, 128, 128) == -3          # token stride not 16-byte
    assert attn(q.data_ptr(), 256, 128, 256, 2, 1, 96, 128) == -2           # head_dim
    assert attn(q.data_ptr(), 256, 128, 256, 2, 1, 128, 48) == -2           # block_size
    assert attn(q.data_ptr(), 256, 128, 64, 2, 1, 128, 128) == -2           # fewer tokens than a block
    assert attn(q.data_ptr(), 256, 128, 256, 3, 2, 128, 128) == -2          # heads not a multiple of kv heads
    assert attn(None, 256, 128, 256, 2, 1, 128, 128) == -1
    torch.cuda.synchronize()
    assert lib.spf_device_timeouts() == 0


def test_budget_clamps_and_max_budget():
    """max_budget below min_budget wins (the reference clamps low first, high last)."""
    n, h = 4096, 4
    g = torch.Generator().manual_seed(3)
    vert = torch.rand(h, n, generator=g); vert /= vert.sum(-1, keepdim=True)
    sl = torch.rand(h, n, generator=g); sl /= sl.sum(-1, keepdim=True)
    nv, ns, _, _ = native.profile_budgets(vert.to(DEV), sl.to(DEV), 128, 0.95, 8, 3)
    assert nv.tolist() == [3] * h and ns.tolist() == [3] * h
    nv, ns, _, _ = native.profile_budgets(vert.to(DEV), sl.to(DEV), 128, 0.95, 8, 10**9)
    want_v, want_s = orc.block_budgets(vert, sl, 128, 0.95, 8, 32)
    assert nv.cpu().long().tolist() == want_v.tolist() and ns.cpu().long().tolist() == want_s.tolist()
