"""The allocation-free variant of the last-block profile (spf_lastblock_profile_static).

It exists for callers that are not allowed to allocate device memory where the profile is
computed - a plugin inside another runtime's fixed memory plan, a serving loop with a frozen
pool - and keeps its pass-1 scratch in a fixed array inside the library.  The test drives it
through the C ABI exactly as such a caller would (inputs and outputs only), twice in a row,
and requires the result of the ordinary entry point, which takes caller-owned scratch.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.  It does not depend on them and passes alone in a fresh process.
"""
import pytest
import torch

from shareprefill_b200 import native
from shareprefill_b200.workloads import AttentionWorkload, make_qkv

pytestmark = pytest.mark.gpu


def _static_profile(q, k, block_size, vertical, slash):
    lib = native.load()
    n, h, d = q.shape
    rc = lib.spf_lastblock_profile_static(
        q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1),
        n, h, k.shape[1], d, block_size, vertical.data_ptr(), slash.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    return rc


@pytest.mark.parametrize("seq_len,heads,kv,d,bs", [(4096, 8, 2, 128, 128), (1000, 6, 2, 64, 64)])
def test_static_scratch_profile_equals_regular_entry_point(seq_len, heads, kv, d, bs):
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    wl = AttentionWorkload("noalloc", 70, seq_len, heads, kv, head_dim=d, num_head_clusters=2,
                           shared_rank=4, block_size=bs, q_gain=2.0)
    outs = []
    for call in range(2):                      # two calls in a row share the one scratch array
        q, k, _ = (t.to(dev) for t in make_qkv(wl, call))
        want_v, want_s = native.lastblock_profile(q, k, bs)
        got_v = torch.full_like(want_v, float("nan"))
        got_s = torch.full_like(want_s, float("nan"))
        torch.cuda.synchronize()
        held_before = torch.cuda.memory_allocated()
        rc = _static_profile(q, k, bs, got_v, got_s)
        torch.cuda.synchronize()
        assert rc == 0, native.load().spf_status_string(rc)
        assert torch.cuda.memory_allocated() == held_before, "nothing may be taken from torch's pool"
        # same kernels, same order of operations: the tolerance of the profile tests is more
        # than needed, the results are expected to be identical
        torch.testing.assert_close(got_v, want_v, rtol=2e-2, atol=1e-6)
        torch.testing.assert_close(got_s, want_s, rtol=2e-2, atol=1e-6)
        assert torch.equal(got_v, want_v) and torch.equal(got_s, want_s)
        outs.append(got_v.clone())
    assert not torch.equal(outs[0], outs[1]), "the two calls used different inputs"


def test_static_scratch_rejects_oversized_requests():
    dev = torch.device("cuda:0")
    lib = native.load()
    # 64 heads x 64K tokens needs ~16.8 MiB of scratch: beyond the fixed array
    n, h, d = 65536, 64, 128
    assert lib.spf_lastblock_scratch_bytes(n, h, 128) > 8 * 1024 * 1024 + 128 * 1024
    q = torch.zeros(1, dtype=torch.bfloat16, device=dev)   # never dereferenced: rejected up front
    out = torch.zeros(1, dtype=torch.float32, device=dev)
    rc = lib.spf_lastblock_profile_static(q.data_ptr(), h * d, d, q.data_ptr(), 8 * d, d, n, h, 8, d, 128,
                                          out.data_ptr(), out.data_ptr(), None)
    assert rc == -6 and b"maximum" in lib.spf_status_string(rc)
    # the largest documented shapes fit
    assert lib.spf_lastblock_scratch_bytes(32768, 32, 128) <= 8 * 1024 * 1024 + 128 * 1024
    assert lib.spf_lastblock_scratch_bytes(131072, 8, 128) <= 8 * 1024 * 1024 + 128 * 1024
