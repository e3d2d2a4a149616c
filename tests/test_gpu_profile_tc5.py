"""Last-block profile: the tcgen05 kernels (head_dim 128) against the CPU oracle and against the
mma.sync kernels on the same inputs."""

import pytest
import torch

from oracle import spf_oracle as orc
from shareprefill_b200 import native

pytestmark = pytest.mark.gpu


def _profile(q, k, bs, kernel):
    lib = native.load()
    lib.spf_force_generic_kernels(0, 1 if kernel == "generic" else 0)
    try:
        v, s = native.lastblock_profile(q, k, bs)
        torch.cuda.synchronize()
    finally:
        lib.spf_force_generic_kernels(0, 0)
    return v, s


@pytest.mark.parametrize("n,h,hkv,bs", [
    (1024, 8, 2, 128),      # four heads per CTA
    (1000, 7, 1, 128),      # ragged length, group of 7: CTAs with 4 and 3 heads
    (4096, 4, 4, 64),       # one head per CTA, block smaller than the 128-row tile
    (777, 6, 3, 32),        # two heads per CTA, ragged, small block
    (20000, 32, 8, 128),    # several key tiles per CTA
    (256, 2, 1, 16),
])
def test_profile_tc5_matches_oracle_and_generic(n, h, hkv, bs):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(n + h)
    q = (torch.randn(n, h, 128, generator=g) * 1.5).bfloat16()
    k = torch.randn(n, hkv, 128, generator=g).bfloat16()
    qd, kd = q.to(dev), k.to(dev)
    v5, s5 = _profile(qd, kd, bs, "tc5")
    assert native.load().spf_device_timeouts() == 0, "a bounded wait in the tcgen05 kernels ran out"
    vg, sg = _profile(qd, kd, bs, "generic")
    # same rounding points, different summation order and exponential argument rounding
    torch.testing.assert_close(v5, vg, rtol=2e-3, atol=1e-7)
    torch.testing.assert_close(s5, sg, rtol=2e-3, atol=1e-7)
    ones = torch.ones(h, device=dev)
    torch.testing.assert_close(v5.sum(-1), ones, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s5.sum(-1), ones, rtol=1e-4, atol=1e-4)
    if n <= 4096:
        want_v, want_s = orc.last_block_profile(q, k, bs)
        torch.testing.assert_close(v5.cpu(), want_v, rtol=2e-2, atol=1e-6)
        torch.testing.assert_close(s5.cpu(), want_s, rtol=2e-2, atol=1e-6)


def test_profile_tc5_strided_views():
    """[H,N,D]-contiguous tensors seen as [N,H,D] views go through TMA unchanged."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(11)
    n, h, hkv = 1500, 4, 2
    q = torch.randn(h, n, 128, generator=g).bfloat16().to(dev).transpose(0, 1)
    k = torch.randn(hkv, n, 128, generator=g).bfloat16().to(dev).transpose(0, 1)
    v5, s5 = _profile(q, k, 128, "tc5")
    vg, sg = _profile(q, k, 128, "generic")
    torch.testing.assert_close(v5, vg, rtol=2e-3, atol=1e-7)
    torch.testing.assert_close(s5, sg, rtol=2e-3, atol=1e-7)
