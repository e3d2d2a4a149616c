"""The tcgen05/TMEM attention kernel (block_size = head_dim = 128) against the CPU oracle and
against the generic mma.sync kernel on the same inputs."""
import math

import pytest
import torch

from oracle import spf_oracle as orc
from shareprefill_b200 import native

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _assert_out_close(got, want, name=""):
    """max-abs 2e-2 / mean-abs 2e-3; where |want| >= 4 one bf16 ulp (2^-7 relative) already
    exceeds 2e-2, so a one-ulp difference of the bf16 output is accepted there."""
    want = want.float()
    err = (got.float().cpu() - want).abs()
    bound = torch.maximum(torch.full_like(want, MAX_ABS), want.abs() * 2.0 ** -7)
    worst = (err - bound).max().item()
    assert worst <= 0, f"{name}: max abs {err.max().item()} (beyond bound by {worst})"
    assert err.mean().item() <= MEAN_ABS, f"{name}: mean abs {err.mean().item()}"


def _random_sets(nb, h, density, g):
    sets = []
    for _ in range(h):
        m = torch.tril(torch.rand(nb, nb, generator=g) < density)
        m[:, 0] = True
        m |= torch.eye(nb, dtype=torch.bool)
        sets.append(torch.nonzero(m.reshape(-1)).flatten())
    return sets


def _run(q, k, v, bm, kernel):
    lib = native.load()
    lib.spf_force_generic_kernels(1 if kernel == "generic" else 0, 0)
    try:
        out = native.sparse_attention(q, k, v, bm, 128, 1.0 / math.sqrt(128))
        torch.cuda.synchronize()
    finally:
        lib.spf_force_generic_kernels(0, 0)
    return out


@pytest.mark.parametrize("n,h,hkv,density", [
    (640, 4, 2, 0.5),        # two heads per CTA, both K/V reuse paths
    (1000, 7, 1, 0.4),       # odd group: the last CTA of the group carries a single head; ragged N
    (2048, 2, 2, 1.0),       # one head per KV head, dense triangle
    (1536, 8, 2, 0.15),      # sparse rows: heads of a pair visit different columns
])
def test_tc5_matches_oracle_and_generic(n, h, hkv, density):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(n + h)
    q = torch.randn(n, h, 128, generator=g).bfloat16()
    k = torch.randn(n, hkv, 128, generator=g).bfloat16()
    v = torch.randn(n, hkv, 128, generator=g).bfloat16()
    nb = -(-n // 128)
    sets = _random_sets(nb, h, density, g)
    bm = native.sets_to_bitmap(sets, nb, dev)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out_tc5 = _run(qd, kd, vd, bm, "tc5")
    assert native.load().spf_device_timeouts() == 0, "a bounded wait in the tcgen05 kernel ran out"
    out_gen = _run(qd, kd, vd, bm, "generic")
    want, _ = orc.sparse_attention(q, k, v, sets, torch.zeros(h, dtype=torch.bool), 128)
    for name, got in (("tcgen05", out_tc5), ("generic", out_gen)):
        _assert_out_close(got, want, name)
    d = (out_tc5.float() - out_gen.float()).abs()
    assert bool((d <= torch.maximum(torch.full_like(d, MAX_ABS), out_gen.float().abs() * 2.0 ** -7)).all())


@pytest.mark.parametrize("n,h,hkv,density", [
    (8192, 16, 4, 0.08),     # 512 work items, sparse rows that differ between the heads of a pair
    (6000, 12, 4, 0.5),      # odd pairs (3 heads per KV head), ragged N
    (4096, 8, 8, 1.0),       # single-head items, dense
])
def test_tc5_many_items_per_cta_matches_generic(n, h, hkv, density):
    """Many more (query block, head pair) items than SMs: several waves of CTAs, rows of very
    different lengths, both issue modes (heads of a pair that visit the same or different blocks)."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(n + 3 * h)
    q = torch.randn(n, h, 128, generator=g).bfloat16().to(dev)
    k = torch.randn(n, hkv, 128, generator=g).bfloat16().to(dev)
    v = torch.randn(n, hkv, 128, generator=g).bfloat16().to(dev)
    nb = -(-n // 128)
    m = torch.tril(torch.rand(h, nb, nb, generator=g) < density)
    m[:, :, 0] = True
    m |= torch.eye(nb, dtype=torch.bool)
    m[1, 5:9] = False        # rows without any block (also no diagonal) in one head of a pair
    m[2, 7] = False
    sets = [torch.nonzero(m[i].reshape(-1)).flatten() for i in range(h)]
    bm = native.sets_to_bitmap(sets, nb, dev)
    for _ in range(2):       # twice: a second launch right behind the first
        out_tc5 = _run(q, k, v, bm, "tc5")
        assert native.load().spf_device_timeouts() == 0, "a bounded wait in the tcgen05 kernel ran out"
    out_gen = _run(q, k, v, bm, "generic")
    d = (out_tc5.float() - out_gen.float()).abs()
    bound = torch.maximum(torch.full_like(d, MAX_ABS), out_gen.float().abs() * 2.0 ** -7)
    assert bool((d <= bound).all()), f"max abs {d.max().item()}"
    assert d.mean().item() <= MEAN_ABS
    # rows that visit nothing come back as zeros
    assert float(out_tc5[5 * 128:9 * 128, 1].float().abs().max()) == 0.0


def test_tc5_large_logits_trigger_rescale():
    """Scores that grow along the row force the running maximum to move by far more than the
    lazy-rescale margin, so the O accumulator in TMEM is rescaled many times."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(5)
    n, h = 1024, 2
    q = (torch.randn(n, h, 128, generator=g) * 3).bfloat16()
    k = torch.randn(n, 1, 128, generator=g)
    k = (k * torch.linspace(0.2, 4.0, n)[:, None, None]).bfloat16()     # later keys score higher
    v = torch.randn(n, 1, 128, generator=g).bfloat16()
    nb = n // 128
    sets = _random_sets(nb, h, 1.0, g)
    bm = native.sets_to_bitmap(sets, nb, dev)
    out = _run(q.to(dev), k.to(dev), v.to(dev), bm, "tc5")
    assert native.load().spf_device_timeouts() == 0
    want, _ = orc.sparse_attention(q, k, v, sets, torch.zeros(h, dtype=torch.bool), 128)
    _assert_out_close(out, want, "rescale")


def test_tc5_reference_point_moves_when_a_block_overflows_it():
    """A row's exponentials are taken against the maximum of its FIRST block; later blocks whose scores
    lie 2^70 and more above that point must be caught by the block-sum check and redone against their own
    maximum, with O rescaled.  Keys of block 0 are tiny, keys of blocks 2 and 5 are aligned with the
    queries (scores 55 and 90 nats above block 0), the rest is noise."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(11)
    n, h = 1024, 3                                  # an odd group: head pairs and the two-row CTA
    e = torch.ones(128) / math.sqrt(128.0)
    q = (25.0 * e + 0.25 * torch.randn(n, h, 128, generator=g)).bfloat16()
    k = (0.25 * torch.randn(n, 1, 128, generator=g))
    k[:128] *= 0.01
    k[256:384] += 25.0 * e
    k[640:768] += 40.0 * e
    k = k.bfloat16()
    v = torch.randn(n, 1, 128, generator=g).bfloat16()
    nb = n // 128
    sets = _random_sets(nb, h, 1.0, g)
    bm = native.sets_to_bitmap(sets, nb, dev)
    out = _run(q.to(dev), k.to(dev), v.to(dev), bm, "tc5")
    assert native.load().spf_device_timeouts() == 0
    assert bool(torch.isfinite(out.float()).all())
    want, _ = orc.sparse_attention(q, k, v, sets, torch.zeros(h, dtype=torch.bool), 128)
    _assert_out_close(out, want, "moved reference")


def test_tc5_strided_inputs():
    """[H,N,D]-contiguous tensors seen as [N,H,D] views (head stride N*D) go through TMA unchanged."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(9)
    n, h, hkv = 768, 4, 2
    q = torch.randn(h, n, 128, generator=g).bfloat16().to(dev).transpose(0, 1)
    k = torch.randn(hkv, n, 128, generator=g).bfloat16().to(dev).transpose(0, 1)
    v = torch.randn(hkv, n, 128, generator=g).bfloat16().to(dev).transpose(0, 1)
    nb = n // 128
    sets = _random_sets(nb, h, 0.6, g)
    bm = native.sets_to_bitmap(sets, nb, dev)
    out = _run(q, k, v, bm, "tc5")
    want, _ = orc.sparse_attention(q.cpu().contiguous(), k.cpu().contiguous(), v.cpu().contiguous(), sets,
                                   torch.zeros(h, dtype=torch.bool), 128)
    _assert_out_close(out, want, "strided")
