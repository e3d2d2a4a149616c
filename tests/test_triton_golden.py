"""Outputs of the reference's own Triton kernels (block-sparse attention, CSR offsets, K pooling),
recorded on a B200 by tests/golden/make_golden_triton.py, against the CPU oracle (always) and the
CUDA kernels of this package (GPU tests)."""
import importlib.util
import math
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR
from oracle import spf_oracle as orc

spec = importlib.util.spec_from_file_location("make_golden_triton", os.path.join(GOLDEN_DIR, "make_golden_triton.py"))
gen = importlib.util.module_from_spec(spec)
spec.loader.exec_module(gen)

MAX_ABS, MEAN_ABS = 2e-2, 2e-3


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLDEN_DIR, "triton_kernels.npz"))


def _ref_output(gold, name):
    if f"{name}_o_bits" in gold.files:
        return torch.from_numpy(gold[f"{name}_o_bits"]).view(torch.bfloat16), slice(None)
    return torch.from_numpy(gold[f"{name}_o_bits_rows8"]).view(torch.bfloat16), slice(None, None, 8)


def _check_out(got, want):
    want = want.float()
    err = (got.float() - want).abs()
    bound = torch.maximum(torch.full_like(want, MAX_ABS), want.abs() * 2.0 ** -7)   # one bf16 ulp where |o| >= 4
    assert (err - bound).max().item() <= 0, err.max().item()
    assert err.mean().item() <= MEAN_ABS, err.mean().item()


@pytest.mark.parametrize("name", list(gen.CASES))
def test_oracle_attention_matches_reference_kernel(gold, name):
    q, k, v, sets, use_dense, bs = gen.case_inputs(name)
    o, avg = orc.sparse_attention(q, k, v, sets, use_dense, bs)
    want, rows = _ref_output(gold, name)
    _check_out(o[rows], want)
    ref_avg = torch.from_numpy(gold[f"{name}_avg_attn"])
    for h in range(q.shape[1]):
        if bool(use_dense[h]):
            torch.testing.assert_close(avg[h], ref_avg[h], rtol=2e-3, atol=2e-4)
        else:
            assert float(ref_avg[h].abs().max()) == 0.0       # the reference writes pivots only


@pytest.mark.parametrize("name", list(gen.CASES))
def test_oracle_csr_offsets_match_reference_kernel(gold, name):
    q, _, _, sets, _, bs = gen.case_inputs(name)
    nb = -(-q.shape[0] // bs)
    ref_bins = torch.from_numpy(gold[f"{name}_idx_bins"])
    for h, s in enumerate(sets):
        assert torch.equal(orc.csr_row_offsets(torch.sort(s).values, nb), ref_bins[h])


@pytest.mark.parametrize("name", list(gen.CASES))
def test_oracle_pooling_vs_reference_kernel(gold, name):
    """The Triton kernel sums in bf16 with its own reduction tree; the oracle (and the CUDA kernel)
    sum in fp32 and round once.  The two agree to a few bf16 ulps of the block's largest
    magnitude - the reference's result carries the rounding error of its bf16 tree."""
    _, k, _, _, _, bs = gen.case_inputs(name)
    ref = torch.from_numpy(gold[f"{name}_pool_k_bits"]).view(torch.bfloat16).float()
    mine = orc.block_mean_pool(k, bs).float()
    assert (mine - ref).abs().max().item() <= 2e-2
    assert (mine - ref).abs().mean().item() <= 2e-3


# ------------------------------------------------------------------------------------- GPU
@pytest.mark.gpu
@pytest.mark.parametrize("name", list(gen.CASES))
def test_cuda_attention_matches_reference_kernel(gold, name):
    from shareprefill_b200 import native
    dev = torch.device("cuda:0")
    q, k, v, sets, use_dense, bs = gen.case_inputs(name)
    nb = -(-q.shape[0] // bs)
    bm = native.sets_to_bitmap(sets, nb, dev)
    flags = (use_dense.to(torch.int32) * native.HEAD_PIVOT).to(dev)
    slots = torch.where(use_dense, torch.arange(len(sets)), torch.full((len(sets),), -1)).to(torch.int32).to(dev)
    state = native.SharingStateBuffer(len(sets), nb, dev)
    out = native.sparse_attention(q.to(dev), k.to(dev), v.to(dev), bm, bs, 1.0 / math.sqrt(q.shape[2]),
                                  flags, slots, state)
    want, rows = _ref_output(gold, name)
    _check_out(out.cpu()[rows], want)
    ref_avg = torch.from_numpy(gold[f"{name}_avg_attn"])
    for h in torch.nonzero(use_dense).flatten().tolist():
        torch.testing.assert_close(state.field("pivot_attn")[h].cpu(), ref_avg[h], rtol=2e-3, atol=2e-4)
    assert native.load().spf_device_timeouts() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(gen.CASES))
def test_cuda_pooling_vs_reference_kernel(gold, name):
    from shareprefill_b200 import native
    _, k, _, _, _, bs = gen.case_inputs(name)
    _, avg_k = native.pool_qk(None, k.cuda(), bs)
    ref = torch.from_numpy(gold[f"{name}_pool_k_bits"]).view(torch.bfloat16).float()
    d = (avg_k.float().cpu() - ref).abs()
    assert d.max().item() <= 2e-2 and d.mean().item() <= 2e-3
