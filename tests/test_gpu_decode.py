"""Decode-step kernel (one query token against the KV cache) against the fp32 oracle."""
import pytest
import torch

from oracle import spf_oracle as O
from shareprefill_b200 import native

pytestmark = pytest.mark.gpu

# bf16 output of an fp32-accumulated kernel: one bf16 ulp of the value plus accumulation noise
ATOL, RTOL = 2e-3, 2 ** -7


def _case(nk, h, hkv, d, seed, strided=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(h, d, generator=g).to(torch.bfloat16)
    if strided:   # a [Hkv, N, D] cache viewed token-major, as the model cache hands it over
        k = torch.randn(hkv, nk, d, generator=g).to(torch.bfloat16).transpose(0, 1)
        v = torch.randn(hkv, nk, d, generator=g).to(torch.bfloat16).transpose(0, 1)
    else:
        k = torch.randn(nk, hkv, d, generator=g).to(torch.bfloat16)
        v = torch.randn(nk, hkv, d, generator=g).to(torch.bfloat16)
    return q, k, v


@pytest.mark.parametrize("nk,h,hkv,d,strided", [
    (1, 32, 8, 128, False), (5, 32, 8, 128, False), (255, 32, 8, 128, True), (4097, 32, 8, 128, True),
    (70001, 32, 8, 128, False), (1000, 8, 2, 64, True), (33, 4, 4, 64, False), (3001, 64, 8, 128, False),
    (777, 64, 4, 128, True), (2049, 32, 1, 128, False), (130, 48, 2, 64, False), (17, 1, 1, 128, False),
])
def test_decode_matches_oracle(nk, h, hkv, d, strided):
    q, k, v = _case(nk, h, hkv, d, 1234 + nk, strided)
    want = O.decode_attention(q, k, v, d ** -0.5)
    got = native.decode_attention(q.cuda(), k.cuda(), v.cuda(), d ** -0.5).float().cpu()
    err = (got - want).abs()
    assert bool((err <= ATOL + RTOL * want.abs()).all()), float(err.max())


def test_decode_peaked_scores():
    # one key dominates: the result is that key's value row, exactly representable in bf16
    q, k, v = _case(2000, 8, 2, 128, 7)
    k[777] = (q.view(2, 4, 128)[:, 0] * 4).to(torch.bfloat16)
    want = O.decode_attention(q, k, v, 1.0)
    got = native.decode_attention(q.cuda(), k.cuda(), v.cuda(), 1.0).float().cpu()
    assert float((got - want).abs().max()) <= 2e-2


def test_decode_argument_errors():
    q, k, v = _case(64, 8, 2, 128, 3)
    with pytest.raises(native.SpfError):
        native.decode_attention(q.cuda(), k.cuda()[:, :, :96], v.cuda()[:, :, :96], 1.0)   # head_dim mismatch
    with pytest.raises(native.SpfError):
        native.decode_attention(q.cuda()[:7], k.cuda(), v.cuda(), 1.0)                     # 7 heads over 2 KV heads
