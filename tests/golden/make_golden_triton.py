"""Golden vectors from the reference's own Triton kernels, run on a GPU.

The reference's block-sparse attention (attn/shareprefill_attn.py:272-620), its CSR offset kernel
(:187-269) and its pooling kernel (attn/utils.py:131-261) only run on a GPU.  This script runs
them unmodified - from an offline install of the reference under baseline/_ref, made with

    pip install --no-index --no-build-isolation --no-deps --ignore-requires-python \
        --target baseline/_ref <reference checkout>

- on seeded inputs and stores the outputs:

    python tests/golden/make_golden_triton.py --out triton_kernels_full.npz

Inputs are regenerated from the seeds by the tests (torch CPU generator), outputs are stored.  The
committed tests/golden/triton_kernels.npz is that file with the largest case's output thinned to
every eighth row (key ``c128_o_bits_rows8``) to keep the fixture small.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

CASES = {
    # name: (seed, N, H, Hkv, D, block_size, density, dense_heads)
    "a128": (101, 640, 2, 1, 128, 128, 0.6, [0]),
    "b64": (102, 1000, 4, 2, 64, 64, 0.5, [1]),
    "c128": (103, 1536, 4, 2, 128, 128, 0.35, []),
}


def case_inputs(name):
    seed, n, h, hkv, d, bs, density, dense = CASES[name]
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n, h, d, generator=g).bfloat16()
    k = torch.randn(n, hkv, d, generator=g).bfloat16()
    v = torch.randn(n, hkv, d, generator=g).bfloat16()
    nb = -(-n // bs)
    sets = []
    for hh in range(h):
        m = torch.tril(torch.rand(nb, nb, generator=g) < density)
        if hh in dense:
            m = torch.tril(torch.ones(nb, nb, dtype=torch.bool))
        m[:, 0] = True
        m |= torch.eye(nb, dtype=torch.bool)
        sets.append(torch.nonzero(m.reshape(-1)).flatten())
    use_dense = torch.zeros(h, dtype=torch.bool)
    use_dense[dense] = True
    return q, k, v, sets, use_dense, bs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(HERE, "triton_kernels_full.npz"))
    ap.add_argument("--ref", default=os.path.join(ROOT, "baseline", "_ref"))
    args = ap.parse_args()
    sys.path.insert(0, args.ref)
    from shareprefill.attn import shareprefill_attn as ref_attn
    from shareprefill.attn import utils as ref_utils
    out = {}
    for name in CASES:
        q, k, v, sets, use_dense, bs = case_inputs(name)
        qd, kd, vd = (t[None].cuda() for t in (q, k, v))
        block_idx = [[s.cuda() for s in sets]]
        o, avg = ref_attn.triton_block_wise_prefill_attention(qd, kd, vd, block_idx, use_dense[None].cuda(), bs)
        torch.cuda.synchronize()
        out[f"{name}_o_bits"] = o[0].cpu().view(torch.int16).numpy()
        out[f"{name}_avg_attn"] = avg[0].cpu().numpy()
        nb = -(-q.shape[0] // bs)
        padded = torch.nn.utils.rnn.pad_sequence([s.view(-1, 1) for s in sets], batch_first=True,
                                                 padding_value=nb * (nb + 1)).view(1, len(sets), -1)
        bins = ref_attn.triton_column_count_cumsum(padded.sort(-1).values.cuda(), nb)
        out[f"{name}_idx_bins"] = bins[0].cpu().numpy()
        pooled = ref_utils.triton_bnhd_pool(kd, bs)
        out[f"{name}_pool_k_bits"] = pooled[0].cpu().view(torch.int16).numpy()
        print(name, "ok", o.shape, avg.shape, bins.shape, pooled.shape)
    os.makedirs(os.path.dirname(args.out), exist_ok=True)
    np.savez_compressed(args.out, **out)
    print("wrote", args.out)


if __name__ == "__main__":
    main()
