"""Run the reference's own selection code on CPU.  TEST INFRASTRUCTURE ONLY.

The reference's ``AttentionSharing.get_active_blocks`` (shareprefill/attn/attention_sharing.py:105-366)
is plain torch except for two things: the literal device string ``"cuda"`` at a few call sites
(attention_sharing.py:205,219; utils.py:212) and the Triton key-pooling kernel
(``triton_bnhd_pool``, utils.py:211-261).  This module supplies both from the outside - a context
manager that maps ``"cuda"`` to CPU while the reference runs, and the oracle's block mean in place
of the Triton kernel - without touching reference files.  Used by the golden-vector generator and
by the CPU baseline / reference arm of the benchmark; the shipped package never imports it.
"""
from __future__ import annotations

import contextlib
import importlib
import os
import sys

import torch

from . import spf_oracle as orc


@contextlib.contextmanager
def cuda_string_to_cpu():
    real_empty, real_to = torch.empty, torch.Tensor.to

    def empty(*a, **kw):
        if kw.get("device") == "cuda":
            kw["device"] = "cpu"
        return real_empty(*a, **kw)

    def to(self, *a, **kw):
        a = tuple("cpu" if (isinstance(x, str) and x == "cuda") else x for x in a)
        if kw.get("device") == "cuda":
            kw["device"] = "cpu"
        return real_to(self, *a, **kw)

    torch.empty, torch.Tensor.to = empty, to
    try:
        yield
    finally:
        torch.empty, torch.Tensor.to = real_empty, real_to


def block_mean_pool_bnhd(x, kernel_size, pool_type="avg"):
    """Drop-in for ``triton_bnhd_pool`` on ``[B,N,H,D]`` input, batch 1."""
    return orc.block_mean_pool(x[0], kernel_size)[None]


def import_reference_selection(reference_root: str):
    """Import ``shareprefill.attn.attention_sharing`` from a checkout or an installed copy of the
    reference and rebind its Triton pooling to the CPU block mean.  Returns the module."""
    if not os.path.isdir(os.path.join(reference_root, "shareprefill")):
        raise FileNotFoundError(f"no reference package under {reference_root}")
    if reference_root not in sys.path:
        sys.path.insert(0, reference_root)
    att = importlib.import_module("shareprefill.attn.attention_sharing")
    att.triton_bnhd_pool = block_mean_pool_bnhd
    return att


def reference_get_active_blocks(att, state, q, k, layer, num_heads, block_size, min_blocks, max_blocks,
                                pattern_threshold, similarity_threshold, fallback_threshold,
                                queryaware_threshold):
    """``state.get_active_blocks`` of the reference on CPU tensors q ``[N,H,D]``, k ``[N,Hkv,D]``
    (K is repeated to the query-head count, as the reference's entry point does,
    shareprefill_attn.py:33-84).  Returns ``(block_idx, use_dense)`` as the reference does."""
    g = q.shape[1] // k.shape[1]
    with cuda_string_to_cpu():
        return state.get_active_blocks(
            q[None].contiguous(), k.repeat_interleave(g, dim=1)[None].contiguous(), layer, num_heads,
            block_size, min_blocks, max_blocks, pattern_threshold, similarity_threshold,
            fallback_threshold, queryaware_threshold, False)
