"""Attention entry point registered with Hugging Face's attention interface.

Mirrors ``shareprefill_attention_forward`` / ``shareprefill_attention_core``
(attn/shareprefill_attn.py:87-184): same signature, same ``(attn_output[B,N,H,D],
attn_weights)`` return.  Differences that do not change results: K/V are never repeated to
the query head count (the kernels map a query head to its KV head) and q/k/v are consumed
through their strides instead of being copied to ``[B,N,H,D]``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import native


def _token_major(x: torch.Tensor) -> torch.Tensor:
    """``[H,N,D]`` (any strides) -> ``[N,H,D]`` view usable by the kernels, copying only if
    the head dimension is not contiguous or rows are not 16-byte aligned."""
    v = x.transpose(0, 1)
    ok = v.stride(2) == 1 and v.stride(0) % 8 == 0 and v.stride(1) % 8 == 0 and v.data_ptr() % 16 == 0
    return v if ok else v.contiguous()


def sparse_prefill_attention(sharing, q, k, v, layer_idx: int, num_heads: int, config, scale: float):
    """One layer of prefill for batch element views q ``[N,H,D]``, k/v ``[N,Hkv,D]``."""
    block_size = config.block_size
    min_budget = 1 if config.min_budget is None else config.min_budget
    max_budget = 2**31 - 1 if config.max_budget is None else config.max_budget
    pat, use_dense = sharing.get_active_blocks(
        q, k, layer_idx, num_heads, block_size,
        math.ceil(min_budget / block_size), math.ceil(max_budget / block_size),
        config.pattern_threshold, config.similarity_threshold, config.fallback_threshold,
        config.queryaware_threshold, False)
    # layers without a head in a shared cluster cannot elect a pivot: no block-mass pass for them
    state = sharing.state if pat.info.get("can_share", True) else None
    out = native.sparse_attention(q, k, v, pat.bitmap, block_size, scale, pat.flags, pat.slot_of_head, state)
    sharing._mark("attention")
    sharing.update_pivotal_attns(layer_idx, None, use_dense, config.pattern_threshold)
    return out, pat


def shareprefill_attention_core(module, query_states, key_states, value_states, *,
                                gqa_interleave: bool = False):
    bsz, num_heads, q_len, head_dim = query_states.shape
    config = module.config
    softmax_scale = getattr(module, "scaling", 1.0 / math.sqrt(head_dim))
    if gqa_interleave:
        raise NotImplementedError("gqa_interleave=True is not supported by the B200 kernels")

    if q_len != 1:
        if not query_states.is_cuda:
            raise native.SpfError("sparse prefill needs CUDA tensors: there is no CPU fallback")
        assert query_states.dtype == torch.bfloat16
        assert q_len == key_states.shape[2]
        if bsz != 1:
            raise NotImplementedError("the sharing state assumes batch size 1")
        q = _token_major(query_states[0])
        k = _token_major(key_states[0])
        v = _token_major(value_states[0])
        out, pat = sparse_prefill_attention(module.attention_sharing, q, k, v, module.layer_idx,
                                            num_heads, config, softmax_scale)
        attn_weights = None
        if getattr(config, "output_attentions", False):
            attn_weights = dense_avg_attn(module.attention_sharing, pat, num_heads)
        return out[None], attn_weights

    # decode step (one query token): dense attention over the cache with the split-K decode kernel;
    # the reference calls flash_attn_func here (attn/shareprefill_attn.py:146-153), which takes bf16 /
    # fp16 only and applies attention dropout in training mode.  This path has one kernel and no
    # library fallback: dropout (training with attention_dropout > 0) and other dtypes are refused.
    dropout = float(getattr(module, "attention_dropout", 0.0) or 0.0) if module.training else 0.0
    if (query_states.is_cuda and query_states.dtype == torch.bfloat16 and dropout == 0.0
            and head_dim in (64, 128)):
        outs = []
        for b in range(bsz):
            outs.append(native.decode_attention(query_states[b, :, 0, :], _token_major(key_states[b]),
                                                _token_major(value_states[b]), softmax_scale))
        return torch.stack(outs)[:, None], None
    raise native.SpfError(
        "decode step: the B200 kernel needs CUDA bfloat16 tensors, head_dim 64 or 128 and no attention "
        f"dropout (got {query_states.dtype} on {query_states.device}, head_dim {head_dim}, dropout {dropout})")


def dense_avg_attn(sharing, pat, num_heads: int) -> torch.Tensor:
    """The reference's ``avg_attn [1,H,nb,nb]`` (zeros except for this layer's pivots)."""
    nb = pat.num_blocks
    out = torch.zeros(1, num_heads, nb, nb, dtype=torch.float32, device=pat.bitmap.device)
    st = sharing.state
    if st is not None and st.n_slots:
        piv = torch.nonzero(pat.flags & native.HEAD_PIVOT).flatten().tolist()
        slots = pat.slot_of_head.tolist()
        attn = st.field("pivot_attn")
        for h in piv:
            out[0, h] = attn[slots[h]]
    return out


def shareprefill_attention_forward(module, query_states, key_states, value_states,
                                   attention_mask: Optional[torch.Tensor], *, scaling: float = None,
                                   dropout: float = 0.0, **kwargs) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Hugging Face attention interface: q ``[B,H,N,D]``, k/v ``[B,Hkv,N,D]`` ->
    ``(attn_output [B,N,H,D] contiguous, attn_weights or None)``.  ``attention_mask``,
    ``scaling`` and ``dropout`` are ignored as in the reference (the scale is read from
    ``module.scaling``)."""
    sliding_window = kwargs.pop("sliding_window", None)
    if sliding_window is not None:
        raise NotImplementedError("SharePrefill attention does not support sliding-window mode yet.")
    gqa_interleave = kwargs.pop("gqa_interleave", False)
    return shareprefill_attention_core(module, query_states, key_states, value_states,
                                       gqa_interleave=gqa_interleave)
