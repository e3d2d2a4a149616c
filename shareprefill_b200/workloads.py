"""Seeded synthetic Q/K/V for the sparse-prefill attention path.

The reference measures on a prompt file tiled to the target length and on real
Llama weights (eval/efficiency/latency.py:21-87); neither travels, so the
benchmark and the parity tests draw Q/K/V from this generator instead.  The
structure it plants is the structure the selection code looks for:

* a low-rank component shared by the heads of one cluster, so that heads of a
  cluster have similar vertical/slash profiles (cross-head sharing),
* a large key bias on the first four tokens (attention sink / vertical line),
* a sinusoidal positional term in Q and K (local / slash structure),
* optionally RoPE on Q and K, as a Llama/Qwen attention layer would apply.

Layout is token-major: q ``[N, H, D]``, k/v ``[N, Hkv, D]``.
"""
from __future__ import annotations

import dataclasses
import json
import math
from typing import Dict, List, Optional, Tuple

import torch

BASE_SEED = 20250519


@dataclasses.dataclass(frozen=True)
class AttentionWorkload:
    """Shape and knobs of one sparse-prefill attention workload."""

    name: str
    cfg_id: int
    seq_len: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int = 128
    num_layers: int = 1
    num_head_clusters: int = 4
    shared_rank: int = 8
    rope_theta: Optional[float] = None
    block_size: int = 128
    min_budget: int = 1024
    max_budget: Optional[int] = None
    pattern_threshold: float = 0.95
    similarity_threshold: float = 0.5
    fallback_threshold: float = 0.9
    queryaware_threshold: float = 0.1
    q_gain: float = 1.0  # >1 sharpens the softmax ("peaky" variant, sparse regime)

    @property
    def num_blocks(self) -> int:
        return -(-self.seq_len // self.block_size)

    @property
    def group_size(self) -> int:
        return self.num_q_heads // self.num_kv_heads

    def replace(self, **kw) -> "AttentionWorkload":
        return dataclasses.replace(self, **kw)


# The five configurations the benchmark contract names.
WORKLOADS: Dict[str, AttentionWorkload] = {
    "cfg0": AttentionWorkload("cfg0", 0, 8192, 8, 2, num_head_clusters=2, shared_rank=4),
    "cfg1": AttentionWorkload("cfg1", 1, 32768, 32, 8, rope_theta=500000.0),
    "cfg2": AttentionWorkload("cfg2", 2, 131072, 32, 8, num_layers=32, rope_theta=500000.0),
    "cfg3": AttentionWorkload("cfg3", 3, 131072, 28, 4, num_layers=28, rope_theta=1e6,
                              min_budget=2048),
    "cfg4": AttentionWorkload("cfg4", 4, 131072, 64, 8, num_layers=80, rope_theta=500000.0),
}


def _rope(x: torch.Tensor, theta: float) -> torch.Tensor:
    """Rotate-half RoPE on ``x[N, H, D]`` with positions 0..N-1."""
    n, _, d = x.shape
    half = d // 2
    inv_freq = theta ** (-torch.arange(0, half, device=x.device, dtype=torch.float32) * 2.0 / d)
    ang = torch.arange(n, device=x.device, dtype=torch.float32)[:, None] * inv_freq[None, :]
    cos = torch.cat((ang.cos(), ang.cos()), dim=-1)[:, None, :]
    sin = torch.cat((ang.sin(), ang.sin()), dim=-1)[:, None, :]
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rot * sin


def make_qkv(
    wl: AttentionWorkload,
    layer: int = 0,
    *,
    dtype: torch.dtype = torch.bfloat16,
    device: str = "cpu",
    seq_len: Optional[int] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Draw q ``[N,H,D]``, k ``[N,Hkv,D]``, v ``[N,Hkv,D]`` for one layer.

    The draw order is fixed (Q, K, V, then per cluster U, Wq, Wk) so that a
    seed names one input on a given device type.  CPU and CUDA generators give
    different streams; parity tests draw on CPU and copy.
    """
    n = wl.seq_len if seq_len is None else seq_len
    h, hkv, d, g = wl.num_q_heads, wl.num_kv_heads, wl.head_dim, wl.group_size
    gen = torch.Generator(device=device)
    gen.manual_seed(BASE_SEED + 1000 * wl.cfg_id + layer)

    def randn(*shape):
        return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32)

    q = randn(n, h, d)
    k = randn(n, hkv, d)
    v = randn(n, hkv, d)
    c, r = wl.num_head_clusters, wl.shared_rank
    for ci in range(c):
        u = randn(n, r)
        wq = randn(r, d)
        wk = randn(r, d)
        q_heads = [hh for hh in range(h) if (hh // g) % c == ci]
        k_heads = [jj for jj in range(hkv) if jj % c == ci]
        if q_heads:
            q[:, q_heads, :] += ((u @ wq) / math.sqrt(r))[:, None, :]
        if k_heads:
            k[:, k_heads, :] += ((u @ wk) / math.sqrt(r))[:, None, :]
    k[0:4] += 4.0
    half = d // 2
    omega = 10000.0 ** (-torch.arange(half, device=device, dtype=torch.float32) * 2.0 / d)
    ang = torch.arange(n, device=device, dtype=torch.float32)[:, None] * omega[None, :]
    pos = torch.cat((ang.sin(), ang.cos()), dim=-1)[:, None, :]
    q += pos
    k += pos
    if wl.rope_theta is not None:
        q = _rope(q, wl.rope_theta)
        k = _rope(k, wl.rope_theta)
    if wl.q_gain != 1.0:
        q = q * wl.q_gain
    return q.to(dtype), k.to(dtype), v.to(dtype)


def synthetic_lookup(
    num_layers: int,
    num_heads: int,
    num_clusters: int,
    shared: Optional[List[int]] = None,
    group_size: int = 1,
) -> dict:
    """A head-cluster lookup covering every (layer, head) pair.

    Same JSON layout the reference loads (attn/attention_sharing.py:368-378):
    ``{"clusters": {id: [[layer, head], ...]}, "shared_clusters": [id, ...]}``.
    Head ``h`` of every layer belongs to cluster ``(h // group_size) % num_clusters``,
    which is the cluster structure ``make_qkv`` plants.
    """
    clusters = {str(ci): [] for ci in range(num_clusters)}
    for layer in range(num_layers):
        for hh in range(num_heads):
            clusters[str((hh // group_size) % num_clusters)].append([layer, hh])
    if shared is None:
        shared = list(range(num_clusters))
    return {"clusters": clusters, "shared_clusters": [str(s) for s in shared]}


def write_lookup(path: str, lookup: dict) -> str:
    with open(path, "w") as f:
        json.dump(lookup, f)
    return path
