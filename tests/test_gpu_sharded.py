"""Head sharding on one GPU: two shards (each with its own sharing state and only its own
heads' q/k/v) must reproduce the single-shard run bit for bit - patterns, flags and outputs.
The two NCCL all-gathers are replaced by local concatenation / stacking of the shards' tensors;
everything else is the production code path."""
import json
import math

import pytest
import torch

from golden_cases import GoldenCase
from shareprefill_b200 import native
from shareprefill_b200.sharded import kv_group_shard, merge_pivot_summaries, pack_pivot_summaries
from shareprefill_b200.sharing_state import AttentionSharing

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("exchange", ["kernels", "torch"])
@pytest.mark.parametrize("name", ["peaky_share", "ragged_rope", "peaky_default"])
def test_two_shards_equal_one(name, exchange, tmp_path):
    dev = torch.device("cuda:0")
    gc = GoldenCase(name)
    wl = gc.wl
    path = tmp_path / "lookup.json"
    path.write_text(json.dumps(gc.lookup))
    scale = 1.0 / math.sqrt(wl.head_dim)
    kn = dict(similarity_threshold=wl.similarity_threshold, fallback_threshold=wl.fallback_threshold,
              queryaware_threshold=wl.queryaware_threshold)
    world = 2
    shards = [kv_group_shard(wl.num_q_heads, wl.num_kv_heads, r, world) for r in range(world)]
    single = AttentionSharing(str(path))
    parts = [AttentionSharing(str(path), head_range=(s[0], s[1])) for s in shards]
    for layer in range(wl.num_layers):
        q, k, v = (t.to(dev) for t in gc.qkv(layer))
        # reference: all heads in one instance
        pat, dense = single.get_active_blocks(q[None], k[None], layer, wl.num_q_heads, gc.bs, gc.min_blocks,
                                              gc.max_blocks, wl.pattern_threshold, **kn)
        out = native.sparse_attention(q, k, v, pat.bitmap, gc.bs, scale, pat.flags, pat.slot_of_head, single.state)
        single.update_pivotal_attns(layer, None, dense, wl.pattern_threshold)
        # shards: per-head phase on every shard, then the "all-gather", then the cross-head phase
        ctxs = []
        for (h0, h1, k0, k1), sh in zip(shards, parts):
            ctxs.append(sh.profile_heads(q[:, h0:h1], k[:, k0:k1], layer, wl.num_q_heads, gc.bs, gc.min_blocks,
                                         gc.max_blocks, wl.pattern_threshold))
        jsd_all = torch.cat([c["jsd_qa"] for c in ctxs])
        outs, pats = [], []
        for (h0, h1, k0, k1), sh, ctx in zip(shards, parts, ctxs):
            sp, sd = sh.select_blocks(ctx, jsd_all, **kn)
            outs.append(native.sparse_attention(q[:, h0:h1], k[:, k0:k1], v[:, k0:k1], sp.bitmap, gc.bs, scale,
                                                sp.flags, sp.slot_of_head, sh.state))
            sh.update_pivotal_attns(layer, None, sd, wl.pattern_threshold)
            pats.append(sp)
        want = torch.stack([pack_pivot_summaries(sh.state, layer, s[0], s[1]) for s, sh in zip(shards, parts)])
        if exchange == "kernels":   # the pack / merge kernels the NCCL path uses
            gathered = torch.stack([native.pack_pivot_summaries(sh.state, layer, s[0], s[1])
                                    for s, sh in zip(shards, parts)])
            sent = want[:, :, 0] > 0
            assert torch.equal(gathered[:, :, 0], want[:, :, 0]), "flags differ from the torch packing"
            assert torch.equal(gathered[sent], want[sent]), "packed rows differ from the torch packing"
            for sh in parts:
                native.merge_pivot_summaries(sh.state, gathered)
        else:
            for sh in parts:
                merge_pivot_summaries(sh.state, want)
        assert torch.equal(torch.cat([p.bitmap for p in pats]), pat.bitmap), f"layer {layer}: patterns differ"
        assert torch.equal(torch.cat([p.flags for p in pats]), pat.flags), f"layer {layer}: flags differ"
        assert torch.equal(torch.cat(outs, dim=1), out), f"layer {layer}: outputs differ"
    # every shard ends with the same view of the shared clusters as the single instance
    for name_ in ("pivot_head", "pattern_ready", "pattern", "pivot_vertical", "pivot_slash"):
        for sh in parts:
            assert torch.equal(sh.state.field(name_), single.state.field(name_)), name_
    r0 = single.state.field("vs_ratio")
    for sh in parts:
        r = sh.state.field("vs_ratio")
        assert torch.equal(torch.isnan(r), torch.isnan(r0)) and torch.equal(r[~torch.isnan(r)], r0[~torch.isnan(r0)])
