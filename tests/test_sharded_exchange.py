"""Head sharding plumbing on CPU: shard arithmetic and the two per-layer exchanges over gloo with
two ranks (the device kernels are not involved; the state is a CPU stand-in with the same fields)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from shareprefill_b200.sharded import (HeadShardExchange, kv_group_shard, merge_pivot_summaries,
                                        pack_pivot_summaries)


class FakeState:
    def __init__(self, n_slots, nb):
        self.n_slots, self.nb = n_slots, nb
        nbw = (nb + 31) // 32
        s = n_slots
        self.t = {
            "pivot_head": torch.full((s,), -1, dtype=torch.int32), "pivot_layer": torch.full((s,), -1, dtype=torch.int32),
            "pattern_ready": torch.zeros(s, dtype=torch.int32), "vs_ratio": torch.full((s,), float("nan")),
            "pivot_vertical": torch.zeros(s, nb), "pivot_slash": torch.zeros(s, nb),
            "pattern": torch.zeros(s, nb, nbw, dtype=torch.int32),
        }

    def field(self, name):
        return self.t[name]


class FakeSharing:
    def __init__(self, state):
        self.state = state


def test_kv_group_shard():
    assert kv_group_shard(32, 8, 0, 8) == (0, 4, 0, 1)
    assert kv_group_shard(32, 8, 7, 8) == (28, 32, 7, 8)
    assert kv_group_shard(28, 4, 1, 2) == (14, 28, 2, 4)
    assert kv_group_shard(64, 8, 3, 4) == (48, 64, 6, 8)
    with pytest.raises(ValueError):
        kv_group_shard(28, 4, 0, 8)      # a 7-head group cannot be split


def test_pack_and_merge_locally():
    nb = 40
    a, b = FakeState(2, nb), FakeState(2, nb)
    for st in (a, b):                       # both ranks agree on who the pivots are
        st.t["pivot_head"][:] = torch.tensor([1, 6], dtype=torch.int32)
        st.t["pivot_layer"][:] = torch.tensor([3, 3], dtype=torch.int32)
    a.t["vs_ratio"][0] = 0.25; a.t["pivot_vertical"][0] = torch.rand(nb); a.t["pattern"][0] = 7
    b.t["vs_ratio"][1] = 17.5; b.t["pivot_slash"][1] = torch.rand(nb); b.t["pattern"][1] = -5
    g = torch.stack([pack_pivot_summaries(a, 3, 0, 4), pack_pivot_summaries(b, 3, 4, 8)])
    for st in (a, b):
        merge_pivot_summaries(st, g)
        assert st.t["pattern_ready"].tolist() == [1, 1]
        assert st.t["vs_ratio"].tolist() == [0.25, 17.5]
        assert (st.t["pattern"][0] == 7).all() and (st.t["pattern"][1] == -5).all()
    assert torch.equal(a.t["pivot_vertical"], b.t["pivot_vertical"])
    assert torch.equal(a.t["pivot_slash"], b.t["pivot_slash"])
    # a layer without new pivots changes nothing
    before = {k: v.clone() for k, v in a.t.items()}
    g = torch.stack([pack_pivot_summaries(a, 4, 0, 4), pack_pivot_summaries(b, 4, 4, 8)])
    merge_pivot_summaries(a, g)
    for k, v in before.items():
        assert torch.equal(v, a.t[k], ) or (k == "vs_ratio")


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        h0, h1, _, _ = kv_group_shard(8, 2, rank, world)
        ex = HeadShardExchange(h0, h1)
        local = torch.arange(h0, h1, dtype=torch.float32) * 0.5
        allv = ex.gather_heads(local)
        assert torch.equal(allv, torch.arange(8, dtype=torch.float32) * 0.5)
        nb = 33
        st = FakeState(2, nb)
        st.t["pivot_head"][:] = torch.tensor([2, 5], dtype=torch.int32)     # slot 0 -> rank 0, slot 1 -> rank 1
        st.t["pivot_layer"][:] = torch.tensor([1, 1], dtype=torch.int32)
        mine = rank                                                          # the slot this rank owns
        st.t["vs_ratio"][mine] = 1.5 + rank
        st.t["pivot_vertical"][mine] = torch.full((nb,), float(rank + 1))
        st.t["pattern"][mine] = rank + 10
        ex.share_new_pivots(FakeSharing(st), 1)
        assert st.t["pattern_ready"].tolist() == [1, 1]
        assert st.t["vs_ratio"].tolist() == [1.5, 2.5]
        assert (st.t["pattern"][0] == 10).all() and (st.t["pattern"][1] == 11).all()
        assert (st.t["pivot_vertical"][1] == 2.0).all()
        results[rank] = 1
    finally:
        dist.destroy_process_group()


def test_exchange_over_gloo_two_ranks():
    world = 2
    port = 29500 + (os.getpid() % 500)
    with mp.Manager() as m:
        results = m.dict()
        mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: 1, 1: 1}
