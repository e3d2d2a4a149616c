"""Loader for the golden vectors under tests/golden (made by make_golden.py)."""
import hashlib
import json
import math
import os

import numpy as np
import torch

from shareprefill_b200.workloads import AttentionWorkload, make_qkv

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASE_NAMES = ["peaky_share", "peaky_default", "diffuse_qa", "ragged_rope"]


class GoldenCase:
    def __init__(self, name):
        self.name = name
        self.z = np.load(os.path.join(GOLDEN_DIR, f"{name}.npz"))
        meta = json.loads(str(self.z["meta"]))
        self.wl = AttentionWorkload(**meta["workload"])
        self.lookup = meta["lookup"]
        self.bs = self.wl.block_size
        self.nb = self.wl.num_blocks
        self.min_blocks = math.ceil(self.wl.min_budget / self.bs)
        mx = 2**31 - 1 if self.wl.max_budget is None else self.wl.max_budget
        self.max_blocks = math.ceil(mx / self.bs)

    def knobs(self):
        wl = self.wl
        return dict(block_size=wl.block_size, min_blocks=self.min_blocks, max_blocks=self.max_blocks,
                    pattern_threshold=wl.pattern_threshold, similarity_threshold=wl.similarity_threshold,
                    fallback_threshold=wl.fallback_threshold, queryaware_threshold=wl.queryaware_threshold)

    def t(self, key):
        return torch.from_numpy(self.z[key])

    def has(self, key):
        return key in self.z.files

    def sets(self, layer):
        lens = self.z[f"L{layer}_set_len"].tolist()
        cat = self.t(f"L{layer}_set_cat")
        out, o = [], 0
        for n in lens:
            out.append(cat[o:o + n])
            o += n
        return out

    def qkv(self, layer):
        q, k, v = make_qkv(self.wl, layer, dtype=torch.bfloat16)
        hsh = hashlib.sha256()
        for t in (q, k, v):
            hsh.update(t.contiguous().view(torch.uint8).numpy().tobytes())
        want = bytes(self.z[f"L{layer}_digest"].tolist()).hex()
        assert hsh.hexdigest() == want, "seeded generator no longer reproduces the golden inputs"
        return q, k, v

    def qa_scores(self, layer):
        heads = self.z[f"L{layer}_qa_heads"].tolist()
        if not heads:
            return {}
        sc = self.t(f"L{layer}_qa_scores")
        return {h: sc[i] for i, h in enumerate(heads)}

    def avg_attn(self, layer):
        heads = self.z[f"L{layer}_dense_heads"].tolist()
        if not heads:
            return {}
        a = self.t(f"L{layer}_avg_attn")
        return {h: a[i] for i, h in enumerate(heads)}


# ----------------------------------------------------------------------------- benchmark-sized cases
SCALE_CASE_NAMES = ["qa_8k", "mixed_8k", "qwen_8k", "llama70b_8k", "llama_32k", "llama_32k_diffuse", "group_128k"]


def shipped_lookup_path():
    from shareprefill_b200.configuration import SharePrefillConfig
    return SharePrefillConfig(model_name="Llama-3.1-8B-Instruct").sharing_lookup_path


def bitmap_to_sets_cpu(bm: torch.Tensor, nb: int):
    """uint32-as-int64 ``[H][nb][nbw]`` -> per-head sorted flat indices ``row*nb+col``."""
    h, _, nbw = bm.shape
    bits = (bm.to(torch.int64).unsqueeze(-1) >> torch.arange(32)) & 1
    dense = bits.reshape(h, nb, nbw * 32)[:, :, :nb].bool()
    return [torch.nonzero(dense[i].reshape(-1)).flatten() for i in range(h)]


class ScaleCase(GoldenCase):
    """A case at a benchmark configuration's size: the reference's results for every head and its
    un-pooled scores for ``score_heads`` (see make_golden.py, SCALE_CASES)."""

    def __init__(self, name):
        super().__init__(name)
        meta = json.loads(str(self.z["meta"]))
        self.layers = meta["layers"]
        self.score_heads = meta["score_heads"]
        self.all_scores = self.score_heads == list(range(self.wl.num_q_heads))
        if self.lookup == "shipped":
            from shareprefill_b200.sharing_state import load_lookup
            clusters, shared = load_lookup(shipped_lookup_path())
            self.lookup = {"clusters": clusters, "shared_clusters": sorted(shared)}
            self.lookup_file = shipped_lookup_path()
        else:
            self.lookup_file = None

    def bitmap(self, layer):
        """int64 tensor holding the uint32 words ``[H][nb][nbw]``."""
        return torch.from_numpy(self.z[f"L{layer}_bitmap"].astype(np.int64))

    def bitmap_i32(self, layer):
        return torch.from_numpy(self.z[f"L{layer}_bitmap"].view(np.int32))

    def sets(self, layer):
        return bitmap_to_sets_cpu(self.bitmap(layer), self.nb)

    def qa_scores(self, layer):
        heads = self.z[f"L{layer}_qa_score_heads"].tolist()
        if not heads:
            return {}
        sc = self.t(f"L{layer}_qa_scores")
        return {h: sc[i] for i, h in enumerate(heads)}

    def shared_ids(self):
        return [str(c) for c in self.z["shared_ids"].tolist()]


def same_cover_up_to_ties(got: torch.Tensor, want: torch.Tensor, scores: torch.Tensor) -> bool:
    """Are two selections of one head (bool ``[nb*nb]``) the same cumulative-mass cover of ``scores``
    (fp32 ``[nb*nb]``)?  The reference keeps a prefix of ``torch.sort(descending=True)``; several blocks
    may share the score at which the running sum crosses the threshold (equal bf16 logits in one
    softmax row give equal fp32 scores), and torch's default sort leaves the order of equal values
    open - on CPU it is not index order.  So two covers are the same selection when they hold equally
    many blocks and differ only among blocks whose score is that one crossing value."""
    diff = got ^ want
    if not bool(diff.any()):
        return True
    vals = scores[diff]
    return int(got.sum()) == int(want.sum()) and bool((vals == vals[0]).all())


def bitmap_row_bools(bm_words: torch.Tensor, nb: int) -> torch.Tensor:
    """int32/int64 words ``[nb][nbw]`` of one head -> bool ``[nb*nb]``."""
    bits = (bm_words.to(torch.int64).unsqueeze(-1) >> torch.arange(32)) & 1
    return bits.reshape(nb, -1)[:, :nb].bool().reshape(-1)
