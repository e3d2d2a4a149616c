"""CPU-only checks: the C-ABI library loads and exports what the header declares, and the
host-side mirror of the reference API behaves like the reference (no kernels are launched)."""
import ctypes
import json
import os
import re

import pytest
import torch

from conftest import ROOT
from shareprefill_b200 import SharePrefill, native
from shareprefill_b200.configuration import SharePrefillConfig
from shareprefill_b200.sharing_state import AttentionSharing, load_lookup
from shareprefill_b200.workloads import WORKLOADS, make_qkv, synthetic_lookup


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "spf_b200.h")).read()
    declared = set(re.findall(r"\b(spf_[a-z_]+)\s*\(", hdr)) - {"spf_bitmap_words"}
    assert declared == set(native.SIGNATURES), declared ^ set(native.SIGNATURES)
    lib = ctypes.CDLL(native.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    lib = native.load()
    assert lib.spf_version() >= 100
    assert b"NULL" in lib.spf_status_string(-1)


def test_argument_validation_without_a_gpu():
    lib = native.load()
    # null pointers and bad shapes are rejected before anything is launched
    assert lib.spf_pool_qk(None, 0, 0, None, 0, 0, 128, 1, 1, 128, 128, None, None, None) == -1
    assert lib.spf_lastblock_profile(None, 0, 0, None, 0, 0, 128, 1, 1, 128, 128, None, None, None, 0, None) == -1
    assert lib.spf_sharing_state_bytes(1, 10**6) == 0
    assert lib.spf_sharing_state_bytes(2, 64) > 2 * 64 * 64 * 4
    assert lib.spf_lastblock_scratch_bytes(8192, 8, 128) >= 8 * 64 * 128 * 8


def test_state_layout_is_aligned_and_ordered():
    lib = native.load()
    off = (ctypes.c_int64 * 12)()
    assert lib.spf_sharing_state_layout(3, 100, off) == 0
    off = list(off)
    assert off == sorted(off) and all(o % 256 == 0 for o in off)
    assert lib.spf_sharing_state_bytes(3, 100) >= off[-1] + 3 * 100 * 100 * 4


def test_config_defaults_and_errors(tmp_path):
    cfg = SharePrefillConfig(model_name="meta-llama/Llama-3.1-8B-Instruct")
    assert (cfg.pattern_threshold, cfg.similarity_threshold, cfg.fallback_threshold) == (0.9, 0.5, 0.9)
    assert (cfg.queryaware_threshold, cfg.block_size, cfg.min_budget, cfg.max_budget) == (0.1, 128, 1024, None)
    assert os.path.exists(cfg.sharing_lookup_path)
    with pytest.raises(AssertionError):
        SharePrefillConfig(attn_type="other", model_name="x")
    with pytest.raises(AssertionError):
        SharePrefillConfig(model_name="org/unknown-model")
    p = tmp_path / "l.json"
    p.write_text(json.dumps(synthetic_lookup(1, 2, 1)))
    assert SharePrefillConfig(sharing_lookup_path=str(p), model_name="whatever").sharing_lookup_path == str(p)


def test_shipped_lookup_matches_reference_statistics():
    cfg = SharePrefillConfig(model_name="Llama-3.1-8B-Instruct")
    clusters, shared = load_lookup(cfg.sharing_lookup_path)
    assert len(clusters) == 44 and shared == {"9"}
    assert sum(len(v) for v in clusters.values()) == 32 * 32
    assert len(clusters["9"]) == 42 and [14, 17] in clusters["9"]


def test_attention_sharing_lookup(tmp_path):
    with pytest.raises(FileNotFoundError):
        AttentionSharing(str(tmp_path / "missing.json"))
    p = tmp_path / "l.json"
    p.write_text(json.dumps(synthetic_lookup(2, 4, 2, shared=[1], group_size=2)))
    s = AttentionSharing(str(p))
    assert s.find_cluster_id(1, 3) == "1" and s.find_cluster_id(0, 0) == "0"
    assert s.find_cluster_id(5, 0) is None
    assert s._slot_table(0, 4, "cpu").tolist() == [-1, -1, 0, 0]
    with pytest.raises(TypeError):
        s._slot_table(7, 4, "cpu")


def test_bitmap_set_roundtrip():
    nb = 70
    g = torch.Generator().manual_seed(1)
    sets = []
    for _ in range(3):
        m = torch.rand(nb, nb, generator=g) < 0.2
        m = torch.tril(m)
        m[:, 0] = True
        sets.append(torch.nonzero(m.reshape(-1)).flatten())
    bm = native.sets_to_bitmap(sets, nb, "cpu")
    back = native.bitmap_to_sets(bm)
    for a, b in zip(sets, back):
        assert torch.equal(a, b)


def test_workload_generator_is_seeded_and_structured():
    wl = WORKLOADS["cfg0"].replace(seq_len=512)
    q1, k1, v1 = make_qkv(wl, 0, dtype=torch.float32)
    q2, k2, _ = make_qkv(wl, 0, dtype=torch.float32)
    assert torch.equal(q1, q2) and torch.equal(k1, k2)
    assert q1.shape == (512, 8, 128) and k1.shape == (512, 2, 128) and v1.shape == (512, 2, 128)
    q3, _, _ = make_qkv(wl, 1, dtype=torch.float32)
    assert not torch.equal(q1, q3)
    assert k1[:4].mean() > 3.0 > k1[4:].mean().abs()


def _tiny_llama():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=128, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                      max_position_embeddings=4096)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg)


def test_patch_side_effects_and_loud_cpu_failure(tmp_path):
    p = tmp_path / "l.json"
    p.write_text(json.dumps(synthetic_lookup(2, 4, 2, group_size=2)))
    model = _tiny_llama()
    sp = SharePrefill(model_name="tiny", sharing_lookup_path=str(p), block_size=64, min_budget=128,
                      pattern_threshold=0.95)
    out = sp(model)
    assert out is model
    import transformers.models.llama.modeling_llama as ml
    assert "shareprefill" in ml.ALL_ATTENTION_FUNCTIONS
    assert model.config._attn_implementation == "shareprefill"
    assert hasattr(type(model), "reset_attention_sharing") and hasattr(type(model), "_init_attention_sharing")
    sharing = model.reset_attention_sharing()
    assert model.config.block_size == 64 and model.config.pattern_threshold == 0.95
    assert all(l.self_attn.attention_sharing is sharing for l in model.model.layers)
    # no GPU here: the prefill path must refuse to run rather than fall back
    ids = torch.randint(0, 128, (1, 256))
    with pytest.raises(native.SpfError):
        model(ids)
    with pytest.raises(TypeError):
        SharePrefill(model_name="tiny", sharing_lookup_path=str(p))(torch.nn.Linear(2, 2))
    with pytest.raises(FileNotFoundError):
        SharePrefill(model_name="tiny", sharing_lookup_path=str(tmp_path / "nope.json"))(_tiny_llama())
