"""The patched Hugging Face model on a GPU: with budgets that select every block the sparse
path must reproduce eager dense attention."""
import json

import pytest
import torch

from shareprefill_b200 import SharePrefill, native
from shareprefill_b200.workloads import synthetic_lookup

pytestmark = pytest.mark.gpu


def _tiny_llama():
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=128, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                      max_position_embeddings=4096, attn_implementation="eager")
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).to(torch.bfloat16).cuda()


def test_patched_model_matches_eager_when_all_blocks_are_selected(tmp_path):
    p = tmp_path / "l.json"
    p.write_text(json.dumps(synthetic_lookup(2, 4, 2, group_size=2)))
    model = _tiny_llama()
    ids = torch.randint(0, 128, (1, 1000), generator=torch.Generator().manual_seed(1)).cuda()
    with torch.no_grad():
        want = model(ids).logits.float()
    sp = SharePrefill(model_name="tiny", sharing_lookup_path=str(p), block_size=64, min_budget=4096)
    model = sp(model)
    with torch.no_grad():
        got = model(ids).logits.float()
        again = model(ids).logits.float()
    assert torch.equal(got, again), "state must be reset between forwards"
    err = (got - want).abs()
    assert err.max() < 0.15 and err.mean() < 0.01, (err.max().item(), err.mean().item())
    pat = model.attention_sharing.last_pattern
    nb = 16
    assert native.bitmap_row_counts(pat.bitmap)[1].tolist() == [nb * (nb + 1) // 2] * 4


def test_generate_runs_prefill_then_decode(tmp_path):
    p = tmp_path / "l.json"
    p.write_text(json.dumps(synthetic_lookup(2, 4, 2, group_size=2)))
    model = SharePrefill(model_name="tiny", sharing_lookup_path=str(p), block_size=64, min_budget=128)(_tiny_llama())
    ids = torch.randint(0, 128, (1, 300), generator=torch.Generator().manual_seed(2)).cuda()
    with torch.no_grad():
        out = model.generate(ids, max_new_tokens=4, do_sample=False)
    assert out.shape == (1, 304)


def test_latency_driver_runs_on_a_tiny_model():
    from shareprefill_b200 import latency
    res = latency.main(["--model", "tiny", "--lengths", "512,1000", "--num-exp", "1",
                        "--cfg", "block_size=64,min_budget=128,pattern_threshold=0.95"])
    assert [r["length"] for r in res] == [512, 1000] and all(r["seconds"] > 0 for r in res)
