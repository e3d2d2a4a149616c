"""Whole-model prefill latency sweep, the protocol of the reference's latency driver
(eval/efficiency/latency.py:21-100): for each prompt length one warm-up forward, then the mean
wall-clock time of ``num_exp`` forwards with ``use_cache=False``, CUDA-synchronised on both sides.

The reference tiles a downloaded prompt file and loads Llama-3.1-8B-Instruct weights; neither is
available offline, so the model is a random-init Hugging Face Llama of a named shape and the
prompt is a seeded uniform-random token sequence.  ``--attn sdpa`` runs the unpatched model for
comparison.

    python -m shareprefill_b200.latency --model llama-3.1-8b --lengths 8192,32768,131072 --num-exp 3
"""
from __future__ import annotations

import argparse
import gc
import json
import time

import torch

SHAPES = {
    # name: hidden, layers, q heads, kv heads, head_dim, ffn, vocab, rope theta
    "llama-3.1-8b": (4096, 32, 32, 8, 128, 14336, 128256, 500000.0),
    "llama-3.1-70b": (8192, 80, 64, 8, 128, 28672, 128256, 500000.0),
    "qwen2.5-7b-shape": (3584, 28, 28, 4, 128, 18944, 152064, 1000000.0),
    "tiny": (256, 2, 4, 2, 64, 512, 128, 10000.0),
}


def build_model(name: str, max_len: int, attn: str, seed: int = 0):
    from transformers import LlamaConfig, LlamaForCausalLM
    hid, layers, hq, hkv, hd, ffn, vocab, theta = SHAPES[name]
    cfg = LlamaConfig(vocab_size=vocab, hidden_size=hid, intermediate_size=ffn, num_hidden_layers=layers,
                      num_attention_heads=hq, num_key_value_heads=hkv, head_dim=hd, rope_theta=theta,
                      max_position_embeddings=max(max_len, 8192), initializer_range=0.02,
                      attn_implementation="sdpa" if attn == "sdpa" else "eager")
    torch.manual_seed(seed)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device("cuda"):
            model = LlamaForCausalLM(cfg)
    finally:
        torch.set_default_dtype(old)
    return model.eval()


def synthetic_lookup_file(layers: int, heads: int, group: int) -> str:
    import tempfile
    from .workloads import synthetic_lookup
    f = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
    json.dump(synthetic_lookup(layers, heads, 4, shared=[1], group_size=group), f)
    f.close()
    return f.name


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b", choices=sorted(SHAPES))
    ap.add_argument("--lengths", default="1024,8192,16384,32768,65536,131072")
    ap.add_argument("--num-exp", type=int, default=3)
    ap.add_argument("--attn", default="shareprefill", choices=["shareprefill", "sdpa"])
    ap.add_argument("--cfg", default="block_size=128,min_budget=1024,pattern_threshold=0.95,"
                                     "similarity_threshold=0.5,fallback_threshold=0.95")
    args = ap.parse_args(argv)
    lengths = [int(x) for x in args.lengths.split(",")]
    model = build_model(args.model, max(lengths), args.attn)
    hid, layers, hq, hkv, hd, ffn, vocab, theta = SHAPES[args.model]
    if args.attn == "shareprefill":
        from . import SharePrefill
        kw = {}
        for item in args.cfg.split(","):
            k_, v_ = item.split("=")
            kw[k_] = float(v_) if "." in v_ else int(v_)
        if args.model == "llama-3.1-8b":
            model = SharePrefill(model_name="Llama-3.1-8B-Instruct", **kw)(model)
        else:
            model = SharePrefill(model_name=args.model, sharing_lookup_path=synthetic_lookup_file(layers, hq, hq // hkv),
                                 **kw)(model)
    gen = torch.Generator().manual_seed(1)
    results = []
    for n in lengths:
        ids = torch.randint(0, vocab, (1, n), generator=gen).cuda()
        mask = torch.ones_like(ids)
        try:
            with torch.no_grad():
                model(ids, attention_mask=mask, use_cache=False, logits_to_keep=1)
                times = []
                for _ in range(args.num_exp):
                    torch.cuda.empty_cache()
                    gc.collect()
                    torch.cuda.synchronize()
                    t0 = time.time()
                    model(ids, attention_mask=mask, use_cache=False, logits_to_keep=1)
                    torch.cuda.synchronize()
                    times.append(time.time() - t0)
        except torch.cuda.OutOfMemoryError:
            print(f"length {n}: out of memory")
            break
        mean = sum(times) / len(times)
        results.append({"length": n, "seconds": mean})
        print(f"{args.attn} {args.model} length {n}: {mean:.4f} s")
    print(json.dumps({"model": args.model, "attn": args.attn, "num_exp": args.num_exp, "results": results}))
    return results


if __name__ == "__main__":
    main()
