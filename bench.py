"""Benchmark of the sparse-prefill attention path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload cfg2]

One step = one pass of the whole path (pooling, last-block profile, selection, block-sparse
attention, pivot update) over all layers of the workload, layers in order, sharing state
carried from layer to layer and reset at the start of the step.  The default workload is the
128K-token Llama-3.1-8B attention shape (32 query / 8 KV heads, head_dim 128, 32 layers);
Q/K/V are synthetic (shareprefill_b200.workloads) and distinct per layer.

The JSON line carries: ``value`` = ms per step with inputs resident in HBM; ``e2e`` = the same
step driven from pinned HOST buffers (q/k/v copied in per layer, the attention output copied
back per layer, copies overlapped with compute on side streams); ``roofline`` for the
dominant kernel (block-sparse attention, tensor bound) and ``roofline_pool`` for the pooling
kernel (HBM bound); ``cpu_baseline`` = the CPU oracle timed on a bounded sample of the same
workload and extrapolated to a full step.

``--impl reference`` times the reference's algorithm on the host cores only (the CPU oracle,
a port: the reference's Triton kernels cannot run on a CPU), same metric and config.
With N > 1 (torchrun) heads are sharded by KV group; total work is fixed (strong scaling).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from shareprefill_b200.workloads import WORKLOADS, AttentionWorkload, make_qkv, synthetic_lookup  # noqa: E402

STAGES = ["pool", "profile", "select", "attention", "pivot_update"]
DISTINCT_LAYER_INPUTS = 4   # host/device inputs are drawn for this many layers and cycled
# DRAM bytes (read + write) of ONE launch of the block-sparse attention kernel, from ncu captures of
# these workloads on one GPU (profiles/sparse_attn_tc5_cfg1_and_cfg2.md); None where not captured
ATTENTION_DRAM_BYTES_PER_LAUNCH = {("cfg2", 131072, 1.0): 3039617280 + 1056879104,
                                   ("cfg1", 32768, 1.0): 403427072 + 234135296}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm_gbs=d["hbm_gbs"], tflops=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured (MEASURED_PEAKS.json, sustained bf16)")
    return dict(hbm_gbs=6650.0, tflops=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def knobs(wl: AttentionWorkload):
    return dict(block_size=wl.block_size, min_budget=wl.min_budget, max_budget=wl.max_budget,
                pattern_threshold=wl.pattern_threshold, similarity_threshold=wl.similarity_threshold,
                fallback_threshold=wl.fallback_threshold, queryaware_threshold=wl.queryaware_threshold)


def workload_lookup(wl: AttentionWorkload) -> str:
    """Lookup file for the workload: the shipped Llama-3.1-8B table for 32x32 models, a synthetic
    one matching the generator's head clusters otherwise."""
    from shareprefill_b200.configuration import SharePrefillConfig
    if wl.num_q_heads == 32 and wl.num_layers <= 32:
        return SharePrefillConfig(model_name="Llama-3.1-8B-Instruct").sharing_lookup_path
    lk = synthetic_lookup(wl.num_layers, wl.num_q_heads, wl.num_head_clusters, shared=[1],
                          group_size=wl.group_size)
    f = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
    json.dump(lk, f)
    f.close()
    return f.name


def config_dict(wl: AttentionWorkload, n_gpus: int):
    return {"workload": f"{wl.name}: sparse-prefill attention path, {wl.num_layers} layers x "
                        f"(N={wl.seq_len}, {wl.num_q_heads}q/{wl.num_kv_heads}kv heads, D={wl.head_dim}, bf16)",
            "seq_len": wl.seq_len, "layers": wl.num_layers, "q_heads": wl.num_q_heads,
            "kv_heads": wl.num_kv_heads, "head_dim": wl.head_dim, **knobs(wl),
            "q_gain": wl.q_gain, "inputs": f"synthetic, {DISTINCT_LAYER_INPUTS} distinct layer inputs cycled",
            "l2": "per-layer inputs are larger than L2 (no flush needed)",
            "parallelism": "single GPU" if n_gpus == 1 else f"heads sharded by KV group over {n_gpus} GPUs"}


# ------------------------------------------------------------------------------ CPU arm
def cpu_sample(wl: AttentionWorkload, rows_per_head: int = 3, seed_layer: int = 0):
    """Time the CPU oracle on one layer, one KV group of the workload: selection in full,
    attention on a few query-block rows per head; extrapolate to a full step."""
    from oracle import spf_oracle as orc
    g = wl.group_size
    sub = wl.replace(num_q_heads=g, num_kv_heads=1)
    q, k, v = make_qkv(sub, seed_layer, dtype=torch.bfloat16)
    lookup = synthetic_lookup(1, g, 1, shared=[])
    st = orc.SharingOracle(lookup)
    bs, nb = wl.block_size, wl.num_blocks
    t0 = time.perf_counter()
    sets, use_dense, _ = st.get_active_blocks(
        q, k, 0, block_size=bs, min_blocks=math.ceil(wl.min_budget / bs),
        max_blocks=2**31 - 1, pattern_threshold=wl.pattern_threshold,
        similarity_threshold=wl.similarity_threshold, fallback_threshold=wl.fallback_threshold,
        queryaware_threshold=wl.queryaware_threshold)
    t_sel = time.perf_counter() - t0
    rows = sorted({nb - 1, nb // 2, nb // 5, 1}.__iter__())[-rows_per_head:]
    visited_total = sum(len(s) for s in sets)
    sampled = 0
    for s in sets:
        r = torch.div(s, nb, rounding_mode="floor")
        sampled += int(sum((r == x).sum() for x in rows))
    t0 = time.perf_counter()
    orc.sparse_attention(q, k, v, sets, use_dense, bs, rows=rows)
    t_attn = time.perf_counter() - t0
    groups = wl.num_kv_heads
    per_layer = t_sel * groups + t_attn * (visited_total / max(sampled, 1)) * groups
    return dict(ms_per_step=per_layer * wl.num_layers * 1e3, t_select_s=t_sel, t_attn_sample_s=t_attn,
                sampled_blocks=sampled, visited_blocks_group=visited_total,
                sample=f"1 layer, 1 KV group ({g} query heads) of the workload: selection in full, attention on "
                       f"query-block rows {rows} ({sampled} of {visited_total} visited blocks), scaled by "
                       f"visited blocks x {groups} groups x {wl.num_layers} layers (extrapolated)")


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = torch.get_num_threads()
    vals = []
    for i in range(args.warmup + args.steps):
        s = cpu_sample(wl, rows_per_head=2, seed_layer=i % DISTINCT_LAYER_INPUTS)
        if i >= args.warmup:
            vals.append(s)
    ms = sum(v["ms_per_step"] for v in vals) / len(vals)
    line = {"impl": "reference", "metric": "sparse_prefill_attention_ms_per_forward", "value": ms, "unit": "ms",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": config_dict(wl, args.gpus),
            "cpu_baseline": {"value": ms, "unit": "ms", "cores": cores, "kind": "port", "sample": vals[-1]["sample"]},
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------ reference on the GPU
def run_reference_triton_arm(args, wl):
    """Informational arm: the UNMODIFIED reference (its torch selection code and Triton kernels, from
    the offline install under baseline/_ref) on the same GPU and the same inputs, one GPU only.
    Not the contract's reference arm (that one is the CPU port); it shows the incumbent GPU path."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "shareprefill")):
        print(json.dumps({"impl": "reference-triton", "unavailable": "baseline/_ref is not installed"}))
        return
    sys.path.insert(0, ref_dir)
    from shareprefill.attn import shareprefill_attn as ref_attn
    from shareprefill.attn.attention_sharing import AttentionSharing as RefSharing
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    lookup_path = workload_lookup(wl)
    if lookup_path.endswith("_table.json"):      # the reference reads its own JSON layout only
        from shareprefill_b200.clusters.convert_lookup import from_table
        with open(lookup_path) as f:
            lk = from_table(json.load(f))
        tmp = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
        json.dump(lk, tmp)
        tmp.close()
        lookup_path = tmp.name
    sharing = RefSharing(lookup_path)
    L, nd, g = wl.num_layers, min(DISTINCT_LAYER_INPUTS, wl.num_layers), wl.group_size
    bs = wl.block_size
    inputs = []
    for i in range(nd):
        q, k, v = make_qkv(wl, i, device="cuda")
        inputs.append((q[None].contiguous(), k.repeat_interleave(g, dim=1)[None].contiguous(),
                       v.repeat_interleave(g, dim=1)[None].contiguous()))
    stage = {"select": 0.0, "attention": 0.0, "pivot_update": 0.0}

    def step(record):
        sharing.reset_state()
        for layer in range(L):
            q, k, v = inputs[layer % nd]
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record()
            block_idx, use_dense = sharing.get_active_blocks(
                q, k, layer, wl.num_q_heads, bs, math.ceil(wl.min_budget / bs), 2**31 - 1,
                wl.pattern_threshold, wl.similarity_threshold, wl.fallback_threshold, wl.queryaware_threshold, False)
            ev[1].record()
            o, avg = ref_attn.triton_block_wise_prefill_attention(q, k, v, block_idx, use_dense, bs)
            ev[2].record()
            sharing.update_pivotal_attns(layer, avg, use_dense, wl.pattern_threshold)
            ev[3].record()
            if record:
                torch.cuda.synchronize()
                for name, a, b in (("select", 0, 1), ("attention", 1, 2), ("pivot_update", 2, 3)):
                    stage[name] += ev[a].elapsed_time(ev[b])

    for _ in range(args.warmup):
        step(False)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step(True)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    print(json.dumps({"impl": "reference-triton", "metric": "sparse_prefill_attention_ms_per_forward", "value": ms,
                      "unit": "ms", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                      "higher_is_better": False, "dtype": "bf16", "data": "synthetic",
                      "config": config_dict(wl, 1), "stage_ms": {k_: v_ / args.steps for k_, v_ in stage.items()},
                      "note": "K/V repeated to the query-head count as the reference's entry point does; the repeat "
                              "and the [B,N,H,D] copies it makes are outside this timing"}))


# ------------------------------------------------------------------------------ GPU arm
def run_gpu_arm(args, wl):
    import torch.distributed as dist
    from shareprefill_b200 import native
    from shareprefill_b200.attention import sparse_prefill_attention
    from shareprefill_b200.configuration import SharePrefillConfig
    from shareprefill_b200.sharded import HeadShardExchange, kv_group_shard
    from shareprefill_b200.sharing_state import AttentionSharing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    native.load()

    lookup_path = workload_lookup(wl)
    cfg = SharePrefillConfig(model_name="bench", sharing_lookup_path=lookup_path, **knobs(wl))
    hq0, hq1, hk0, hk1 = kv_group_shard(wl.num_q_heads, wl.num_kv_heads, rank, world) if world > 1 else \
        (0, wl.num_q_heads, 0, wl.num_kv_heads)
    exchange = HeadShardExchange(hq0, hq1) if world > 1 else None
    sharing = AttentionSharing(lookup_path, head_range=(hq0, hq1) if world > 1 else None, exchange=exchange)
    scale = 1.0 / math.sqrt(wl.head_dim)
    L = wl.num_layers
    nd = min(DISTINCT_LAYER_INPUTS, L)

    # inputs: drawn on the device (plumbing), this rank's heads only, then mirrored to pinned host
    dev_in = []
    for i in range(nd):
        q, k, v = make_qkv(wl, i, device=str(dev))
        dev_in.append((q[:, hq0:hq1].contiguous(), k[:, hk0:hk1].contiguous(), v[:, hk0:hk1].contiguous()))
        del q, k, v
    torch.cuda.synchronize()

    events = {}

    def on_stage(name):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        events.setdefault("cur", []).append((name, ev))

    def step_resident(record=False):
        sharing.reset_state()
        marks = []
        visited = []
        for layer in range(L):
            q, k, v = dev_in[layer % nd]
            if record:
                events["cur"] = []
                on_stage("begin")
            out, pat = sparse_prefill_attention(sharing, q, k, v, layer, wl.num_q_heads, cfg, scale)
            if record:
                marks.append(events["cur"])
                visited.append((native.bitmap_row_counts(pat.bitmap)[1], pat.flags))
        return marks, visited

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step_resident()
    barrier()
    # host time to ISSUE one step (no synchronisation): tells whether a step is launch bound
    h0 = time.perf_counter()
    step_resident()
    host_issue_ms = (time.perf_counter() - h0) * 1e3
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    sharing.on_stage = on_stage
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = native.LAUNCH_COUNT
    t_begin.record()
    all_marks = []
    for _ in range(args.steps):
        m, visited = step_resident(record=True)
        all_marks.append(m)
    t_end.record()
    launches_timed = native.LAUNCH_COUNT - launches_before
    barrier()
    clocks = sampler.stop()
    sharing.on_stage = None
    ms_step = t_begin.elapsed_time(t_end) / args.steps
    if world > 1:
        t = torch.tensor([ms_step], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t)

    # per-stage device time (this rank), averaged per step
    stage_ms = {s: 0.0 for s in STAGES}
    for m in all_marks:
        for layer_marks in m:
            for (n0, e0), (n1, e1) in zip(layer_marks[:-1], layer_marks[1:]):
                stage_ms[n1] += e0.elapsed_time(e1)
    stage_ms = {k_: v_ / args.steps for k_, v_ in stage_ms.items()}

    # algorithmic work of one step (this rank's heads)
    bs, d = wl.block_size, wl.head_dim
    blocks = 0
    pivot_blocks = 0
    for tot, flags in visited:
        blocks += int(tot.sum())
        pivot_blocks += int(tot[(flags & native.HEAD_PIVOT) != 0].sum())
    flops = blocks * 4.0 * bs * bs * d + pivot_blocks * 2.0 * bs * bs * d
    if world > 1:
        t = torch.tensor([flops, float(blocks)], device=dev, dtype=torch.float64)
        dist.all_reduce(t)
        flops_all, blocks_all = float(t[0]), float(t[1])
    else:
        flops_all, blocks_all = flops, float(blocks)
    peaks = measured_peaks()
    attn_s = stage_ms["attention"] / 1e3
    achieved_tf = flops / attn_s / 1e12 if attn_s > 0 else 0.0
    nq, nkv = hq1 - hq0, hk1 - hk0
    pool_bytes = L * (wl.seq_len * (nq + nkv) * d * 2 + wl.num_blocks * (nq + nkv) * d * 2)
    pool_gbs = pool_bytes / (stage_ms["pool"] / 1e3) / 1e9 if stage_ms["pool"] > 0 else 0.0
    tri = wl.num_blocks * (wl.num_blocks + 1) // 2

    # ---- end to end from pinned host buffers (per-layer H2D of q/k/v, D2H of the output)
    host_in = [tuple(t.cpu().pin_memory() for t in trip) for trip in dev_in]
    n_tok = wl.seq_len
    host_out = [torch.empty(n_tok, nq, d, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    stage_bufs = [tuple(torch.empty_like(t) for t in dev_in[0]) for _ in range(2)]
    out_bufs = [torch.empty(n_tok, nq, d, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    h2d_bytes = L * sum(t.numel() * 2 for t in dev_in[0])
    d2h_bytes = L * n_tok * nq * d * 2

    def step_e2e():
        sharing.reset_state()
        in_ready = [torch.cuda.Event() for _ in range(L)]
        comp_done = [torch.cuda.Event() for _ in range(L)]
        out_done = [torch.cuda.Event() for _ in range(L)]

        def prefetch(layer):
            with torch.cuda.stream(copy_in):
                if layer >= 2:
                    copy_in.wait_event(comp_done[layer - 2])     # staging buffer is free again
                for dst, src in zip(stage_bufs[layer % 2], host_in[layer % nd]):
                    dst.copy_(src, non_blocking=True)
                in_ready[layer].record(copy_in)

        prefetch(0)
        for layer in range(L):
            if layer + 1 < L:
                prefetch(layer + 1)
            main.wait_event(in_ready[layer])
            if layer >= 2:
                main.wait_event(out_done[layer - 2])             # output buffer is free again
            q, k, v = stage_bufs[layer % 2]
            from shareprefill_b200.attention import sparse_prefill_attention as run
            pat_out, _ = run(sharing, q, k, v, layer, wl.num_q_heads, cfg, scale)
            out_bufs[layer % 2].copy_(pat_out)
            comp_done[layer].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(comp_done[layer])
                host_out[layer % 2].copy_(out_bufs[layer % 2], non_blocking=True)
                out_done[layer].record(copy_out)
        main.wait_stream(copy_out)

    e2e_steps = max(1, min(args.steps, 2))
    step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        step_e2e()
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        c = cpu_sample(wl)
        cpu = {"value": c["ms_per_step"], "unit": "ms", "cores": torch.get_num_threads(), "kind": "port",
               "sample": c["sample"]}
    line = {
        "metric": "sparse_prefill_attention_ms_per_forward", "value": ms_step, "unit": "ms",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": config_dict(wl, world),
        "effective_tflops": flops_all / (ms_step / 1e3) / 1e12,
        "visited_block_fraction": blocks_all / (tri * wl.num_q_heads * L),
        "stage_ms_rank0": stage_ms, "host_issue_ms_per_step": host_issue_ms,
        "roofline": {"kernel": "block-sparse attention", "bound": "tensor", "achieved": achieved_tf,
                     "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved_tf / peaks["tflops"],
                     "traffic": ATTENTION_DRAM_BYTES_PER_LAUNCH.get((wl.name, wl.seq_len, wl.q_gain)) if world == 1 else None,
                     "traffic_unit": "bytes per launch (ncu dram read+write)", "of": peaks["source"]},
        "roofline_pool": {"kernel": "Q/K block pooling", "bound": "hbm", "achieved": pool_gbs,
                          "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": pool_gbs / peaks["hbm_gbs"],
                          "traffic": {131072: 1342209280 + 10450176, 32768: 335595008 + 6505472}.get(wl.seq_len)
                          if (world == 1 and wl.num_q_heads == 32 and wl.num_kv_heads == 8) else None,
                          "traffic_unit": "bytes per launch (ncu dram read+write)", "of": peaks["source"]},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
        "gpu_launches": launches_timed,
        "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"])
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--q-gain", type=float, default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    if args.layers:
        wl = wl.replace(num_layers=args.layers)
    if args.seq_len:
        wl = wl.replace(seq_len=args.seq_len)
    if args.q_gain:
        wl = wl.replace(q_gain=args.q_gain)
    if args.impl == "reference":
        run_reference_arm(args, wl)
    elif args.impl == "reference-triton":
        run_reference_triton_arm(args, wl)
    else:
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the sparse-prefill kernels have no CPU fallback")
        run_gpu_arm(args, wl)


if __name__ == "__main__":
    main()
