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

At N = 1 the line also carries, measured after the timed region on ONE layer of the workload:
``incumbent`` = the unmodified reference (its torch selection + Triton kernels, from baseline/_ref)
and torch's dense causal SDPA on the same inputs next to this path; ``sparse_regime`` = one layer
with the queries scaled by 4 (a few percent of the causal blocks visited).

``--impl reference`` times the reference's algorithm on the host cores only: the reference's own
selection code (from baseline/_ref, run on CPU) where it is installed, else its port, plus the
port of the attention kernel (the reference's Triton kernels cannot run on a CPU); same metric and
config, CPU_THREADS host threads in every arm.
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
# host threads of the CPU legs (cpu_baseline, --impl reference): fixed, so that one GPU and a
# torchrun launch (which sets OMP_NUM_THREADS=1) divide by the same denominator
CPU_THREADS = min(16, os.cpu_count() or 1)
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def ncu_dram_bytes(kernel: str, wl) -> "int | None":
    """DRAM bytes (read + write) of ONE launch of ``kernel`` on this workload, from the ncu captures
    tabulated in profiles/ncu_dram_bytes.json; None where that workload was not captured."""
    path = os.path.join(ROOT, "profiles", "ncu_dram_bytes.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        table = json.load(f).get(kernel, {})
    e = table.get(f"{wl.num_q_heads}q{wl.num_kv_heads}kv:{wl.seq_len}:{wl.q_gain:g}")
    return None if e is None else int(e["dram_read_bytes"]) + int(e["dram_write_bytes"])


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
    """Time the reference's CPU path on one layer, one KV group of the workload: selection in full
    (the reference's own get_active_blocks from baseline/_ref where installed, else its port),
    attention (port) on a few query-block rows per head; extrapolate to a full step."""
    from oracle import spf_oracle as orc
    torch.set_num_threads(CPU_THREADS)
    g = wl.group_size
    sub = wl.replace(num_q_heads=g, num_kv_heads=1)
    q, k, v = make_qkv(sub, seed_layer, dtype=torch.bfloat16)
    lookup = synthetic_lookup(1, g, 1, shared=[])
    bs, nb = wl.block_size, wl.num_blocks
    kn = dict(block_size=bs, min_blocks=math.ceil(wl.min_budget / bs), max_blocks=2**31 - 1,
              pattern_threshold=wl.pattern_threshold, similarity_threshold=wl.similarity_threshold,
              fallback_threshold=wl.fallback_threshold, queryaware_threshold=wl.queryaware_threshold)
    kind = "port"
    att = None
    try:
        from oracle.reference_shim import import_reference_selection, reference_get_active_blocks
        att = import_reference_selection(REF_DIR)
    except Exception:  # noqa: BLE001 - not installed, or its imports fail on this box: time the port
        att = None
    if att is not None:
        with tempfile.NamedTemporaryFile("w", suffix=".json", delete=False) as f:
            json.dump(lookup, f)
        ref_state = att.AttentionSharing(f.name)
        os.remove(f.name)
        t0 = time.perf_counter()
        block_idx, dense = reference_get_active_blocks(
            att, ref_state, q, k, 0, g, bs, kn["min_blocks"], kn["max_blocks"], kn["pattern_threshold"],
            kn["similarity_threshold"], kn["fallback_threshold"], kn["queryaware_threshold"])
        t_sel = time.perf_counter() - t0
        sets, use_dense = [block_idx[0][h].to(torch.int64) for h in range(g)], dense[0]
        kind = "ref-selection+port-attention"
    else:
        st = orc.SharingOracle(lookup)
        t0 = time.perf_counter()
        sets, use_dense, _ = st.get_active_blocks(q, k, 0, **kn)
        t_sel = time.perf_counter() - t0
    rows = sorted({nb - 1, nb // 2, nb // 5, 1}.__iter__())[-rows_per_head:]
    visited_total = sum(len(s_) for s_ in sets)
    sampled = 0
    for s_ in sets:
        r = torch.div(s_, nb, rounding_mode="floor")
        sampled += int(sum((r == x).sum() for x in rows))
    t0 = time.perf_counter()
    orc.sparse_attention(q, k, v, sets, use_dense, bs, rows=rows)
    t_attn = time.perf_counter() - t0
    groups = wl.num_kv_heads
    per_layer = t_sel * groups + t_attn * (visited_total / max(sampled, 1)) * groups
    return dict(ms_per_step=per_layer * wl.num_layers * 1e3, t_select_s=t_sel, t_attn_sample_s=t_attn,
                sampled_blocks=sampled, visited_blocks_group=visited_total, kind=kind,
                sample=f"1 layer, 1 KV group ({g} query heads) of the workload on {CPU_THREADS} host threads: "
                       f"selection in full ({'the reference code' if att is not None else 'port'}), attention "
                       f"(port) on query-block rows {rows} ({sampled} of {visited_total} visited blocks), "
                       f"scaled by visited blocks x {groups} groups x {wl.num_layers} layers (extrapolated)")


def run_reference_arm(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(CPU_THREADS)
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
            "cpu_baseline": {"value": ms, "unit": "ms", "cores": cores, "kind": vals[-1]["kind"],
                             "sample": vals[-1]["sample"]},
            "e2e": {"value": ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------ reference on the GPU
def _reference_gpu_modules(wl):
    """The UNMODIFIED reference from baseline/_ref: (AttentionSharing instance, attention module), or a
    string saying why it cannot run."""
    if not os.path.isdir(os.path.join(REF_DIR, "shareprefill")):
        return "baseline/_ref is not installed"
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        from shareprefill.attn import shareprefill_attn as ref_attn
        from shareprefill.attn.attention_sharing import AttentionSharing as RefSharing
    except Exception as e:  # noqa: BLE001
        return f"the reference does not import here: {type(e).__name__}: {e}"
    lookup_path = workload_lookup(wl)
    if lookup_path.endswith("_table.json"):      # the reference reads its own JSON layout only
        from shareprefill_b200.clusters.convert_lookup import from_table
        with open(lookup_path) as f:
            lk = from_table(json.load(f))
        tmp = tempfile.NamedTemporaryFile("w", suffix=".json", delete=False)
        json.dump(lk, tmp)
        tmp.close()
        lookup_path = tmp.name
    return RefSharing(lookup_path), ref_attn


def _reference_gpu_layer(sharing, ref_attn, wl, q, k, v, layer, stage=None):
    """One layer through the reference's own entry points (attn/attention_sharing.py:105-366,
    attn/shareprefill_attn.py:474-620); q/k/v are [1,N,H,D] with K/V already repeated."""
    bs = wl.block_size
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
    if stage is not None:
        torch.cuda.synchronize()
        for name, a, b in (("select", 0, 1), ("attention", 1, 2), ("pivot_update", 2, 3)):
            stage[name] += ev[a].elapsed_time(ev[b])
    return o


def run_reference_triton_arm(args, wl):
    """Informational arm: the UNMODIFIED reference (its torch selection code and Triton kernels, from
    the offline install under baseline/_ref) on the same GPU and the same inputs, one GPU only.
    Not the contract's reference arm (that one runs on the host cores); it shows the incumbent GPU path."""
    mods = _reference_gpu_modules(wl)
    if isinstance(mods, str):
        print(json.dumps({"impl": "reference-triton", "unavailable": mods}))
        return
    sharing, ref_attn = mods
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    L, nd, g = wl.num_layers, min(DISTINCT_LAYER_INPUTS, wl.num_layers), wl.group_size
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
            _reference_gpu_layer(sharing, ref_attn, wl, q, k, v, layer, stage if record else None)

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


def _event_ms(fn, warmup=1, reps=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def one_layer_ours(wl, q, k, v, lookup_path, cfg, reps=3):
    """One layer of this path on resident inputs: (ms, per-stage ms, visited blocks weighted by their
    flops - a pivot's block counts 1.5 -, visited fraction)."""
    from shareprefill_b200 import native
    from shareprefill_b200.attention import sparse_prefill_attention
    from shareprefill_b200.sharing_state import AttentionSharing
    sharing = AttentionSharing(lookup_path)
    scale = 1.0 / math.sqrt(wl.head_dim)
    marks = []

    def run():
        sharing.reset_state()
        return sparse_prefill_attention(sharing, q, k, v, 0, wl.num_q_heads, cfg, scale)

    ms = _event_ms(run, 2, reps)
    sharing.on_stage = lambda name: marks.append((name, _recorded_event()))
    marks.append(("begin", _recorded_event()))
    _, pat = run()
    torch.cuda.synchronize()
    sharing.on_stage = None
    stage = {n1: e0.elapsed_time(e1) for (_, e0), (n1, e1) in zip(marks[:-1], marks[1:])}
    tot = native.bitmap_row_counts(pat.bitmap)[1]
    blocks = int(tot.sum())
    # heads elected pivot in this layer also get the block-mass sweep: half the flops of a visit again
    pivot_blocks = int(tot[(pat.flags & native.HEAD_PIVOT) != 0].sum())
    tri = wl.num_blocks * (wl.num_blocks + 1) // 2
    return ms, stage, blocks + 0.5 * pivot_blocks, blocks / (tri * wl.num_q_heads)


def _recorded_event():
    ev = torch.cuda.Event(enable_timing=True)
    ev.record()
    return ev


def measure_incumbents(wl, lookup_path, cfg, peaks):
    """After the timed region, one GPU, ONE layer of the workload on the same inputs: this path, the
    unmodified reference (torch selection + Triton kernels) and torch's dense causal SDPA; then one
    layer of the sparse regime (queries scaled by 4)."""
    q, k, v = make_qkv(wl, 0, device="cuda")
    ours_ms, ours_stage, blocks, frac = one_layer_ours(wl, q, k, v, lookup_path, cfg)
    inc = {"workload": f"one layer of {wl.name} (N={wl.seq_len}, layer-0 inputs), 1 warm-up + 3 timed passes, CUDA events",
           "ours_ms_per_layer": ours_ms, "ours_stage_ms": ours_stage, "ours_visited_fraction": frac}
    # dense causal attention of the library (every causal block, no selection)
    import torch.nn.functional as F
    qh, kh, vh = (t.transpose(0, 1)[None] for t in (q, k, v))
    backend = "torch default"

    def dense():
        return F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=wl.group_size > 1)

    try:
        from torch.nn.attention import SDPBackend, sdpa_kernel
        with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
            dense_ms = _event_ms(dense)
        backend = "cuDNN"
    except Exception:  # noqa: BLE001 - that backend refuses the shape here: let torch choose
        torch.cuda.synchronize()
        dense_ms = _event_ms(dense)
    tri = wl.num_blocks * (wl.num_blocks + 1) // 2
    dense_flops = tri * wl.num_q_heads * 4.0 * wl.block_size ** 2 * wl.head_dim
    inc.update(dense_sdpa_ms_per_layer=dense_ms, dense_sdpa_backend=backend,
               dense_sdpa_tflops=dense_flops / dense_ms / 1e9)
    # the unmodified reference on the same GPU
    mods = _reference_gpu_modules(wl)
    if isinstance(mods, str):
        inc["triton_reference"] = {"unavailable": mods}
    else:
        sharing, ref_attn = mods
        g = wl.group_size
        rq, rk, rv = (q[None].contiguous(), k.repeat_interleave(g, dim=1)[None].contiguous(),
                      v.repeat_interleave(g, dim=1)[None].contiguous())
        try:
            sharing.reset_state()
            _reference_gpu_layer(sharing, ref_attn, wl, rq, rk, rv, 0)        # warm-up (Triton JIT)
            stage = {"select": 0.0, "attention": 0.0, "pivot_update": 0.0}
            for _ in range(3):
                sharing.reset_state()
                _reference_gpu_layer(sharing, ref_attn, wl, rq, rk, rv, 0, stage)
            stage = {k_: v_ / 3 for k_, v_ in stage.items()}
            inc["triton_reference"] = {"ms_per_layer": sum(stage.values()), "stage_ms": stage}
        except Exception as e:  # noqa: BLE001
            inc["triton_reference"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        del rq, rk, rv
    del q, k, v, qh, kh, vh
    torch.cuda.empty_cache()
    # sparse regime: queries x4
    wl4 = wl.replace(q_gain=4.0)
    q, k, v = make_qkv(wl4, 0, device="cuda")
    ms4, stage4, blocks4, frac4 = one_layer_ours(wl4, q, k, v, lookup_path, cfg)
    tf4 = blocks4 * 4.0 * wl.block_size ** 2 * wl.head_dim / (stage4["attention"] / 1e3) / 1e12
    sparse = {"q_gain": 4, "ms_per_layer": ms4, "stage_ms": stage4, "visited": frac4, "tflops": tf4,
              "frac": tf4 / peaks["tflops"], "of": peaks["source"]}
    return inc, sparse


def bind_to_gpu_numa_node(device_index: int):
    """Pin this process to the CPU cores of the NUMA node the GPU hangs off, so that the pinned host
    buffers it allocates next are placed (first touch) in that node's memory: with one rank per GPU
    all staging traffic otherwise crosses the socket interconnect of whichever node the ranks started
    on.  Returns a short description for the JSON line; does nothing where sysfs has no answer."""
    try:
        pr = torch.cuda.get_device_properties(device_index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return "no NUMA information"
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return f"node {node}: none of its cores is available to this process"
        os.sched_setaffinity(0, cpus)
        return f"bound to NUMA node {node} ({len(cpus)} cores)"
    except (OSError, ValueError, AttributeError) as e:
        return f"not bound ({type(e).__name__})"


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
    numa = bind_to_gpu_numa_node(local) if world > 1 else "single process: not bound"
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

    timeouts = native.load().spf_device_timeouts()
    if timeouts:
        raise SystemExit(f"{timeouts} bounded device-side waits gave up during the run: results are invalid")
    incumbent = sparse = None
    if world == 1 and not args.no_incumbents:
        del dev_in, stage_bufs, out_bufs, host_in, host_out
        torch.cuda.empty_cache()
        incumbent, sparse = measure_incumbents(wl, lookup_path, cfg, peaks)
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        c = cpu_sample(wl)
        cpu = {"value": c["ms_per_step"], "unit": "ms", "cores": torch.get_num_threads(), "kind": c["kind"],
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
                     "traffic": ncu_dram_bytes("sparse_attn_tc5_kernel", wl) if world == 1 else None,
                     "traffic_unit": "bytes per launch (ncu dram read+write)", "of": peaks["source"]},
        "roofline_pool": {"kernel": "Q/K block pooling", "bound": "hbm", "achieved": pool_gbs,
                          "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": pool_gbs / peaks["hbm_gbs"],
                          "traffic": ncu_dram_bytes("pool_blocks_kernel", wl) if world == 1 else None,
                          "traffic_unit": "bytes per launch (ncu dram read+write)", "of": peaks["source"]},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes,
                "host_buffers": numa},
        "gpu_launches": launches_timed,
        "device_timeouts": timeouts,
        "clocks": clocks,
    }
    if incumbent is not None:
        line["incumbent"] = incumbent
        line["sparse_regime"] = sparse
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
    ap.add_argument("--no-incumbents", action="store_true",
                    help="skip the one-layer reference / dense SDPA / sparse-regime measurements (N=1)")
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
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if wl.num_kv_heads % world:
            # heads shard by whole KV groups only: splitting a group would duplicate its K/V
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"unavailable": f"{wl.name} has {wl.num_kv_heads} KV heads: it shards over at most "
                                                 f"{wl.num_kv_heads} GPUs by whole KV groups, not over {world}",
                                  "n_gpus": world, "config": config_dict(wl, world)}))
            return
        run_gpu_arm(args, wl)


if __name__ == "__main__":
    main()
