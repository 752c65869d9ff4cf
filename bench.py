"""Benchmark of the tree-attention hot path (GPU precompute + fused sparse tree attention).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One STEP is one decode step of a tree-speculating model: the tree's block metadata is rebuilt
once from its parent array (one precompute launch) and then used by LAYERS attention calls, one
per transformer layer, each on its own Q/K/V.  The layer buffers are distinct and together far
larger than the L2 cache, so every call streams its K/V rows from HBM.

Printed JSON (one line, rank 0):
  value        gathered-KV GB/s over the whole step (inputs resident in HBM, step replayed as a
               CUDA graph), summed over ranks; ms_per_step and us_per_call give the latency view
  e2e          the same metric through the public Python API / C ABI with HOST buffers: every
               step copies parent, Q, K, V from pinned host memory and copies O back; copy-in,
               attention and copy-out of consecutive calls overlap on three streams (the figure
               is bound by the host-to-device link: three tensors in for one out)
  roofline     attention kernel: algorithmic gathered-KV bytes per launch / average launch
               duration (CUDA events around a graph of LAYERS back-to-back launches) against the
               measured HBM copy bandwidth
  cpu_baseline the oracle port of the reference's CPU path (metadata precompute + dense masked
               attention, torch on all host cores) on a bounded sample of the same workload

With N > 1 (launched by torch.distributed.run) every rank runs the same step on its own GPU and
its own seeded inputs; there is no collective in the timed region (weak scaling).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

# dram__bytes_read.sum + dram__bytes_write.sum per attention launch, from the ncu captures summarised
# in profiles/attn_tma_kernel_medusa256_forest64.md (same per-launch work as the bench)
NCU_TRAFFIC_BYTES = {"medusa256": 6.36e6, "forest64": 515.7e6, "random1024": 25.3e6, "deep4096": 242.4e6}
# the same for prefix_umma_kernel (profiles/prefix_umma_kernel_medusa256_prefix4096.md)
NCU_PREFIX_TRAFFIC_BYTES = {"medusa256_prefix4096": 70.9e6}

METRIC = "tree_attn_gathered_kv_bandwidth"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TENSOR_TFLOPS = 1590.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="medusa256")
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--kernel", default="auto")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--shard", action="store_true",
                    help="strong scaling: split the workload's trees or heads over the ranks and "
                         "all-gather the outputs (NCCL) once per step")
    return ap.parse_args()


def measured_tensor_peak():
    """Dense 16-bit tensor throughput (TFLOP/s) of a kernel timed alone: the measured burst figure."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_TENSOR_TFLOPS, "fallback"


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


# ---------------------------------------------------------------------------------------------
# workload description shared by both arms
# ---------------------------------------------------------------------------------------------
def describe(w, layers):
    """Algorithmic bytes of one attention call, from the metadata definition on the CPU."""
    from fstattention_b200 import configs  # noqa: F401
    es = 4 if w.dtype == "fp32" else 2
    rows = 0
    for par in w.trees:
        rows += gathered_rows_of(par, w.block_m)
        rows += w.prefix * -(-len(par) // w.block_m)       # every block reads the whole prefix
    kv_bytes = rows * w.heads * w.head_dim * es * 2
    qo_bytes = 2 * len(w.trees) * w.heads * w.n_nodes * w.head_dim * es
    return {"gathered_kv_bytes_per_call": kv_bytes, "q_o_bytes_per_call": qo_bytes,
            "gathered_rows_per_head": rows}


def gathered_rows_of(parent, bm):
    """sum over blocks of |unique strict ancestors| + |block rows not among them| (real rows)."""
    n = len(parent)
    total = 0
    for lo in range(0, n, bm):
        anc = set()
        for k in range(lo, min(lo + bm, n)):
            x = parent[k]
            while x >= 0 and x not in anc:
                anc.add(x)
                x = parent[x]
        leaves = sum(1 for k in range(lo, min(lo + bm, n)) if k not in anc)
        total += len(anc) + leaves
    return total


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.002)                        # the timed region is a few milliseconds

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle port of the reference's CPU path
# ---------------------------------------------------------------------------------------------
def cpu_reference_step(w, sample_layers, tensors):
    """Metadata precompute + dense masked attention for `sample_layers` layers, on the CPU."""
    from oracle import tree_oracle as orc
    for par in w.trees:
        lin, lvl = orc.lineage_from_parent(par)
        mask = orc.block_padded_mask(lin, w.block_m)[: w.n_nodes, : w.n_nodes]
        orc.block_metadata(lin, lvl, w.block_m, w.max_ancestors)
        for (q, k, v) in tensors[:sample_layers]:
            orc.dense_tree_attention(q, k, v, mask, w.sm_scale, head_chunk=8)


def time_cpu_reference(w, info, steps, warmup, sample_layers=2, budget_s=25.0):
    torch.set_num_threads(os.cpu_count() or 1)
    dtype = {"fp16": torch.float16, "fp32": torch.float32, "bf16": torch.bfloat16}[w.dtype]
    g = torch.Generator().manual_seed(0)
    trees = w.trees[:1] if len(w.trees) > 1 else w.trees          # bounded sample: one tree
    ws = type(w)(**{**w.__dict__, "trees": trees})
    tensors = [tuple(torch.randn((1, w.heads, w.n_nodes, w.head_dim), generator=g).to(dtype)
                     for _ in range(3)) for _ in range(sample_layers)]
    times = []
    t_begin = time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        cpu_reference_step(ws, sample_layers, tensors)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if time.perf_counter() - t_begin > budget_s and len(times) >= 3:
            break
    per_call_bytes = info["gathered_kv_bytes_per_call"] / len(w.trees)
    med = statistics.median(times)
    gbs = per_call_bytes * sample_layers / med / 1e9
    return {"value": gbs, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": (f"{len(times)} steps of: 1 tree metadata precompute + {sample_layers} dense "
                       f"masked attention calls ({w.dtype}, as the reference writes it)"),
            "ms_per_sample_step": med * 1e3, "host_cpus": os.cpu_count()}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def run_ours(args, rank, world):
    import fstattention_b200 as fst
    from fstattention_b200 import configs
    import torch.distributed as dist

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    w = configs.workload(args.workload)
    info = describe(w, args.layers)
    dtype = {"fp16": torch.float16, "fp32": torch.float32, "bf16": torch.bfloat16}[w.dtype]
    T, H, N, D, L = len(w.trees), w.heads, w.n_nodes, w.head_dim, args.layers

    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    layers = [tuple(torch.randn((T, H, N + (w.prefix if i else 0), D), generator=g, device=dev,
                                dtype=torch.float32).to(dtype) for i in range(3)) for _ in range(L)]
    outs = [torch.empty((T, H, N, D), device=dev, dtype=dtype) for _ in range(L)]
    parent = torch.tensor(w.trees if T > 1 else w.trees[0], dtype=torch.int32, device=dev)
    meta = fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, reference_format=False)
    resident_mb = sum(t.numel() * t.element_size() for trip in layers for t in trip) / 1e6
    # The dynamic-tree configuration grows a new tree every step: 100 seeded trees wait on the
    # device and each timed step starts by copying the next one over `parent` (the decoder's own
    # tree construction stands in as a 4 KB device copy), so precompute and attention meet a
    # different tree every time.
    dynamic = w.name == "random1024"
    if dynamic:
        seeds = list(range(100))
        parents = torch.tensor([configs.workload(w.name, s_).trees[0] for s_ in seeds], dtype=torch.int32, device=dev)
        kv_by_seed = [describe(configs.workload(w.name, s_), args.layers)["gathered_kv_bytes_per_call"] for s_ in seeds]

        def next_tree(i):
            parent.copy_(parents[i % len(seeds)], non_blocking=True)
    else:
        next_tree = None

    def step():
        fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, out=meta, check=False)
        for (q, k, v), o in zip(layers, outs):
            fst.fst_attention(q, k, v, meta, sm_scale=w.sm_scale, out=o, kernel=args.kernel)

    def attention_only():
        for (q, k, v), o in zip(layers, outs):
            fst.fst_attention(q, k, v, meta, sm_scale=w.sm_scale, out=o, kernel=args.kernel)

    def precompute_only():
        for _ in range(16):
            fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, out=meta, check=False)

    def capture(fn):
        fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(graph):
            fn()
        return graph

    g_step, g_attn, g_pre = capture(step), capture(attention_only), capture(precompute_only)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(graph, reps, before=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(reps):
            if before is not None:
                before(i)
            graph.replay()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    for _ in range(max(args.warmup, 3)):
        g_step.replay()
    sampler = ClockSampler(local)
    sampler.start()
    total_ms = timed(g_step, args.steps, next_tree)
    clocks = sampler.stop()
    ms_per_step = total_ms / args.steps
    assert meta.check() is meta and fst.last_status(dev) == 0
    if dynamic:                                           # the per-kernel figures below are for tree 0
        next_tree(0)
        g_step.replay()
    for _ in range(3):
        g_attn.replay()
    attn_ms = timed(g_attn, args.steps) / args.steps
    for _ in range(3):
        g_pre.replay()
    pre_us = timed(g_pre, args.steps) / args.steps / 16 * 1e3
    assert meta.check() is meta and fst.last_status(dev) == 0

    kv = info["gathered_kv_bytes_per_call"]
    kv_step = kv if not dynamic else sum(kv_by_seed[i % len(seeds)] for i in range(args.steps)) / args.steps
    value = world * kv_step * L / (ms_per_step * 1e-3) / 1e9
    launch_us = attn_ms * 1e3 / L
    peak, peak_kind = measured_hbm_peak()
    achieved = kv / (launch_us * 1e-6) / 1e9

    # ---- cold single-call latency: L2 flushed by a 512 MB memset between calls
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    lat = []
    q, k, v = layers[0]
    for i in range(30):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fst.fst_attention(q, k, v, meta, sm_scale=w.sm_scale, out=outs[0], kernel=args.kernel)
        e1.record()
        torch.cuda.synchronize()
        if i >= 5:
            lat.append(e0.elapsed_time(e1) * 1e3)
    del flush

    # ---- end to end: host buffers in, host buffers out, through the public API
    e2e = None
    if not args.no_e2e:
        e2e_layers = min(L, 16)
        # without a prefix q, k and v have one shape: the host keeps them as views of one pinned
        # buffer per call (a fused qkv), which then crosses PCIe in a single copy
        fused = w.prefix == 0
        if fused:
            host_in = [torch.stack([t.cpu() for t in trip]).pin_memory() for trip in layers[:e2e_layers]]
        else:
            host_in = [tuple(t.cpu().pin_memory() for t in trip) for trip in layers[:e2e_layers]]
        host_out = [torch.empty((T, H, N, D), dtype=dtype).pin_memory() for _ in range(e2e_layers)]
        host_parent = parent.cpu().pin_memory()
        # Three streams, two device slots: the copy-in of call i+1, the attention of call i and the
        # copy-out of call i-1 overlap (PCIe is full duplex and the copy engines are separate), as
        # a host that feeds the library from its own buffers would arrange it.
        if fused:
            slots = [torch.empty((3,) + tuple(layers[0][0].shape), dtype=dtype, device=dev) for _ in range(2)]
        else:
            slots = [tuple(torch.empty_like(t) for t in layers[0]) for _ in range(2)]    # k, v carry the prefix rows
        slot_out = [torch.empty_like(outs[0]) for _ in range(2)]
        dpar = torch.empty_like(parent)
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        s_cmp = torch.cuda.current_stream(dev)
        ev_in = [torch.cuda.Event() for _ in range(2)]      # inputs of the slot have arrived
        ev_cmp = [torch.cuda.Event() for _ in range(2)]     # attention on the slot is done
        ev_out = [torch.cuda.Event() for _ in range(2)]     # the slot's output has left

        def e2e_step():
            dpar.copy_(host_parent, non_blocking=True)
            fst.build_tree_metadata(dpar, w.block_m, w.max_ancestors, out=meta, check=False)
            for i, (hin, ho) in enumerate(zip(host_in, host_out)):
                sl = i & 1
                dq, dk, dv = slots[sl]                      # (rows of the fused slot, or the three tensors)
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_cmp[sl])         # the slot's previous inputs have been used
                    if fused:
                        slots[sl].copy_(hin, non_blocking=True)
                    else:
                        dq.copy_(hin[0], non_blocking=True)
                        dk.copy_(hin[1], non_blocking=True)
                        dv.copy_(hin[2], non_blocking=True)
                    ev_in[sl].record(s_in)
                s_cmp.wait_event(ev_in[sl])
                if i >= 2:
                    s_cmp.wait_event(ev_out[sl])            # the slot's previous output has left
                fst.fst_attention(dq, dk, dv, meta, sm_scale=w.sm_scale, out=slot_out[sl], kernel=args.kernel)
                ev_cmp[sl].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[sl])
                    ho.copy_(slot_out[sl], non_blocking=True)
                    ev_out[sl].record(s_out)
            torch.cuda.synchronize()

        for _ in range(3):
            e2e_step()
        e2e_steps = max(3, min(args.steps, 10))
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        dt = (time.perf_counter() - t0) / e2e_steps
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = t.item()
        tensor_bytes = T * H * N * D * (4 if w.dtype == "fp32" else 2)
        in_bytes = sum(t.numel() * t.element_size() for t in layers[0])
        e2e = {"value": world * kv * e2e_layers / dt / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": e2e_layers * in_bytes + parent.numel() * 4,
               "d2h_bytes_per_step": e2e_layers * tensor_bytes,
               "ms_per_step": dt * 1e3, "calls_per_step": e2e_layers,
               "us_per_call": dt * 1e6 / e2e_layers,
               "overlap": "copy-in, attention and copy-out of consecutive calls on three streams, two device slots",
               "inputs": "q, k, v are views of one pinned buffer per call, one copy" if fused else "q, k, v pinned separately, three copies per call"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = time_cpu_reference(w, info, steps=10, warmup=2)

    if rank != 0:
        return
    # A long dense prefix makes the call compute-bound: the prefix goes to the tcgen05 kernel and
    # the bound is the tensor cores.  Algorithmic flops: every query block forms block_m x rows
    # scores and as many products with V, 2 * head_dim flops each.
    plan = fst.launch_plan(layers[0][0], w.prefix, w.block_m, args.kernel)
    roofline_tensor = None
    if "prefix_umma_kernel" in plan["kernels"]:
        tpeak, tkind = measured_tensor_peak()
        esize = 4 if w.dtype == "fp32" else 2
        flops = 4.0 * D * w.block_m * (kv / (2 * D * esize))
        tf = flops / (launch_us * 1e-6) / 1e12
        roofline_tensor = {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak,
                           "traffic": NCU_PREFIX_TRAFFIC_BYTES.get(w.name), "peak_source": f"of {tkind}", "kernel": "prefix_umma_kernel",
                           "flops_per_call": flops, "prefix_runs": plan["prefix_runs"],
                           "note": "time is the whole call: prefix kernel, tree kernel beside it, merge kernel"}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": {"workload": w.name, "trees": T, "nodes": N, "heads": H, "head_dim": D,
                   "block_m": w.block_m, "max_ancestors": w.max_ancestors, "prefix": w.prefix,
                   "calls_per_step": L, "step": "1 precompute launch + calls_per_step attention launches (CUDA graph)",
                   "l2": f"{L} distinct layer buffers, {resident_mb:.0f} MB resident > 126 MB L2",
                   "kernel": args.kernel, "per_rank": "same step on every rank, own inputs",
                   **({"dynamic_trees": "100 seeded trees on the device, a new one every step; roofline and "
                                "per-kernel figures are for seed 0"} if dynamic else {})},
        "us_per_call": ms_per_step * 1e3 / L,
        "attention_us_per_call_back_to_back": launch_us,
        "attention_us_per_call_cold_l2": statistics.median(lat),
        "precompute_us": pre_us,
        "gathered_kv_bytes_per_call": kv,
        "q_o_bytes_per_call": info["q_o_bytes_per_call"],
        "gpu_launches": args.steps * (L * len(plan["kernels"]) + 1),
        "kernels_per_call": plan["kernels"],
        "clocks": clocks,
        "roofline": roofline_tensor if roofline_tensor is not None else {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES.get(w.name), "peak_source": f"of {peak_kind}",
                     "kernel": "attn_tma_kernel" if args.kernel in ("auto", "tma") else f"attn_{args.kernel}_kernel", "achieved_incl_q_o": (kv + info["q_o_bytes_per_call"]) / (launch_us * 1e-6) / 1e9,
                     "frac_of_nominal_8000": achieved / 8000.0},
    }
    if e2e is not None:
        line["e2e"] = e2e
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))


def run_sharded(args, rank, world):
    """One problem split over the ranks (by tree or by head) + one all-gather of outputs per step."""
    import fstattention_b200 as fst
    from fstattention_b200 import configs, sharding
    import torch.distributed as dist

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    w = configs.workload(args.workload)
    if w.shard not in ("tree", "head"):
        raise SystemExit(f"workload {w.name} has no shard axis")
    info = describe(w, args.layers)
    dtype = {"fp16": torch.float16, "fp32": torch.float32, "bf16": torch.bfloat16}[w.dtype]
    T, H, N, D, L = len(w.trees), w.heads, w.n_nodes, w.head_dim, args.layers
    n_units = T if w.shard == "tree" else H
    lo, hi = sharding.shard_bounds(n_units, world, rank)
    Tl, Hl = (hi - lo, H) if w.shard == "tree" else (T, hi - lo)
    trees = w.trees[lo:hi] if w.shard == "tree" else w.trees

    g = torch.Generator(device=dev).manual_seed(99 + rank)
    layers = [tuple(torch.randn((Tl, Hl, N, D), generator=g, device=dev, dtype=torch.float32).to(dtype)
                    for _ in range(3)) for _ in range(L)]
    # outputs of all layers of the step in one buffer so that one collective moves them
    if w.shard == "tree":
        out_local = torch.empty((L, Tl, Hl, N, D), device=dev, dtype=dtype)
        out_full = torch.empty((world, L, Tl, Hl, N, D), device=dev, dtype=dtype)
    else:
        out_local = torch.empty((L, Tl, Hl, N, D), device=dev, dtype=dtype)
        out_full = torch.empty((world, L, Tl, Hl, N, D), device=dev, dtype=dtype)
    if n_units % world:
        raise SystemExit("the sharded bench wants the unit count to divide evenly")
    parent = torch.tensor(trees if len(trees) > 1 else trees[0], dtype=torch.int32, device=dev)
    meta = fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, reference_format=False)

    def compute():
        fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, out=meta, check=False)
        for i, (q, k, v) in enumerate(layers):
            fst.fst_attention(q, k, v, meta, sm_scale=w.sm_scale, out=out_local[i], kernel=args.kernel)

    compute()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        compute()

    def step():
        graph.replay()
        if world > 1:
            dist.all_gather_into_tensor(out_full.view(-1), out_local.view(-1))

    def timed(fn, reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms / reps

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local)
    sampler.start()
    ms_step = timed(step, args.steps)
    clocks = sampler.stop()
    ms_compute = timed(graph.replay, args.steps)
    assert fst.last_status(dev) == 0
    if rank != 0:
        return
    kv = info["gathered_kv_bytes_per_call"]
    peak, peak_kind = measured_hbm_peak()
    line = {
        "metric": METRIC, "value": kv * L / (ms_step * 1e-3) / 1e9, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": w.dtype,
        "data": "synthetic",
        "config": {"workload": w.name, "trees": T, "nodes": N, "heads": H, "head_dim": D,
                   "block_m": w.block_m, "max_ancestors": w.max_ancestors, "calls_per_step": L,
                   "shard": w.shard, "units_per_rank": hi - lo,
                   "step": "1 precompute + calls_per_step attention launches on the local shard (CUDA graph), "
                           "then one NCCL all-gather of the step's outputs",
                   "l2": f"{L} layer buffers per rank", "kernel": args.kernel},
        "us_per_call": ms_step * 1e3 / L, "compute_only_us_per_call": ms_compute * 1e3 / L,
        "all_gather_bytes_per_step": out_full.numel() * out_full.element_size(),
        "gathered_kv_bytes_per_call": kv, "gpu_launches": args.steps * (L + 1), "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": kv / world / (ms_compute * 1e-3 / L) / 1e9, "peak": peak,
                     "unit": "GB/s", "frac": kv / world / (ms_compute * 1e-3 / L) / 1e9 / peak, "traffic": None,
                     "peak_source": f"of {peak_kind}", "kernel": "attn_tma_kernel", "per": "GPU, compute only"},
    }
    print(json.dumps(line))


def run_reference(args, rank, world):
    """The reference's CPU path (oracle port) timed on the host cores, same metric and config."""
    if rank != 0:
        return
    from fstattention_b200 import configs
    w = configs.workload(args.workload)
    info = describe(w, args.layers)
    sample_layers = 2
    cpu = time_cpu_reference(w, info, steps=args.steps, warmup=max(args.warmup, 1),
                             sample_layers=sample_layers, budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cpu["ms_per_sample_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
        "data": "synthetic",
        "config": {"workload": w.name, "trees": len(w.trees), "nodes": w.n_nodes, "heads": w.heads,
                   "head_dim": w.head_dim, "block_m": w.block_m, "max_ancestors": w.max_ancestors,
                   "calls_per_step": sample_layers},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group("nccl")
    try:
        if args.shard:
            run_sharded(args, rank, world)
        else:
            run_ours(args, rank, world)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
