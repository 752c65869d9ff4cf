"""Benchmark of the tree-attention hot path (GPU precompute + fused sparse tree attention).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference-triton]
                  [--workload NAME]

One STEP is one decode step of a tree-speculating model: the tree's block metadata is rebuilt
once from its parent array (one precompute launch) and then used by LAYERS attention calls, one
per transformer layer, each on its own Q/K/V.  The layer buffers are distinct and together far
larger than the L2 cache, so every call streams its K/V rows from HBM.

Printed JSON (one line, rank 0):
  value        gathered-KV GB/s over the whole step (inputs resident in HBM, step replayed as a
               CUDA graph), summed over ranks; ms_per_step and us_per_call give the latency view
  e2e          the same metric through the public Python API / C ABI with HOST buffers: every
               step copies parent, Q, K, V from pinned host memory and copies O back; copy-in,
               attention and copy-out of consecutive calls overlap on three streams
  roofline     attention kernel of the headline workload: algorithmic gathered-KV bytes per
               launch / average launch duration (CUDA events around a graph of LAYERS
               back-to-back launches) against the measured HBM copy bandwidth
  workloads    the other single-GPU configurations (dynamic 1024-node tree, 64 batched trees,
               deep 4096-node tree with 64- and 128-row blocks), each event-timed over a graph
               of a few layers on rotating buffers larger than L2: us per call, gathered-KV
               fraction and DRAM-byte fraction of the measured HBM bandwidth
  sharded      the two configurations that split over GPUs (trees of the batched forest, heads
               of the deep tree): per-GPU compute, the step with the NCCL all-gather of outputs
               (after every layer, and overlapped with the next layer's attention), and the
               gathered output checked against a single-GPU recomputation and the CPU oracle
  cpu_baseline the reference's CPU path (its own utils.py for the metadata when a copy of the
               reference sits under baseline/_ref, else the oracle port; the oracle's
               restatement of its dense masked attention) on a bounded sample, composed to the
               same step as the GPU arm

With N > 1 (launched by torch.distributed.run) the top-level figures are replicas: every rank
runs the headline step on its own GPU and inputs, no collective in the timed region.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.util
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

METRIC = "tree_attn_gathered_kv_bandwidth"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_TENSOR_TFLOPS = 1590.0
REF_DIR = os.path.join(ROOT, "baseline", "_ref")          # a copy of the reference (not in history)
TRAFFIC_JSON = os.path.join(ROOT, "profiles", "dram_traffic.json")
DTYPES = {"fp16": torch.float16, "fp32": torch.float32, "bf16": torch.bfloat16}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-triton"])
    ap.add_argument("--workload", default="medusa256")
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--kernel", default="auto")
    ap.add_argument("--block-m", type=int, default=None, help="override the workload's query block size")
    ap.add_argument("--max-ancestors", type=int, default=None, help="override the workload's ancestor bound")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="skip the workloads / sharded sub-objects")
    ap.add_argument("--no-reference-gpu", action="store_true",
                    help="skip timing the reference's own Triton kernel beside the headline figure")
    ap.add_argument("--shard", action="store_true",
                    help="only the sharded measurement of --workload (forest64 or deep4096), as the top-level line")
    return ap.parse_args()


def measured_peak(key, fallback):
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)[key]), "measured"
    except Exception:
        return fallback, "fallback"


def measured_hbm_peak():
    return measured_peak("hbm_gbs", FALLBACK_HBM_GBS)


def measured_tensor_peak():
    """Dense 16-bit tensor throughput (TFLOP/s) of a kernel timed alone: the measured burst figure."""
    return measured_peak("bf16_tflops", FALLBACK_TENSOR_TFLOPS)


# ---------------------------------------------------------------------------------------------
# workload description shared by all arms
# ---------------------------------------------------------------------------------------------
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


def describe(w):
    """Algorithmic bytes of one attention call, from the metadata definition on the CPU."""
    es = 4 if w.dtype == "fp32" else 2
    rows = 0
    for par in w.trees:
        rows += gathered_rows_of(par, w.block_m)
        rows += w.prefix * -(-len(par) // w.block_m)       # every block reads the whole prefix
    kv_bytes = rows * w.heads * w.head_dim * es * 2
    qo_bytes = 2 * len(w.trees) * w.heads * w.n_nodes * w.head_dim * es
    return {"gathered_kv_bytes_per_call": kv_bytes, "q_o_bytes_per_call": qo_bytes,
            "gathered_rows_per_head": rows}


def workload_config(w, calls_per_step):
    """What is computed, the same dictionary in every arm (how an arm runs it is said elsewhere)."""
    return {"workload": w.name, "trees": len(w.trees), "nodes": w.n_nodes, "heads": w.heads,
            "head_dim": w.head_dim, "block_m": w.block_m, "max_ancestors": w.max_ancestors,
            "prefix": w.prefix, "calls_per_step": calls_per_step,
            "step": "1 tree-metadata precompute + calls_per_step attention calls on distinct Q/K/V"}


def kernel_source_digest():
    """Hash of the attention kernels' sources: a DRAM-traffic capture is quoted only for the
    sources it was taken from."""
    h = hashlib.sha1()
    csrc = os.path.join(ROOT, "fstattention_b200", "csrc")
    for name in ("fst_attention_tma.cuh", "fst_attention_persist.cuh", "fst_attention_mma.cuh", "fst_prefix_umma.cu"):
        try:
            with open(os.path.join(csrc, name), "rb") as f:
                h.update(f.read())
        except OSError:
            h.update(name.encode())
    return h.hexdigest()[:16]


def ncu_traffic(case):
    """(bytes per launch, where the figure comes from) for a workload, or (None, why not)."""
    try:
        with open(TRAFFIC_JSON) as f:
            rec = json.load(f)
    except Exception:
        return None, "no capture on file"
    ent = rec.get("captures", {}).get(case)
    if ent is None:
        return None, "no capture on file"
    if rec.get("kernel_sources_sha1") != kernel_source_digest():
        return None, "capture on file is older than the kernel sources: not quoted"
    return float(ent["dram_bytes_per_launch"]), f"ncu capture ({ent['kernel']}), not measured in this run"


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
# CPU arm: the reference's CPU path
# ---------------------------------------------------------------------------------------------
def load_reference_utils():
    """The reference's own utils.py from the copy under baseline/_ref, or None."""
    path = os.path.join(REF_DIR, "utils.py")
    if not os.path.exists(path):
        return None
    try:
        spec = importlib.util.spec_from_file_location("fst_reference_utils", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    except Exception:
        return None


def time_cpu_reference(w, info, calls_per_step, steps, warmup, sample_calls=2, budget_s=25.0):
    """The reference's CPU path on a bounded sample: per sample step one metadata precompute
    (the reference's utils.py when present, else the oracle port of it; timed on one tree) and
    `sample_calls` dense masked attention calls (the oracle's restatement of
    fstattention.py:214-219, in the workload's dtype; one tree).  The two legs are timed apart
    and composed to the GPU arm's step: 1 precompute + calls_per_step attention calls."""
    from oracle import tree_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    dtype = DTYPES[w.dtype]
    g = torch.Generator().manual_seed(0)
    par = w.trees[0]
    lin, lvl = orc.lineage_from_parent(par)
    mask = orc.block_padded_mask(lin, w.block_m)[: w.n_nodes, : w.n_nodes]
    ref_utils = load_reference_utils()
    tensors = [tuple(torch.randn((1, w.heads, w.n_nodes, w.head_dim), generator=g).to(dtype)
                     for _ in range(3)) for _ in range(sample_calls)]

    def precompute():
        if ref_utils is not None:
            ref_utils.create_full_attention_mask(lin.clone())
            ref_utils.create_fst_attention_kernel_inputs(lin.clone(), lvl, block_m=w.block_m,
                                                         max_ancestors=w.max_ancestors)
        else:
            orc.block_padded_mask(lin, w.block_m)
            orc.block_metadata(lin, lvl, w.block_m, w.max_ancestors)

    t_pre, t_att = [], []
    t_begin = time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        precompute()
        t1 = time.perf_counter()
        for (q, k, v) in tensors:
            orc.dense_tree_attention(q, k, v, mask, w.sm_scale, head_chunk=8)
        t2 = time.perf_counter()
        if i >= warmup:
            t_pre.append(t1 - t0)
            t_att.append((t2 - t1) / sample_calls)
        if time.perf_counter() - t_begin > budget_s and len(t_pre) >= 3:
            break
    pre, att = statistics.median(t_pre), statistics.median(t_att)
    n_trees = len(w.trees)
    step_s = n_trees * (pre + calls_per_step * att)       # the reference handles one tree per call
    gbs = info["gathered_kv_bytes_per_call"] * calls_per_step / step_s / 1e9
    return {"value": gbs, "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": "port",
            "legs": {"precompute": {"kind": "reference" if ref_utils is not None else "port",
                                    "what": "create_full_attention_mask + create_fst_attention_kernel_inputs"
                                            + (" (the reference's utils.py)" if ref_utils is not None else " (oracle port)"),
                                    "ms_per_tree": pre * 1e3},
                     "attention": {"kind": "port",
                                   "what": f"dense masked attention as fstattention.py:214-219 writes it ({w.dtype}), "
                                           "restated (it is inline in a test that needs a GPU)",
                                   "ms_per_call_per_tree": att * 1e3}},
            "sample": (f"{len(t_pre)} sample steps of one tree: 1 precompute + {sample_calls} attention calls, timed apart; "
                       f"composed to trees x (1 precompute + {calls_per_step} calls)"),
            "ms_per_step_composed": step_s * 1e3, "host_cpus": os.cpu_count()}


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
class Timer:
    """CUDA-event timing on torch's current stream, bracketed by a barrier and a device
    synchronisation on both sides, maximum over ranks."""

    def __init__(self, dev, world):
        self.dev, self.world = dev, world

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def __call__(self, fn, reps, before=None):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record()
        for i in range(reps):
            if before is not None:
                before(i)
            fn()
        e1.record()
        self.barrier()
        ms = e0.elapsed_time(e1)
        if self.world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms


def capture(fn):
    fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


def with_block(w, block_m, max_ancestors):
    return type(w)(**{**w.__dict__, "block_m": block_m, "max_ancestors": max_ancestors})


def measure_case(fst, w, layers_n, reps, dev, kernel="auto", case=None):
    """One workload, whole problem on this GPU: a graph of `layers_n` attention calls on rotating
    buffers, event-timed; plus the precompute alone."""
    info = describe(w)
    dtype = DTYPES[w.dtype]
    T, H, N, D = len(w.trees), w.heads, w.n_nodes, w.head_dim
    g = torch.Generator(device=dev).manual_seed(77)
    layers = [tuple(torch.randn((T, H, N, D), generator=g, device=dev, dtype=torch.float32).to(dtype)
                    for _ in range(3)) for _ in range(layers_n)]
    outs = [torch.empty((T, H, N, D), device=dev, dtype=dtype) for _ in range(layers_n)]
    parent = torch.tensor(w.trees if T > 1 else w.trees[0], dtype=torch.int32, device=dev)
    meta = fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, reference_format=False)

    def attention():
        for (q, k, v), o in zip(layers, outs):
            fst.fst_attention(q, k, v, meta, sm_scale=w.sm_scale, out=o, kernel=kernel)

    def precompute():
        for _ in range(8):
            fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, out=meta, check=False)

    timer = Timer(dev, 1)
    g_att, g_pre = capture(attention), capture(precompute)
    for _ in range(3):
        g_att.replay()
    us = timer(g_att.replay, reps) / reps / layers_n * 1e3
    for _ in range(3):
        g_pre.replay()
    pre_us = timer(g_pre.replay, reps) / reps / 8 * 1e3
    assert meta.check() is meta and fst.last_status(dev) == 0
    peak, peak_kind = measured_hbm_peak()
    kv = info["gathered_kv_bytes_per_call"]
    traffic, source = ncu_traffic(case or w.name)
    plan = fst.launch_plan(layers[0][0], w.prefix, w.block_m, kernel)
    resident = sum(t.numel() * t.element_size() for trip in layers for t in trip) / 1e6
    out = {"config": workload_config(w, layers_n), "us_per_call": us, "precompute_us": pre_us,
           "gathered_kv_bytes_per_call": kv, "q_o_bytes_per_call": info["q_o_bytes_per_call"],
           "gathered_kv_gbs": kv / us / 1e3, "frac_gathered_kv": kv / us / 1e3 / peak,
           "dram_bytes_per_call": traffic, "dram_gbs": None if traffic is None else traffic / us / 1e3,
           "frac_dram": None if traffic is None else traffic / us / 1e3 / peak,
           "traffic_source": source, "peak_gbs": peak, "peak_source": f"of {peak_kind}",
           "kernels_per_call": plan["kernels"],
           "l2": f"{layers_n} distinct layer buffers, {resident:.0f} MB of inputs resident > 126 MB L2"}
    del layers, outs, g_att, g_pre
    torch.cuda.empty_cache()
    return out


def measure_tree_build(fst, dev, reps):
    """A decode step that grows its tree on the GPU: top-k scores -> parent array -> block
    metadata, nothing crossing to the host (1020 nodes: the reference's create_tree(7) shape)."""
    depth, topk, lwf = 7, 4, 0.5
    g = torch.Generator(device=dev).manual_seed(3)
    scores = torch.log_softmax(torch.randn((depth + 1, topk), generator=g, device=dev), dim=-1)
    n = fst.tree_topk_nodes(depth, topk, lwf)
    parent = fst.build_tree_topk(scores, left_weight_factor=lwf)
    meta = fst.build_tree_metadata(parent, 64, 128, reference_format=False)

    def build_only():
        for _ in range(8):
            fst.build_tree_topk(scores, left_weight_factor=lwf)

    def build_and_precompute():
        for _ in range(8):
            par = fst.build_tree_topk(scores, left_weight_factor=lwf)
            fst.build_tree_metadata(par, 64, 128, out=meta, check=False)

    timer = Timer(dev, 1)
    out = {"nodes": n, "depth": depth, "topk": topk, "left_weight_factor": lwf, "block_m": 64}
    for key, fn in (("build_us", build_only), ("build_plus_precompute_us", build_and_precompute)):
        graph = capture(fn)
        for _ in range(3):
            graph.replay()
        out[key] = timer(graph.replay, reps) / reps / 8 * 1e3
    assert meta.check() is meta
    return out


def seeded_full(shape, seed, dev, dtype):
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(dtype)


def measure_sharded(fst, name, rank, world, dev, layers_n, reps, kernel="auto"):
    """forest64 split by trees / deep4096 split by heads over the ranks, through
    sharding.sharded_fst_attention, with the all-gather of outputs; rank 0 returns the record."""
    import torch.distributed as dist
    from fstattention_b200 import configs, sharding
    w = configs.workload(name)
    axis = w.shard
    info = describe(w)
    dtype = DTYPES[w.dtype]
    T, H, N, D = len(w.trees), w.heads, w.n_nodes, w.head_dim
    n_units = T if axis == "tree" else H
    lo, hi = sharding.shard_bounds(n_units, world, rank)
    dim = sharding.AXES[axis]
    # every rank draws the whole tensor from the same seed and keeps its slice, so that any
    # rank can rebuild any other rank's inputs for the check below
    layers = []
    for i in range(layers_n):
        trip = []
        for j in range(3):
            full = seeded_full((T, H, N, D), 1000 + 3 * i + j, dev, dtype)
            trip.append(full.narrow(dim, lo, hi - lo).contiguous())
            del full
        layers.append(tuple(trip))
    trees = w.trees[lo:hi] if axis == "tree" else w.trees
    parent = torch.tensor(trees if len(trees) > 1 else trees[0], dtype=torch.int32, device=dev)
    meta = fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, reference_format=False)
    full_shape = (T, H, N, D)
    fulls = [torch.empty(full_shape, device=dev, dtype=dtype) for _ in range(layers_n)] if world > 1 else None
    locals_ = [torch.empty_like(layers[0][0]) for _ in range(layers_n)]

    def compute_only():
        fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, out=meta, check=False)
        for (q, k, v), o in zip(layers, locals_):
            sharding.sharded_fst_attention(q, k, v, meta, w.sm_scale, axis, n_units, gather=False, out=o, kernel=kernel)

    def step_serial():
        fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, out=meta, check=False)
        for i, ((q, k, v), o) in enumerate(zip(layers, locals_)):
            sharding.sharded_fst_attention(q, k, v, meta, w.sm_scale, axis, n_units, out=o, kernel=kernel,
                                           gathered=fulls[i])

    def step_overlapped():
        fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, out=meta, check=False)
        works = []
        for i, ((q, k, v), o) in enumerate(zip(layers, locals_)):
            _, work = sharding.sharded_fst_attention(q, k, v, meta, w.sm_scale, axis, n_units, out=o, kernel=kernel,
                                                     gathered=fulls[i], async_gather=True)
            works.append(work)
        for work in works:
            work.wait()

    shared = None
    if world > 1:
        try:                                              # one shared full tensor per layer, every rank's copy mapped everywhere
            shared = [sharding.GatheredOutput(full_shape, dtype, dev) for _ in range(layers_n)]
        except Exception as exc:                          # noqa: BLE001
            shared = f"{type(exc).__name__}: {exc}"[:300]

    def step_fused():
        fst.build_tree_metadata(parent, w.block_m, w.max_ancestors, out=meta, check=False)
        for (q, k, v), g in zip(layers, shared):
            sharding.sharded_fst_attention(q, k, v, meta, w.sm_scale, axis, n_units, scatter_to=g, kernel=kernel)

    timer = Timer(dev, world)
    g_compute = capture(compute_only)
    for _ in range(3):
        g_compute.replay()
    ms_compute = timer(g_compute.replay, reps) / reps
    rec = {"config": {**workload_config(w, layers_n), "shard": axis, "units_per_rank": hi - lo},
           "n_gpus": world, "compute_us_per_call": ms_compute * 1e3 / layers_n,
           "step_ms_no_gather": ms_compute,
           "gathered_kv_bytes_per_call": info["gathered_kv_bytes_per_call"]}
    peak, peak_kind = measured_hbm_peak()
    per_gpu = info["gathered_kv_bytes_per_call"] / world / (ms_compute * 1e-3 / layers_n) / 1e9
    rec["per_gpu_roofline"] = {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s",
                               "frac": per_gpu / peak, "peak_source": f"of {peak_kind}"}
    if world > 1:
        for _ in range(3):
            step_serial()
        ms_serial = timer(step_serial, reps) / reps
        for _ in range(3):
            step_overlapped()
        ms_overlap = timer(step_overlapped, reps) / reps
        # the collective alone, same buffers
        def gathers():
            for i in range(layers_n):
                sharding.all_gather_outputs(locals_[i], axis, n_units, out=fulls[i])
        for _ in range(3):
            gathers()
        ms_gather = timer(gathers, reps) / reps
        out_bytes = fulls[0].numel() * fulls[0].element_size()
        if isinstance(shared, list):
            for _ in range(3):
                step_fused()
            ms_fused = timer(step_fused, reps) / reps
            sent = out_bytes / world * (world - 1)        # what one GPU sends per layer
            rec["fused"] = {"what": "attention and all-gather in one kernel: each CTA stores its tile into every rank's "
                                    "copy of the output (TMA stores over NVLink), then a device-side barrier per layer",
                            "step_ms": ms_fused, "us_per_layer": ms_fused * 1e3 / layers_n,
                            "nvlink_out_bytes_per_gpu_per_layer": sent,
                            "nvlink_out_gbs_per_gpu": sent / (ms_fused / layers_n * 1e-3) / 1e9,
                            "value_gbs": info["gathered_kv_bytes_per_call"] * layers_n / (ms_fused * 1e-3) / 1e9}
        else:
            rec["fused"] = {"unavailable": shared}
        rec.update({"step_ms": ms_serial, "step_ms_overlapped": ms_overlap,
                    "all_gather_ms_per_layer": ms_gather / layers_n,
                    "all_gather_bytes_per_layer": out_bytes,
                    "all_gather_bus_gbs": out_bytes * (world - 1) / world / (ms_gather / layers_n * 1e-3) / 1e9,
                    "limiter": "the all-gather of outputs" if ms_gather > ms_compute else "the attention kernel",
                    "value_with_gather_gbs": info["gathered_kv_bytes_per_call"] * layers_n / (ms_overlap * 1e-3) / 1e9})
        # ---- parity, outside the timed region: the gathered output of layer 0 against rank 0's
        #      own single-GPU computation of units that another rank (the last one) computed
        step_serial()
        if isinstance(shared, list):
            step_fused()
        torch.cuda.synchronize()
        if isinstance(shared, list):                      # the kernel-gathered tensor against the NCCL-gathered one
            same = torch.tensor([int(torch.equal(shared[0].local, fulls[0]))], device=dev)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            rec["fused"]["equals_nccl_gather_on_every_rank"] = bool(same.item())
        if rank == 0:
            units = [n_units - 1, n_units - 2]
            q, k, v = (seeded_full((T, H, N, D), 1000 + j, dev, dtype) for j in range(3))
            worst = 0.0
            for u in units:
                qs, ks, vs = (t.narrow(dim, u, 1).contiguous() for t in (q, k, v))
                m1 = fst.build_tree_metadata(w.trees[u] if axis == "tree" else w.trees[0], w.block_m, w.max_ancestors,
                                             reference_format=False)
                want = fst.fst_attention(qs, ks, vs, m1, sm_scale=w.sm_scale, kernel=kernel)
                got = fulls[0].narrow(dim, u, 1)
                worst = max(worst, (got.float() - want.float()).abs().max().item())
            rec["parity_max_abs"] = worst
            rec["parity_units"] = f"{axis}s {units} (computed by rank {world - 1}), layer 0, against rank 0's own kernel run"
            # and a slice of the same against the CPU oracle (the checker, fp32 evaluation)
            from oracle import tree_oracle as orc
            u = units[0]
            if axis == "tree":
                sl = (slice(u, u + 1), slice(0, 4))
                par = w.trees[u]
            else:
                sl = (slice(0, 1), slice(u, u + 1))
                par = w.trees[0]
            lin, _ = orc.lineage_from_parent(par)
            mask = orc.full_attention_mask(lin, pad_rows=0)
            rows = torch.arange(N - 128, N)
            exact = orc.dense_tree_attention(q[sl][:, :, rows].cpu(), k[sl].cpu(), v[sl].cpu(), mask[rows], w.sm_scale,
                                             torch.float32)
            rec["parity_vs_oracle_max_abs"] = (fulls[0][sl][:, :, rows].cpu().float() - exact).abs().max().item()
            del q, k, v
    assert fst.last_status(dev) == 0
    del layers, locals_, fulls, g_compute, shared
    torch.cuda.empty_cache()
    return rec


def reference_triton_times(cases, dev, reps=20):
    """The reference's own Triton kernel and wrapper (the part of its fstattention.py above the
    test, from the copy under baseline/_ref), JIT-compiled here and timed with the protocol of
    measure_case: a CUDA graph of calls on rotating buffers, CUDA events.  The reference shares
    one tree between all batch elements, so a batch of different trees is one call per tree.
    Returns {case: {...}} or {"unavailable": why}."""
    path = os.path.join(REF_DIR, "fstattention.py")
    if not os.path.exists(path) or load_reference_utils() is None:
        return {"unavailable": "no copy of the reference under baseline/_ref"}
    try:
        import triton  # noqa: F401
        sys.path.insert(0, REF_DIR)
        head = open(path).read().split("def test_op", 1)[0]
        ns = {"__name__": "fst_reference_head"}
        exec(compile(head, path, "exec"), ns)
        ref_attention = ns["fst_attention"]
    except Exception as exc:                              # noqa: BLE001
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    finally:
        if REF_DIR in sys.path:
            sys.path.remove(REF_DIR)
    from oracle import tree_oracle as orc
    ref_utils = load_reference_utils()
    out = {}
    for case, w, layers_n in cases:
        try:
            dtype = DTYPES[w.dtype]
            T, H, N, D = len(w.trees), w.heads, w.n_nodes, w.head_dim
            g = torch.Generator(device=dev).manual_seed(5)
            metas = []
            for par in w.trees:
                lin, lvl = orc.lineage_from_parent(par)
                metas.append(tuple(t.to(dev) for t in ref_utils.create_fst_attention_kernel_inputs(
                    lin.clone(), lvl, block_m=w.block_m, max_ancestors=w.max_ancestors)))
            layers = [tuple(torch.randn((T, H, N, D), generator=g, device=dev, dtype=torch.float32).to(dtype)
                            for _ in range(3)) for _ in range(layers_n)]

            def calls():
                for (q, k, v) in layers:
                    for t, (ai, am, li) in enumerate(metas):
                        ref_attention(q[t:t + 1], k[t:t + 1], v[t:t + 1], ai, am, li, w.sm_scale,
                                      BLOCK_M=w.block_m, MAX_ANCESTORS=w.max_ancestors)

            graph = capture(calls)
            for _ in range(3):
                graph.replay()
            us = Timer(dev, 1)(graph.replay, reps) / reps / layers_n * 1e3
            out[case] = {"us_per_call": us, "launches_per_call": len(metas),
                         "gathered_kv_gbs": describe(w)["gathered_kv_bytes_per_call"] / us / 1e3}
            del layers, graph
            torch.cuda.empty_cache()
        except Exception as exc:                          # noqa: BLE001
            out[case] = {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}
    return out


def sweep_workload(configs, fst, n_ctx):
    """One point of the reference's own benchmark sweep (fstattention.py:240-296): B 4, H 48,
    D 64, fp16, the create_tree forest for that context, 128-row blocks, 64 ancestors."""
    lin, lvl = fst.create_tree(fst.DEPTH_MAPPING[n_ctx])
    par = fst.parent_from_lineage(lin, lvl).tolist()
    w = configs.Workload(f"sweep{n_ctx}", [par], heads=48 * 4, head_dim=64, dtype="fp16", block_m=128,
                         max_ancestors=fst.MAX_ANCESTOR_MAPPING[n_ctx],
                         notes="batch 4 x 48 heads share one tree: folded into 192 heads")
    return w


def run_ours(args, rank, world):
    import fstattention_b200 as fst
    from fstattention_b200 import configs
    import torch.distributed as dist

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    w = configs.workload(args.workload)
    if args.block_m or args.max_ancestors:
        w = with_block(w, args.block_m or w.block_m, args.max_ancestors or w.max_ancestors)
    info = describe(w)
    dtype = DTYPES[w.dtype]
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
        kv_by_seed = [describe(configs.workload(w.name, s_))["gathered_kv_bytes_per_call"] for s_ in seeds]

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

    g_step, g_attn, g_pre = capture(step), capture(attention_only), capture(precompute_only)
    timer = Timer(dev, world)

    for _ in range(max(args.warmup, 3)):
        g_step.replay()
    sampler = ClockSampler(local)
    sampler.start()
    total_ms = timer(g_step.replay, args.steps, next_tree)
    if len(sampler.samples) < 25:                         # a short run: keep the step going until the clock record
        extra = 0                                         # has a few dozen samples (untimed repeats of the same step)
        while len(sampler.samples) < 25 and extra < 2000:
            g_step.replay()
            extra += 1
        torch.cuda.synchronize()
    clocks = sampler.stop()
    ms_per_step = total_ms / args.steps
    assert meta.check() is meta and fst.last_status(dev) == 0
    if dynamic:                                           # the per-kernel figures below are for tree 0
        next_tree(0)
        g_step.replay()
    for _ in range(3):
        g_attn.replay()
    attn_ms = timer(g_attn.replay, args.steps) / args.steps
    for _ in range(3):
        g_pre.replay()
    pre_us = timer(g_pre.replay, args.steps) / args.steps / 16 * 1e3
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

        def e2e_step(compute=True):
            if compute:
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
                if compute:
                    fst.fst_attention(dq, dk, dv, meta, sm_scale=w.sm_scale, out=slot_out[sl], kernel=args.kernel)
                ev_cmp[sl].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[sl])
                    ho.copy_(slot_out[sl], non_blocking=True)
                    ev_out[sl].record(s_out)
            torch.cuda.synchronize()

        def wall(fn, n):
            timer.barrier()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            timer.barrier()
            dt = (time.perf_counter() - t0) / n
            if world > 1:
                t = torch.tensor([dt], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dt = t.item()
            return dt

        for _ in range(3):
            e2e_step()
        e2e_steps = max(3, min(args.steps, 10))
        dt = wall(e2e_step, e2e_steps)
        # the same copies with no attention between them: what the host side alone allows when
        # all ranks of the node copy at once
        dt_copy = wall(lambda: e2e_step(False), e2e_steps)
        tensor_bytes = T * H * N * D * (4 if w.dtype == "fp32" else 2)
        in_bytes = sum(t.numel() * t.element_size() for t in layers[0])
        e2e = {"value": world * kv * e2e_layers / dt / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": e2e_layers * in_bytes + parent.numel() * 4,
               "d2h_bytes_per_step": e2e_layers * tensor_bytes,
               "ms_per_step": dt * 1e3, "calls_per_step": e2e_layers,
               "us_per_call": dt * 1e6 / e2e_layers,
               "copies_only_us_per_call": dt_copy * 1e6 / e2e_layers,
               "copies_only_node_h2d_gbs": world * in_bytes * e2e_layers / dt_copy / 1e9,
               "overlap": "copy-in, attention and copy-out of consecutive calls on three streams, two device slots",
               "inputs": "q, k, v are views of one pinned buffer per call, one copy" if fused else "q, k, v pinned separately, three copies per call"}
        del host_in, host_out, slots, slot_out

    # ---- the other configurations, single GPU (rank 0 of a 1-GPU run), and the sharded ones
    del layers, outs, g_step, g_attn, g_pre
    torch.cuda.empty_cache()
    workloads, sharded, ref_gpu = None, None, None
    reps = max(5, min(args.steps, 20))
    if not args.no_workloads and args.workload == "medusa256":
        if world == 1:
            deep = configs.workload("deep4096")
            workloads = {
                "random1024": measure_case(fst, configs.workload("random1024"), 8, reps, dev, args.kernel),
                "forest64": measure_case(fst, configs.workload("forest64"), 2, reps, dev, args.kernel),
                "deep4096": measure_case(fst, deep, 3, reps, dev, args.kernel),
                "deep4096_bm128": measure_case(fst, with_block(deep, 128, 256), 3, reps, dev, args.kernel,
                                               case="deep4096_bm128"),
                "device_built_tree": measure_tree_build(fst, dev, reps),
            }
        sharded = {name: measure_sharded(fst, name, rank, world, dev, 4, reps, args.kernel)
                   for name in ("forest64", "deep4096")}
        if world == 1 and not args.no_reference_gpu:
            cases = [("medusa256", w, 40), ("forest64", configs.workload("forest64"), 2)]
            ref_gpu = reference_triton_times(cases, dev)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = time_cpu_reference(w, info, L, steps=10, warmup=2)

    if rank != 0:
        return
    # A long dense prefix makes the call compute-bound: the prefix goes to the tcgen05 kernel and
    # the bound is the tensor cores.  Algorithmic flops: every query block forms block_m x rows
    # scores and as many products with V, 2 * head_dim flops each.
    probe = torch.empty((T, H, N, D), device=dev, dtype=dtype)
    plan = fst.launch_plan(probe, w.prefix, w.block_m, args.kernel)
    del probe
    traffic, traffic_source = ncu_traffic(w.name)
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": traffic, "traffic_source": traffic_source, "peak_source": f"of {peak_kind}",
                "kernel": plan["kernels"][0] if args.kernel == "auto" else f"attn_{args.kernel}_kernel",
                "achieved_incl_q_o": (kv + info["q_o_bytes_per_call"]) / (launch_us * 1e-6) / 1e9,
                "frac_of_nominal_8000": achieved / 8000.0, "target_frac": 0.70}
    if "prefix_umma_kernel" in plan["kernels"]:
        tpeak, tkind = measured_tensor_peak()
        esize = 4 if w.dtype == "fp32" else 2
        flops = 4.0 * D * w.block_m * (kv / (2 * D * esize))
        tf = flops / (launch_us * 1e-6) / 1e12
        roofline = {"bound": "tensor", "achieved": tf, "peak": tpeak, "unit": "TFLOP/s", "frac": tf / tpeak,
                    "traffic": traffic, "traffic_source": traffic_source, "peak_source": f"of {tkind}",
                    "kernel": "prefix_umma_kernel", "flops_per_call": flops, "prefix_runs": plan["prefix_runs"],
                    "note": "time is the whole call: prefix kernel, tree kernel beside it, merge kernel"}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": workload_config(w, L),
        "run": {"how": "the step is a replayed CUDA graph: 1 precompute launch + calls_per_step attention launches",
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
        "roofline": roofline,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if workloads is not None:
        line["workloads"] = workloads
    if sharded is not None:
        line["sharded"] = sharded
    if ref_gpu is not None:
        line["vs_reference_gpu"] = {
            "what": "the reference's own Triton kernel (fstattention.py:21-181) JIT-compiled on this GPU, same "
                    "graph / rotating-buffer protocol; a batch of different trees is one reference call per tree",
            "reference": ref_gpu,
            "speedup": {c: ref_gpu[c]["us_per_call"] / (launch_us if c == w.name else workloads[c]["us_per_call"])
                        for c in ref_gpu if isinstance(ref_gpu.get(c), dict) and "us_per_call" in ref_gpu[c]
                        and (c == w.name or (workloads and c in workloads))}}
    print(json.dumps(line))


def run_sharded(args, rank, world):
    """--shard: the sharded measurement of one workload as the top-level line."""
    import fstattention_b200 as fst
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    sampler = ClockSampler(local)
    sampler.start()
    rec = measure_sharded(fst, args.workload, rank, world, dev, args.layers, max(5, args.steps), args.kernel)
    clocks = sampler.stop()
    if rank != 0:
        return
    L = args.layers
    step_ms = rec.get("step_ms_overlapped", rec["step_ms_no_gather"])
    line = {"metric": METRIC, "value": rec["gathered_kv_bytes_per_call"] * L / (step_ms * 1e-3) / 1e9, "unit": UNIT,
            "n_gpus": world, "steps": max(5, args.steps), "warmup": 3, "ms_per_step": step_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": rec["config"], "gpu_launches": max(5, args.steps) * (L + 1), "clocks": clocks,
            "roofline": rec["per_gpu_roofline"], "sharded": rec}
    print(json.dumps(line))


def run_reference(args, rank, world):
    """The reference's CPU path timed on the host cores, same metric, config and step as the GPU arm."""
    if rank != 0:
        return
    from fstattention_b200 import configs
    w = configs.workload(args.workload)
    info = describe(w)
    L = args.layers
    cpu = time_cpu_reference(w, info, L, steps=args.steps, warmup=max(args.warmup, 1), budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cpu["ms_per_step_composed"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": w.dtype,
        "data": "synthetic", "config": workload_config(w, L),
        "run": {"how": "host cores, torch CPU; precompute and attention timed apart on a bounded sample and composed "
                       "to 1 precompute + calls_per_step attention calls"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_reference_triton(args, rank, world):
    """The reference's own GPU kernel (Triton, JIT) on this box: the headline workload, the
    batched forest and points of the reference's own sweep, beside this library on the same shapes."""
    if rank != 0:
        return
    import fstattention_b200 as fst
    from fstattention_b200 import configs
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    cases = [("medusa256", configs.workload("medusa256"), 40), ("forest64", configs.workload("forest64"), 2)]
    for n_ctx in (2 ** i for i in range(10, 17)):            # the reference's own x axis (fstattention.py:245)
        cases.append((f"sweep{n_ctx}", sweep_workload(configs, fst, n_ctx), max(2, 32768 // n_ctx)))
    ref = reference_triton_times(cases, dev)
    ours = {}
    if "unavailable" not in ref:
        for case, w, layers_n in cases:
            ours[case] = measure_case(fst, w, layers_n, 20, dev)["us_per_call"]
    line = {"impl": "reference-triton", "metric": "tree_attn_us_per_call", "unit": "us", "higher_is_better": False,
            "reference": ref, "ours_us_per_call": ours,
            "speedup": {c: ref[c]["us_per_call"] / ours[c] for c in ours if "us_per_call" in ref.get(c, {})}}
    print(json.dumps(line))


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.impl == "reference-triton":
        run_reference_triton(args, rank, world)
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
