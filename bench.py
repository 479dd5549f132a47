#!/usr/bin/env python
"""Benchmark of the graph-attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W            (this package's CUDA kernels)
    python bench.py --impl reference --gpus N --steps K --warmup W

One step = one forward + backward pass of the fused attention chain
(maskedmm -> scale -> sparse_softmax -> vector_spmm and its gradients) over one synthetic graph.
The default workload is the R-MAT scale-21 power-law graph (edge factor 16, a/b/c/d =
.57/.19/.19/.05, duplicates and self-loops removed, self-loops added, int32 CSR), 4 heads x 32,
fp32, with the chunk tables of partition_csr(chunk_size=32).  With N > 1 every rank runs the
same workload on its own independently seeded graph (data-parallel, no collective in the data
path: weak scaling).  The metric is edges*heads per second over all ranks.

Printed keys beyond the contract: `roofline` (dominant kernel, algorithmic bytes / CUDA-event
time, against the measured HBM copy bandwidth), `cpu_baseline` (the torch CPU chain on a bounded
sample), `kernels` (per-kernel mean milliseconds of one step), `phases` (forward / backward ms).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch as th  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "fwd+bwd graph-attention edges*heads/s"
UNIT = "edges*heads/s"


# --------------------------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------------------------
WORKLOADS = {
    # name: (graph maker, heads, dim, dtype)
    "rmat21_attention": dict(kind="rmat", scale=21, edge_factor=16, heads=4, dim=32, dtype="f32"),
    "er_small_attention": dict(kind="er", n=4096, k=15, heads=8, dim=64, dtype="f32"),
    "banded_attention": dict(kind="banded", batch=4, length=8192, window=128, heads=8, dim=64, dtype="bf16"),
    "zipf_attention": dict(kind="zipf", n=1_000_000, total=50_000_000, heads=2, dim=64, dtype="f32"),
}
DTYPES = {"f32": th.float32, "bf16": th.bfloat16, "f64": th.float64}


def make_graph(spec, seed, device):
    from custom_op_benchmark_b200 import graphs
    if spec["kind"] == "rmat":
        return graphs.rmat_graph(spec["scale"], spec["edge_factor"], seed=seed, device=device)
    if spec["kind"] == "er":
        return graphs.er_graph(spec["n"], spec["k"], seed=seed).to(device)
    if spec["kind"] == "banded":
        return graphs.banded_graph(spec["batch"], spec["length"], spec["window"], device=device)
    if spec["kind"] == "zipf":
        return graphs.zipf_graph(spec["n"], spec["total"], seed=seed, device=device)
    raise ValueError(spec["kind"])


def describe(spec):
    if spec["kind"] == "rmat":
        return "R-MAT scale %d, edge factor %d" % (spec["scale"], spec["edge_factor"])
    if spec["kind"] == "er":
        return "Erdos-Renyi n=%d, %d in-neighbours + self-loop" % (spec["n"], spec["k"])
    if spec["kind"] == "banded":
        return "banded attention %d x %d, window +-%d" % (spec["batch"], spec["length"], spec["window"])
    return "rank-size (Zipf 1.1) in-degrees n=%d, %d edges" % (spec["n"], spec["total"])


def algorithmic_bytes(n_dst, n_src, e, h, d, s, i):
    """Compulsory bytes (every input read once, every output written once, no intermediate)."""
    f_dst, f_src = n_dst * h * d * s, n_src * h * d * s
    idx = (e + n_dst + 1) * i
    idx_t = (e + n_src + 1) * i
    stat = n_dst * h * 4
    return {
        # q, k, v read, o written, indices, lse written
        "attention_fwd": f_dst + 2 * f_src + f_dst + idx + stat,
        # q, o, dO, k, v read, dq written, indices, lse read, delta written
        "attention_bwd_dst": 3 * f_dst + 2 * f_src + f_dst + idx + 2 * stat,
        # k, v, q, dO read, dk, dv written, transposed indices, lse and delta read
        "attention_bwd_src": 2 * f_src + 2 * f_dst + 2 * f_src + idx_t + 2 * stat,
        # whole step with every tensor touched once: forward 4F + I + 4NH, backward 8F + 2I + P + 4NH
        "step": (2 * f_dst + 2 * f_src + idx + stat) + (4 * f_dst + 4 * f_src + idx + idx_t + e * i + stat),
    }


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        rows = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 9] or [r for _, r in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        num = lambda v: float(v) if v.replace(".", "", 1).isdigit() else None
        sm = [num(r[1]) for r in rows if num(r[1]) is not None]
        reasons = set()
        for r in rows:
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        pw = [num(r[3]) for r in rows if num(r[3]) is not None]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": num(rows[0][2]),
                "power_w_max": max(pw) if pw else None, "samples": len(rows), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------
# the GPU arm
# --------------------------------------------------------------------------------------------
def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def traffic_for(kernel, workload):
    """DRAM bytes per launch of `kernel` on `workload` from the committed ncu summary, if any."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if os.path.exists(path):
        return json.load(open(path)).get(workload, {}).get(kernel)
    return None


def run_gpu(args):
    from custom_op_benchmark_b200 import _capi, graphop, wrapper
    from custom_op_benchmark_b200.part_csr import partition_csr

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=th.device("cuda", local))
    dev = th.device("cuda", local)
    th.cuda.set_device(dev)
    spec = dict(WORKLOADS[args.workload])
    if args.scale and spec["kind"] == "rmat":
        spec["scale"] = args.scale
    h, d, dtype = spec["heads"], spec["dim"], DTYPES[spec["dtype"]]
    scale = d ** -0.5

    # -- inputs: graph resident on the device, features drawn on the host (pinned) -----------
    g = make_graph(spec, seed=rank, device=dev)
    row, ptr = partition_csr(g.indptr, 32)
    col, ptr_t = partition_csr(g.indptr_t, 32)
    row, ptr, col, ptr_t = (t.to(th.int32) for t in (row, ptr, col, ptr_t))
    e, n_dst, n_src = g.n_edges, g.n_dst, g.n_src
    gen = th.Generator().manual_seed(1000 + rank)
    host = [th.randn(n, h, d, generator=gen).to(dtype).pin_memory() for n in (n_dst, n_src, n_src, n_dst)]
    Q, K, V, dO = (t.to(dev) for t in host)
    lib = _capi.lib()

    def step_device():
        o, lse = graphop.attention_forward(row, ptr, g.indices, Q, K, V, scale)
        return o, graphop.attention_backward(row, ptr, g.indices, col, ptr_t, g.indices_t, Q, K, V, o, lse, dO, scale)

    warmup = args.warmup if args.lean else max(args.warmup, 3)
    for _ in range(warmup):
        step_device()
    th.cuda.synchronize()
    if args.lean:
        # capture mode for profilers: the timed steps only, nothing else launched afterwards
        a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            step_device()
        b.record()
        th.cuda.synchronize()
        print(json.dumps({"lean": True, "workload": args.workload, "edges": e, "nodes": n_dst, "heads": h, "dim": d,
                          "ms_per_step": a.elapsed_time(b) / args.steps}))
        return

    # -- timed region: K steps, inputs resident, CUDA events on the launching stream ----------
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    if world > 1:
        dist.barrier()
    th.cuda.synchronize()
    ev = [th.cuda.Event(enable_timing=True) for _ in range(2 * args.steps + 1)]
    launches0 = lib.graphop_launch_count()
    t_wall0 = time.time()
    ev[0].record()
    for i in range(args.steps):
        o, lse = graphop.attention_forward(row, ptr, g.indices, Q, K, V, scale)
        ev[2 * i + 1].record()
        graphop.attention_backward(row, ptr, g.indices, col, ptr_t, g.indices_t, Q, K, V, o, lse, dO, scale)
        ev[2 * i + 2].record()
    th.cuda.synchronize()
    t_wall1 = time.time()
    launches = lib.graphop_launch_count() - launches0
    if world > 1:
        dist.barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    fwd_ms = statistics.mean(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(args.steps))
    bwd_ms = statistics.mean(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(args.steps))

    # -- end to end: the autograd Function a user calls, host buffers copied in and out every step
    outs = [th.empty_like(t).pin_memory() for t in (host[0], host[0], host[1], host[2])]
    dQ_, dK_, dV_, dO_ = (th.empty_like(t) for t in (Q, K, V, dO))

    def step_e2e():
        q = dQ_.copy_(host[0], non_blocking=True).requires_grad_(True)
        k = dK_.copy_(host[1], non_blocking=True).requires_grad_(True)
        v = dV_.copy_(host[2], non_blocking=True).requires_grad_(True)
        go = dO_.copy_(host[3], non_blocking=True)
        out = wrapper.GraphAttention.apply(row, ptr, g.indices, col, ptr_t, g.indices_t, q, k, v, scale)
        out.backward(go)
        outs[0].copy_(out.detach(), non_blocking=True)
        outs[1].copy_(q.grad, non_blocking=True)
        outs[2].copy_(k.grad, non_blocking=True)
        outs[3].copy_(v.grad, non_blocking=True)
        for t in (dQ_, dK_, dV_):
            t.requires_grad_(False)
            t.grad = None

    e2e_steps = max(2, min(args.steps, 5))
    step_e2e()
    th.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(e2e_steps):
        step_e2e()
    b.record()
    th.cuda.synchronize()
    e2e_ms = a.elapsed_time(b) / e2e_steps
    sampler.stop()
    clocks = sampler.summary(t_wall0, t_wall1)

    # -- per-kernel times of the same step, CUDA events behind every kernel ---------------------
    per_kernel = {}
    prof_steps = max(2, min(args.steps, 5))
    step_device()            # the e2e loop left the allocator in another state: settle it before timing
    th.cuda.synchronize()
    recs = _capi.profile(lambda: [step_device() for _ in range(prof_steps)], th.cuda.current_stream().cuda_stream)
    for name, ms in recs:
        per_kernel.setdefault(name, []).append(ms)
    kernels = {k: {"launches_per_step": len(v) / prof_steps, "ms_per_step": sum(v) / prof_steps}
               for k, v in per_kernel.items()}

    # -- reduce over ranks ---------------------------------------------------------------------
    stats = th.tensor([total_ms, e2e_ms, fwd_ms, bwd_ms], dtype=th.float64, device=dev)
    work = th.tensor([float(e) * h], dtype=th.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms, fwd_ms, bwd_ms = stats.tolist()
    units = work.item()  # edges*heads of all ranks, per step

    if rank == 0:
        s_bytes, i_bytes = Q.element_size(), 4
        alg = algorithmic_bytes(n_dst, n_src, e, h, d, s_bytes, i_bytes)
        top = max((k for k in kernels if k in alg), key=lambda k: kernels[k]["ms_per_step"])
        top_ms = kernels[top]["ms_per_step"] / max(1.0, kernels[top]["launches_per_step"])
        peak, peak_kind = measured_peak()
        achieved = alg[top] / (top_ms * 1e-3) / 1e9
        ms_per_step = total_ms / args.steps
        feat_bytes = sum(t.numel() * t.element_size() for t in host)
        out = {
            "metric": METRIC, "value": units / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": spec["dtype"],
            "data": "synthetic",
            "config": {"workload": args.workload, "graph": describe(spec), "nodes": n_dst, "edges": e, "heads": h,
                       "dim": d, "index": "int32 CSR, chunk tables of partition_csr(32)", "per_rank": "own graph",
                       "l2": "inputs (%.1f GB of node features) larger than the 126 MB L2" % (feat_bytes / 1e9),
                       "resident": "graph structure; e2e copies Q, K, V, dO in and O, dQ, dK, dV out every step"},
            "e2e": {"value": units / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": feat_bytes, "d2h_bytes_per_step": feat_bytes},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "phases": {"forward_ms": fwd_ms, "backward_ms": bwd_ms},
            "roofline": {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": peak_kind, "algorithmic_bytes": alg[top],
                         "ms": top_ms, "traffic": traffic_for(top, args.workload),
                         "step_algorithmic_bytes": alg["step"],
                         "step_frac": alg["step"] / (ms_per_step * 1e-3) / 1e9 / peak},
            "kernels": kernels,
        }
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(spec, args.cpu_sample_scale)
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# the CPU baseline and the reference arm
# --------------------------------------------------------------------------------------------
def cpu_baseline(spec, sample_scale):
    """The torch CPU chain (oracle/cpu_baseline.py) timed on a bounded sample of the workload."""
    from custom_op_benchmark_b200 import graphs
    from oracle import cpu_baseline as cb
    h, d = spec["heads"], spec["dim"]
    if spec["kind"] == "rmat":
        g = graphs.rmat_graph(min(sample_scale, spec["scale"]), spec["edge_factor"], seed=0)
        sample = "R-MAT scale %d, edge factor %d (same generator and parameters), %d edges" % (
            min(sample_scale, spec["scale"]), spec["edge_factor"], g.n_edges)
    elif spec["kind"] == "er":
        g = graphs.er_graph(spec["n"], spec["k"], seed=0)
        sample = "the whole workload"
    elif spec["kind"] == "banded":
        g = graphs.banded_graph(1, spec["length"], spec["window"])
        sample = "one of the %d sequences" % spec["batch"]
    else:
        g = graphs.zipf_graph(spec["n"] // 25, spec["total"] // 25, cap=spec["total"] // 25, seed=0)
        sample = "the same degree law at 1/25 of the nodes and edges"
    gen = th.Generator().manual_seed(1)
    Q, K, V, dO = (th.randn(n, h, d, generator=gen) for n in (g.n_dst, g.n_src, g.n_src, g.n_dst))
    sec = cb.time_chain(g.indptr, g.indices, Q, K, V, d ** -0.5, dO, repeats=1)
    return {"value": g.n_edges * h / sec, "unit": UNIT, "cores": th.get_num_threads(), "host_cpus": os.cpu_count(),
            "kind": "port", "seconds": sec,
            "sample": sample + "; torch CPU fp32 chain, forward + backward through autograd"}


def run_reference(args):
    """Reference arm.  The reference is a CUDA-only extension with no CPU implementation of its
    own, so this arm times the torch CPU restatement of its chain on the host cores, every step a
    bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    spec = dict(WORKLOADS[args.workload])
    h = spec["heads"]
    base = None
    secs = []
    for _ in range(max(1, min(args.warmup, 1)) + max(1, min(args.steps, 3))):
        base = cpu_baseline(spec, args.cpu_sample_scale)
        secs.append(base["seconds"])
    secs = secs[1:] or secs
    sec = statistics.mean(secs)
    edges_heads = base["value"] * base["seconds"]
    value = edges_heads / sec
    base["value"] = value
    world = int(os.environ.get("WORLD_SIZE", "1"))
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
           "steps": len(secs), "warmup": 1, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "f32", "data": "synthetic",
           "config": {"workload": args.workload, "graph": describe(spec), "heads": h, "dim": spec["dim"],
                      "note": "the reference has no CPU code path; this is the torch CPU restatement of its chain"},
           "cpu_baseline": base,
           "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="graphop_b200", choices=["graphop_b200", "reference"])
    ap.add_argument("--workload", default="rmat21_attention", choices=sorted(WORKLOADS))
    ap.add_argument("--scale", type=int, default=0, help="override the R-MAT scale (smaller runs)")
    ap.add_argument("--cpu-sample-scale", type=int, default=18)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--lean", action="store_true",
                    help="warm-up and timed steps only (for ncu captures); prints a reduced line")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
