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
    # the fused chain (maskedmm -> scale -> sparse_softmax -> vector_spmm), forward + backward
    "rmat21_attention": dict(kind="rmat", scale=21, edge_factor=16, heads=4, dim=32, dtype="f32", ops="attention"),
    "er_small_attention": dict(kind="er", n=4096, k=15, heads=8, dim=64, dtype="f32", ops="attention"),
    "banded_attention": dict(kind="banded", batch=4, length=8192, window=128, heads=8, dim=64, dtype="bf16",
                             ops="attention"),
    # the banded layer on ONE sequence of 32768 positions, its graph cut by rows over the ranks, K / V halo rows exchanged every step (strong scaling)
    "banded_halo_attention": dict(kind="banded", batch=1, length=32768, window=128, heads=8, dim=64, dtype="bf16",
                                  ops="halo_attention"),
    "zipf_attention": dict(kind="zipf", n=1_000_000, total=50_000_000, heads=2, dim=64, dtype="f32", ops="attention"),
    # the fused chain with the node_mul_edge term in the scores (relative-position attention), forward + backward
    "rmat21_attention_bias": dict(kind="rmat", scale=21, edge_factor=16, heads=4, dim=32, dtype="f32",
                                  ops="attention_bias"),
    # node_mul_edge + vector_spmm, forward + backward, softmax-normalised edge weights (GAT style)
    "rmat21_gat": dict(kind="rmat", scale=21, edge_factor=16, heads=4, dim=32, dtype="f32", ops="gat"),
    # maskedmm + sparse_softmax, forward + backward, inputs scaled by 3 (max-subtraction stress)
    "zipf_sddmm_softmax": dict(kind="zipf", n=1_000_000, total=50_000_000, heads=2, dim=64, dtype="f32",
                               ops="sddmm_softmax"),
    # vector_spmm forward + backward on ONE graph cut by destination rows over the ranks (strong scaling):
    # source features all-gathered forward, dy all-gathered backward
    "rmat24_spmm": dict(kind="rmat", scale=24, edge_factor=32, heads=1, dim=128, dtype="f32", ops="sharded_spmm"),
}
DTYPES = {"f32": th.float32, "bf16": th.bfloat16, "f64": th.float64}


class Twin:
    """libgraphop_b200_bench.so: the library's sources compiled a second time with launch accounting and a CUDA
    event behind every kernel (custom_op_benchmark_b200/csrc/bench/graphop_bench.h).  The timed region of the
    benchmark runs through the product library; the same step is replayed through this twin to split its time
    over the kernels, to count the launches and to time the gather probe."""

    def __init__(self, path=None):
        import ctypes
        from custom_op_benchmark_b200 import _capi
        path = path or os.path.join(ROOT, "custom_op_benchmark_b200", "libgraphop_b200_bench.so")
        if not os.path.exists(path):
            raise ImportError("%s is missing; build it with `python -m custom_op_benchmark_b200.build`" % path)
        self._capi, self._ct = _capi, ctypes
        h = _capi.bind(ctypes.CDLL(path), strict=False)
        P, I64, INT, SZ = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
        h.graphop_bench_launch_count.argtypes, h.graphop_bench_launch_count.restype = [], ctypes.c_longlong
        h.graphop_bench_profile_begin.argtypes, h.graphop_bench_profile_begin.restype = [P], INT
        h.graphop_bench_profile_end.argtypes, h.graphop_bench_profile_end.restype = [P, SZ, P, INT], INT
        h.graphop_bench_gather_probe_i32.argtypes = [P, I64, P, P, INT, P, P]
        h.graphop_bench_gather_probe_i32.restype = INT
        self.h = h

    class _Routed:
        def __init__(self, capi, handle):
            self.capi, self.handle = capi, handle

        def __enter__(self):
            self.capi.lib()                      # make sure the product library is what gets restored
            self.saved, self.capi._lib = self.capi._lib, self.handle

        def __exit__(self, *exc):
            self.capi._lib = self.saved

    def routed(self):
        """Context in which the package's ops call the twin instead of the product library."""
        return Twin._Routed(self._capi, self.h)

    def launch_count(self):
        return int(self.h.graphop_bench_launch_count())

    def profile(self, fn, stream, max_entries=8192):
        """Runs fn() through the twin with per-kernel timing on; returns [(kernel name, milliseconds), ...]."""
        ct = self._ct
        with self.routed():
            if self.h.graphop_bench_profile_begin(stream) != 0:
                raise RuntimeError("graphop_bench_profile_begin failed")
            try:
                fn()
            finally:
                names = ct.create_string_buffer(64 * max_entries)
                ms = (ct.c_float * max_entries)()
                n = self.h.graphop_bench_profile_end(ct.cast(names, ct.c_void_p), len(names),
                                                     ct.cast(ms, ct.c_void_p), max_entries)
        if n < 0:
            raise RuntimeError("graphop_bench_profile_end failed")
        return list(zip(names.value.decode().split("\n")[:n], [float(v) for v in ms[:n]]))

    def gather_probe(self, idx, t0, t1, row_bytes, sink, stream):
        rc = self.h.graphop_bench_gather_probe_i32(idx.data_ptr(), idx.numel(), t0.data_ptr(),
                                                   t1.data_ptr() if t1 is not None else None, row_bytes,
                                                   sink.data_ptr(), stream)
        if rc:
            raise RuntimeError("graphop_bench_gather_probe_i32 failed: %d" % rc)


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


def _nbytes(ts):
    return sum(t.numel() * t.element_size() for t in ts)


def _pinned(t):
    """Page-locked copy of a host tensor; the pageable tensor itself if the host refuses to pin that much."""
    try:
        return t.pin_memory()
    except RuntimeError:
        return t


class Workload:
    """One rank's inputs and its step.  `host` tensors are pinned (the e2e leg copies them in every
    step), `alg` maps a kernel name of the library's profile to its compulsory bytes per launch."""

    def __init__(self, spec, rank, dev):
        from custom_op_benchmark_b200.part_csr import partition_csr
        self.spec, self.dev = spec, dev
        self.h, self.d, self.dtype = spec["heads"], spec["dim"], DTYPES[spec["dtype"]]
        g = make_graph(spec, seed=rank, device=dev)
        row, ptr = partition_csr(g.indptr, 32)
        col, ptr_t = partition_csr(g.indptr_t, 32)
        self.R = [row.to(th.int32), ptr.to(th.int32), g.eid, g.indices]
        self.C = [col.to(th.int32), ptr_t.to(th.int32), g.eid_t, g.indices_t]
        self.g, self.e, self.n_dst, self.n_src = g, g.n_edges, g.n_dst, g.n_src
        # graph plans: what depends on the graph alone (owner of every position, shape flags), built once like the
        # chunk tables above; `planned` = False times the chunk-table entry points, which rebuild it in every call
        from custom_op_benchmark_b200 import graphop
        th.cuda.synchronize()
        t0 = time.time()
        self.plan_r = graphop.GraphPlan(*self.R, g.n_dst)
        self.plan_t = graphop.GraphPlan(*self.C, g.n_src)
        th.cuda.synchronize()
        self.plan_build_ms = (time.time() - t0) * 1e3
        self.planned = True
        self.gen = th.Generator().manual_seed(1000 + rank)

    def _host(self, *shape, mag=1.0):
        return (th.randn(*shape, generator=self.gen) * mag).to(self.dtype).pin_memory()

    def _release(self, leaves):
        for t in leaves:
            t.requires_grad_(False)
            t.grad = None

    def units(self):
        return float(self.e) * self.h

    def sizes(self):
        s, i = th.empty(0, dtype=self.dtype).element_size(), 4
        f_dst, f_src = self.n_dst * self.h * self.d * s, self.n_src * self.h * self.d * s
        return dict(s=s, i=i, F_dst=f_dst, F_src=f_src, S=self.e * self.h * s, I=(self.e + self.n_dst + 1) * i,
                    I_t=(self.e + self.n_src + 1) * i, stat=self.n_dst * self.h * 4, Be=self.e * self.d * s,
                    P=self.e * i)

    def e2e_bytes(self):
        return _nbytes(self.host), _nbytes(self.outs)

    def gather_streams(self):
        """{kernel name: (int32 index stream, table, table or None)}: what each walker kernel gathers per edge."""
        return {}

    def gather_bytes(self, kernel):
        """B_gather of `kernel`: its compulsory bytes with every gathered node tensor counted once per edge
        (the traffic of a machine without caches), or None when the kernel gathers nothing we track."""
        streams = self.gather_streams()
        if kernel not in streams or kernel not in self.alg:
            return None
        _, t0, t1 = streams[kernel]
        tables = [t for t in (t0, t1) if t is not None]
        once = sum(t.numel() * t.element_size() for t in tables)
        per_edge = sum(t[0].numel() * t.element_size() for t in tables) * self.e
        return self.alg[kernel] - once + per_edge

    def gather_floor(self, twin, reps=5):
        """Milliseconds of graphop_bench_gather_probe_i32 (the gathers alone, nothing done with the rows) for
        every kernel of gather_streams() whose rows are at most 512 bytes; {} when there is none."""
        out = {}
        sink = th.zeros(1, dtype=th.int32, device=self.dev)
        stream = th.cuda.current_stream().cuda_stream
        for name, (idx, t0, t1) in self.gather_streams().items():
            row_bytes = t0[0].numel() * t0.element_size()
            if idx.dtype != th.int32 or row_bytes > 512 or row_bytes % 16:
                continue

            def go():
                twin.gather_probe(idx, t0, t1, row_bytes, sink, stream)
            for _ in range(3):
                go()
            a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                go()
            b.record()
            th.cuda.synchronize()
            out[name] = a.elapsed_time(b) / reps
        return out


class AttentionWorkload(Workload):
    name = "fused attention forward + backward"
    resident = "graph structure; e2e copies Q, K, V, dO in and O, dQ, dK, dV out every step"

    def __init__(self, spec, rank, dev):
        super().__init__(spec, rank, dev)
        n, m, h, d = self.n_dst, self.n_src, self.h, self.d
        self.host = [self._host(n, h, d), self._host(m, h, d), self._host(m, h, d), self._host(n, h, d)]
        self.Q, self.K, self.V, self.dO = (t.to(dev) for t in self.host)
        self.scale = d ** -0.5
        self.outs = [th.empty_like(t).pin_memory() for t in (self.host[0], self.host[0], self.host[1], self.host[2])]
        z = self.sizes()
        self.alg = {
            # q, k, v read, o written, indices, lse written
            "attention_fwd": z["F_dst"] + 2 * z["F_src"] + z["F_dst"] + z["I"] + z["stat"],
            # the tensor-core kernel of dense-band graphs reads (first, count) per node instead of the edge list
            "attention_fwd_banded": z["F_dst"] + 2 * z["F_src"] + z["F_dst"] + 2 * self.n_dst * 4 + z["stat"],
            "attention_bwd_dst_banded": 3 * z["F_dst"] + 2 * z["F_src"] + z["F_dst"] + 2 * self.n_dst * 4 + 3 * z["stat"],
            "attention_bwd_src_banded": 2 * z["F_src"] + 2 * z["F_dst"] + 2 * z["F_src"] + 2 * self.n_src * 4 + 2 * z["stat"],
            # q, o, dO, k, v read, dq written, indices, lse read, delta written
            "attention_bwd_dst": 3 * z["F_dst"] + 2 * z["F_src"] + z["F_dst"] + z["I"] + 2 * z["stat"],
            # k, v, q, dO read, dk, dv written, transposed indices, lse and delta read
            "attention_bwd_src": 2 * z["F_src"] + 2 * z["F_dst"] + 2 * z["F_src"] + z["I_t"] + 2 * z["stat"],
        }
        # every tensor once: forward 4F + I + 4NH, backward 8F + 2I + P + 4NH
        self.alg_step = (2 * z["F_dst"] + 2 * z["F_src"] + z["I"] + z["stat"]) + \
                        (4 * z["F_dst"] + 4 * z["F_src"] + z["I"] + z["I_t"] + z["P"] + z["stat"])

    def gather_streams(self):
        return {"attention_fwd": (self.R[3], self.K, self.V), "attention_bwd_dst": (self.R[3], self.K, self.V),
                "attention_bwd_src": (self.C[3], self.Q, self.dO)}

    def forward(self):
        from custom_op_benchmark_b200 import graphop
        R = self.R
        if self.planned:
            self.o, self.lse = graphop.attention_forward_planned(self.plan_r, self.Q, self.K, self.V, self.scale)
        else:
            self.o, self.lse = graphop.attention_forward(R[0], R[1], R[3], self.Q, self.K, self.V, self.scale)

    def backward(self):
        from custom_op_benchmark_b200 import graphop
        R, C = self.R, self.C
        if self.planned:
            return graphop.attention_backward_planned(self.plan_r, self.plan_t, self.Q, self.K, self.V, self.o,
                                                      self.lse, self.dO, self.scale)
        return graphop.attention_backward(R[0], R[1], R[3], C[0], C[1], C[3], self.Q, self.K, self.V, self.o, self.lse,
                                          self.dO, self.scale, eid_t=C[2])

    def max_err(self):
        from oracle import edge_list_f64 as ref
        self.forward()
        got = [self.o, self.lse] + list(self.backward())
        want = ref.attention_f64(self.g.indptr, self.g.indices, self.Q, self.K, self.V, self.scale, self.dO)
        out = {}
        for name, a, b in zip(("o", "lse", "dq", "dk", "dv"), got, want):
            keep = th.isfinite(b)
            out[name] = ref.max_err(a[keep], b[keep])[0]
        return dict(out, max_err=max(out.values()),
                    what="every element of O, lse, dQ, dK, dV of one step against the float64 edge-list reference "
                         "on the same inputs, |x - ref| / (1 + |ref|)")

    def e2e_compute(self, stage):
        from custom_op_benchmark_b200 import wrapper
        R, C = self.R, self.C
        q, k, v = (t.detach().requires_grad_(True) for t in stage[:3])
        if self.planned:
            out = wrapper.GraphAttentionPlanned.apply(self.plan_r, self.plan_t, q, k, v, self.scale)
        else:
            out = wrapper.GraphAttention.apply(R[0], R[1], R[3], C[0], C[1], C[3], q, k, v, self.scale, C[2])
        out.backward(stage[3])
        return [out.detach(), q.grad, k.grad, v.grad]


class AttentionBiasWorkload(AttentionWorkload):
    name = "fused attention with an edge term in the scores, forward + backward"
    resident = "graph structure and the (edges, dim) edge-term tensor rel; e2e copies Q, K, V, dO in and O, dQ, dK, " \
               "dV out every step (d_rel stays on the device)"

    def __init__(self, spec, rank, dev):
        super().__init__(spec, rank, dev)
        gen = th.Generator(device=dev).manual_seed(2000 + rank)
        self.rel = (th.randn(self.e, self.d, generator=gen, device=dev) * 0.5).to(self.dtype)
        z = self.sizes()
        pairs = self.e * self.h * 8
        self.alg = {
            "attention_bias_fwd": self.alg["attention_fwd"] + z["Be"],
            # as attention_bwd_dst, plus rel read and (p, ds) of every edge written
            "attention_bias_bwd_dst": self.alg["attention_bwd_dst"] + z["Be"] + pairs,
            # owner of every position and the pairs read, q read, d_rel written
            "attention_bias_grad": z["P"] + pairs + z["F_dst"] + z["Be"],
            # q, dO read, dk, dv written, transposed indices and edge ids, the pairs read
            "attention_bwd_src_pairs": 2 * z["F_dst"] + 2 * z["F_src"] + z["I_t"] + z["P"] + pairs,
        }
        self.alg_step += 3 * z["Be"]        # rel read by both passes, d_rel written
        self.planned = False                 # the edge-term entry points take chunk tables

    def gather_streams(self):
        return {"attention_bias_fwd": (self.R[3], self.K, self.V), "attention_bias_bwd_dst": (self.R[3], self.K, self.V)}

    def forward(self):
        from custom_op_benchmark_b200 import graphop
        R = self.R
        self.o, self.lse = graphop.attention_bias_forward(R[0], R[1], R[3], self.Q, self.K, self.V, self.rel,
                                                          self.scale)

    def backward(self):
        from custom_op_benchmark_b200 import graphop
        R, C = self.R, self.C
        return graphop.attention_bias_backward(R[0], R[1], R[3], C[0], C[1], C[2], C[3], self.Q, self.K, self.V,
                                               self.rel, self.o, self.lse, self.dO, self.scale)

    def max_err(self):
        from oracle import edge_list_f64 as ref
        self.forward()
        got = [self.o, self.lse] + list(self.backward())
        want = ref.attention_f64(self.g.indptr, self.g.indices, self.Q, self.K, self.V, self.scale, self.dO,
                                 rel=self.rel)
        out = {}
        for name, a, b in zip(("o", "lse", "dq", "dk", "dv", "d_rel"), got, want):
            keep = th.isfinite(b)
            out[name] = ref.max_err(a[keep], b[keep])[0]
        return dict(out, max_err=max(out.values()),
                    what="every element of O, lse, dQ, dK, dV, d_rel of one step against the float64 edge-list "
                         "reference on the same inputs, |x - ref| / (1 + |ref|)")

    def e2e_compute(self, stage):
        from custom_op_benchmark_b200 import wrapper
        R, C = self.R, self.C
        q, k, v = (t.detach().requires_grad_(True) for t in stage[:3])
        rel = self.rel.detach().requires_grad_(True)
        out = wrapper.GraphAttentionBias.apply(R[0], R[1], R[3], C[0], C[1], C[2], C[3], q, k, v, rel, self.scale)
        out.backward(stage[3])
        return [out.detach(), q.grad, k.grad, v.grad]


class GatWorkload(Workload):
    name = "node_mul_edge + vector_spmm, forward + backward"
    resident = "graph structure; e2e copies X, B_edge, the edge weights and both upstream gradients in, both " \
               "outputs and the three gradients out every step"

    def __init__(self, spec, rank, dev):
        from custom_op_benchmark_b200 import graphop
        super().__init__(spec, rank, dev)
        n, h, d, e = self.n_dst, self.h, self.d, self.e
        raw = th.rand(e, h, generator=self.gen).to(self.dtype).to(dev)
        w = graphop.sparse_softmax_forward(*self.R[:3], raw)          # sparse_softmax-normalised weights
        self.host = [self._host(n, h, d), self._host(e, d), w.cpu().pin_memory(), self._host(e, h), self._host(n, h, d)]
        self.X, self.Be, self.w, self.dY1, self.dY2 = (t.to(dev) for t in self.host)
        self.outs = [th.empty(s, dtype=self.dtype).pin_memory() for s in ((e, h), (n, h, d), (e, d), (n, h, d), (e, h))]
        z = self.sizes()
        gather = 2 * z["F_dst"] + z["S"] + z["I"]
        self.alg = {"edge_dot": gather, "aggregate": gather,
                    "aggregate_edge_feat": z["F_dst"] + z["Be"] + z["S"] + z["I"],
                    "edge_mix_heads": z["F_dst"] + 2 * z["Be"] + z["S"]}
        # node_mul_edge fwd F + Be + S, bwd 2F + 2Be + S; spmm fwd 2F + S + I, bwd 3F + 2S + 2I + P
        self.alg_step = (z["F_dst"] + z["Be"] + z["S"]) + (2 * z["F_dst"] + 2 * z["Be"] + z["S"]) + \
                        (2 * z["F_dst"] + z["S"] + z["I"]) + (3 * z["F_dst"] + 2 * z["S"] + 2 * z["I"] + z["P"])

    def forward(self):
        from custom_op_benchmark_b200 import graphop
        if self.planned:
            self.y1 = graphop.node_mul_edge_forward_planned(self.plan_r, self.X, self.Be)
            self.y2 = graphop.vector_spmm_forward_planned(self.plan_r, self.w, self.X)
        else:
            self.y1 = graphop.node_mul_edge_forward(*self.R[:3], self.X, self.Be)
            self.y2 = graphop.vector_spmm_forward(*self.R, self.w, self.X)

    def backward(self):
        from custom_op_benchmark_b200 import graphop
        if self.planned:
            a = graphop.node_mul_edge_backward_planned(self.plan_r, self.X, self.Be, self.dY1)
            b = graphop.vector_spmm_backward_planned(self.plan_r, self.plan_t, self.w, self.dY2, self.X)
        else:
            a = graphop.node_mul_edge_backward(*self.R[:3], self.X, self.Be, self.dY1)
            b = graphop.vector_spmm_backward(*self.R, *self.C, self.w, self.dY2, self.X)
        return a + b

    def max_err(self):
        from oracle import edge_list_f64 as ref
        self.forward()
        da, dbe, dw, dx = self.backward()
        want = ref.gat_f64(self.g.indptr, self.g.indices, self.X, self.Be, self.w, self.dY1, self.dY2)
        got = (self.y1, self.y2, da + dx, dbe, dw)     # X feeds both ops: its gradient is the sum of the two
        out = {name: ref.max_err(a, b)[0] for name, a, b in zip(("y1", "y2", "dX", "dBe", "dw"), got, want)}
        return dict(out, max_err=max(out.values()),
                    what="every element of both outputs and the three gradients against the float64 edge-list "
                         "reference, |x - ref| / (1 + |ref|)")

    def e2e_compute(self, stage):
        from custom_op_benchmark_b200 import wrapper
        x, be, w = (t.detach().requires_grad_(True) for t in stage[:3])
        y1 = wrapper.NodeMulEdge.apply(*self.R[:3], x, be)
        y2 = wrapper.VectorSPMM.apply(*self.R, *self.C, w, x)
        th.autograd.backward([y1, y2], [stage[3], stage[4]])
        return [y1.detach(), y2.detach(), be.grad, x.grad, w.grad]


class SddmmSoftmaxWorkload(Workload):
    name = "maskedmm + sparse_softmax, forward + backward"
    resident = "graph structure; e2e copies Q, K and the upstream gradient in, the probabilities and dQ, dK out"

    def __init__(self, spec, rank, dev):
        super().__init__(spec, rank, dev)
        n, m, h, d, e = self.n_dst, self.n_src, self.h, self.d, self.e
        self.host = [self._host(n, h, d, mag=3.0), self._host(m, h, d, mag=3.0), self._host(e, h)]
        self.Q, self.K, self.dP = (t.to(dev) for t in self.host)
        self.outs = [th.empty(s, dtype=self.dtype).pin_memory() for s in ((e, h), (n, h, d), (m, h, d))]
        z = self.sizes()
        gather = z["F_dst"] + z["F_src"] + z["S"] + z["I"]
        self.alg = {"edge_dot": gather, "aggregate": gather,
                    "softmax_fwd_tile": 2 * z["S"] + (self.n_dst + 1) * z["i"],
                    "softmax_bwd_tile": 3 * z["S"] + (self.n_dst + 1) * z["i"]}
        # SDDMM fwd 2F + S + I, bwd 4F + S + 2I + P; softmax fwd 2S + (N+1)i, bwd 3S + (N+1)i
        self.alg_step = (2 * z["F_dst"] + z["S"] + z["I"]) + (4 * z["F_dst"] + z["S"] + 2 * z["I"] + z["P"]) + \
                        5 * z["S"] + 2 * (self.n_dst + 1) * z["i"]

    def forward(self):
        from custom_op_benchmark_b200 import graphop
        if self.planned:
            self.s = graphop.maskedmm_csr_forward_planned(self.plan_r, self.Q, self.K)
            self.p = graphop.sparse_softmax_forward_planned(self.plan_r, self.s)
        else:
            self.s = graphop.maskedmm_csr_forward(*self.R, self.Q, self.K)
            self.p = graphop.sparse_softmax_forward(*self.R[:3], self.s)

    def backward(self):
        from custom_op_benchmark_b200 import graphop
        if self.planned:
            ds = graphop.sparse_softmax_backward_planned(self.plan_r, self.p, self.dP)
            return graphop.maskedmm_csr_backward_planned(self.plan_r, self.plan_t, self.Q, self.K, ds)
        ds = graphop.sparse_softmax_backward(*self.R[:3], self.p, self.dP)
        return graphop.maskedmm_csr_backward(*self.R, *self.C, self.Q, self.K, ds)

    def max_err(self):
        from oracle import edge_list_f64 as ref
        self.forward()
        dq, dk = self.backward()
        want = ref.sddmm_softmax_f64(self.g.indptr, self.g.indices, self.Q, self.K, self.dP)
        out = {name: ref.max_err(a, b)[0] for name, a, b in zip(("s", "p", "dq", "dk"), (self.s, self.p, dq, dk), want)}
        return dict(out, max_err=max(out.values()),
                    what="every score, probability and gradient element against the float64 edge-list reference, "
                         "|x - ref| / (1 + |ref|)")

    def e2e_compute(self, stage):
        from custom_op_benchmark_b200 import wrapper
        q, k = (t.detach().requires_grad_(True) for t in stage[:2])
        s = wrapper.MaskedMMCSR.apply(*self.R, *self.C, q, k)
        p = wrapper.SparseSoftmax.apply(*self.R[:3], s)
        p.backward(stage[2])
        return [p.detach(), q.grad, k.grad]


def sharding_local_indptr(row, indptr_, n_rows):
    """Plain CSR indptr (n_rows + 1, int64) of a shard from its chunk table (row, indptr_)."""
    cnt = th.zeros(n_rows, dtype=th.int64, device=row.device)
    ip = indptr_.to(th.int64)
    cnt.index_add_(0, row.to(th.int64), ip[1:] - ip[:-1])
    out = th.zeros(n_rows + 1, dtype=th.int64, device=row.device)
    th.cumsum(cnt, 0, out=out[1:])
    return out + int(ip[0]) if ip.numel() else out


def hashed_uniform(ids, cols, seed):
    """(len(ids), cols) float32 in (0, 1), a pure function of (id, column, seed): any rank can reproduce any
    row of a sharded tensor without holding it (a 32-bit integer mixer over int64 torch ops)."""
    c = th.arange(cols, device=ids.device, dtype=th.int64).view(1, -1)
    x = (ids.to(th.int64).view(-1, 1) * 2654435761 + c * 40503 + (seed * 7919 + 12345)) & 0xFFFFFFFF
    for _ in range(2):
        x = ((x ^ (x >> 16)) * 0x45D9F3B) & 0xFFFFFFFF
    x = x ^ (x >> 16)
    return (x.to(th.float32) + 0.5) * (1.0 / 4294967296.0)


def hashed_normal(ids, cols, seed, chunk=1 << 20):
    """(len(ids), cols) float32 ~ N(0, 1) by Box-Muller over two hashed uniforms; rows computed in chunks."""
    out = th.empty(ids.numel(), cols, dtype=th.float32, device=ids.device)
    for lo in range(0, ids.numel(), chunk):
        part = ids[lo:lo + chunk]
        u1, u2 = hashed_uniform(part, cols, 2 * seed), hashed_uniform(part, cols, 2 * seed + 1)
        out[lo:lo + chunk] = th.sqrt(-2.0 * th.log(u1)) * th.cos(6.283185307179586 * u2)
    return out


class ShardedSpmmWorkload:
    """vector_spmm forward + backward over a graph row-partitioned across the ranks (sharding.py).
    Every rank generates the same seeded graph and keeps its own shard."""
    name = "vector_spmm forward + backward, destination rows sharded over the ranks"
    resident = "graph shard and this rank's edge weights; e2e copies this rank's x shard and dy rows in, y rows " \
               "and dx rows out; the weights of the transposed shard's edges are exchanged every step"
    scaling = "strong"

    def __init__(self, spec, rank, dev, world):
        from custom_op_benchmark_b200 import sharding
        self.spec, self.dev, self.world, self.rank = spec, dev, world, rank
        self.h, self.d, self.dtype = spec["heads"], spec["dim"], DTYPES[spec["dtype"]]
        g = make_graph(spec, seed=0, device=dev)          # the same graph on every rank
        self.e, self.n_dst, self.n_src = g.n_edges, g.n_dst, g.n_src
        self.sh = sh = sharding.shard_graph(g, rank, world, chunk_size=32)
        # world > 1: fetch only the node rows this shard's edges reference (built once per graph)
        mode = spec.get("exchange", "needed")
        self.ex = sharding.plan_shard_exchange(sh) if (world > 1 and mode in ("needed", "peer")) else None
        self.peer = world > 1 and mode == "peer"
        del g
        th.cuda.empty_cache()
        # every input is a pure function of its global id (edge id, source node, destination node), so that any
        # rank can rebuild the rows it needs for checking; a rank holds only its own rows and its own edges' weights
        ar = lambda lo, n: th.arange(lo, lo + n, device=dev, dtype=th.int64)
        self.w_local = hashed_uniform(ar(sh.edge_lo, sh.indices.numel()), 1, 7).view(-1)
        xb = sharding.even_bounds(self.n_src, world)
        rows_x = int(xb[rank + 1] - xb[rank])
        self.x_shard = hashed_normal(ar(int(xb[rank]), rows_x), self.d, 11)
        self.dy_local = hashed_normal(ar(int(sh.dst_bounds[rank]), sh.rows), self.d, 13)
        self.host = [_pinned(self.x_shard.cpu()), _pinned(self.dy_local.cpu())]
        self.outs = [_pinned(th.empty(sh.rows, self.d)), _pinned(th.empty(sh.cols, self.d))]
        self.peer_note = None
        if self.peer:
            # the two row-sharded inputs live in symmetric memory: every rank pulls the rows it references out of the
            # owners' blocks with one kernel (plain peer loads over NVLink), no collective in the data path
            try:
                self.px = sharding.PeerRows(rows_x, (self.d,), th.float32, dev)
                self.pdy = sharding.PeerRows(sh.rows, (self.d,), th.float32, dev)
                ok = th.ones(1, device=dev)
            except Exception as exc:       # no peer mapping on this machine: the all-to-all of packed rows instead
                self.peer_note = "symmetric memory unavailable (%s): all-to-all used" % str(exc)[:100]
                ok = th.zeros(1, device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)      # the ranks agree on one path
            self.peer = bool(ok.item() > 0)
            if self.peer:
                self.px.local.copy_(self.x_shard)
                self.pdy.local.copy_(self.dy_local)
                self.px.barrier()
                self.pdy.barrier()
        s, i = 4, 4
        e_loc, e_t = sh.indices.numel(), sh.eid_t.numel()
        F = lambda n: n * self.h * self.d * s
        # per rank: gathered source rows read once, owned rows written once, weights, indices
        self.alg = {"aggregate": F(self.n_src) + F(sh.rows) + e_loc * s + (e_loc + sh.rows + 1) * i,
                    "edge_dot": F(self.n_src) + F(sh.rows) + e_loc * s + (e_loc + sh.rows + 1) * i}
        self.alg_step = (F(self.n_src) + F(sh.rows) + e_loc * s + (e_loc + sh.rows + 1) * i) + \
                        (F(self.n_src) + F(self.n_dst) + F(sh.rows) + F(sh.cols) + 2 * e_loc * s + e_t * s +
                         (e_loc + e_t + sh.rows + sh.cols + 2) * i + e_t * i)

    def units(self):
        return float(self.sh.indices.numel()) * self.h   # this rank's edges: the sum over ranks is E * H

    def forward(self):
        from custom_op_benchmark_b200 import sharding
        if self.peer:
            self.px.barrier()       # every block is in place before anyone pulls (a training step writes x each time)
            self.y, self.x_all = sharding.sharded_spmm_forward(self.sh, self.w_local, self.px, exchange=self.ex)
            return
        self.y, self.x_all = sharding.sharded_spmm_forward(self.sh, self.w_local, self.x_shard, exchange=self.ex)

    def backward(self):
        from custom_op_benchmark_b200 import sharding
        if self.peer:
            self.pdy.barrier()
            return sharding.sharded_spmm_backward(self.sh, self.w_local, self.pdy, self.x_all, exchange=self.ex)
        return sharding.sharded_spmm_backward(self.sh, self.w_local, self.dy_local, self.x_all, exchange=self.ex)

    def e2e_compute(self, stage):
        from custom_op_benchmark_b200 import sharding
        if self.peer:
            self.px.barrier()       # nobody is still pulling from the blocks about to be overwritten
            self.px.local.copy_(stage[0])
            self.pdy.local.copy_(stage[1])
            self.px.barrier()
            y, x_all = sharding.sharded_spmm_forward(self.sh, self.w_local, self.px, exchange=self.ex)
            _, dx = sharding.sharded_spmm_backward(self.sh, self.w_local, self.pdy, x_all, exchange=self.ex)
            return [y, dx]
        y, x_all = sharding.sharded_spmm_forward(self.sh, self.w_local, stage[0], exchange=self.ex)
        _, dx = sharding.sharded_spmm_backward(self.sh, self.w_local, stage[1], x_all, exchange=self.ex)
        return [y, dx]

    def e2e_bytes(self):
        return _nbytes(self.host), _nbytes(self.outs)

    def max_err(self, count=4000):
        """Sampled rows of this rank's y, dedata and dx against a float64 reference built from the hashed inputs
        (any row of x, dy or w is recomputed from its global id, so the exchanges are checked too)."""
        from oracle import edge_list_f64 as ref
        from custom_op_benchmark_b200 import sharding
        sh, dev, d = self.sh, self.dev, self.d
        self.forward()
        dedata, dx = self.backward()
        errs = {}
        # y and dedata: sampled local destination rows, their edges' global sources
        ip = sharding_local_indptr(sh.row, sh.indptr, sh.rows)
        rows = ref.pick_rows(ip, count=count)
        pos, local = ref.edges_of_rows(ip, rows)
        src = sh.indices.index_select(0, pos).to(th.int64)
        uniq, inv = th.unique(src, return_inverse=True)
        x_rows = hashed_normal(uniq, d, 11).to(th.float64)
        w = hashed_uniform(pos + sh.edge_lo, 1, 7).view(-1).to(th.float64)
        want_y = th.zeros(rows.numel(), d, dtype=th.float64, device=dev)
        for lo in range(0, pos.numel(), 1 << 20):
            sl = slice(lo, lo + (1 << 20))
            want_y.index_add_(0, local[sl], w[sl].view(-1, 1) * x_rows.index_select(0, inv[sl]))
        errs["y"] = ref.max_err(self.y.index_select(0, rows), want_y)[0]
        dy_rows = hashed_normal(rows + int(sh.dst_bounds[sh.rank]), d, 13).to(th.float64)
        want_dw = th.empty(pos.numel(), dtype=th.float64, device=dev)
        for lo in range(0, pos.numel(), 1 << 20):
            sl = slice(lo, lo + (1 << 20))
            want_dw[sl] = (dy_rows.index_select(0, local[sl]) * x_rows.index_select(0, inv[sl])).sum(-1)
        errs["dedata"] = ref.max_err(dedata.view(-1).index_select(0, pos), want_dw)[0]
        # dx: sampled owned source rows of the transposed shard, weights by global edge id, dy by global node id
        ipt = sharding_local_indptr(sh.col, sh.indptr_t, sh.cols)
        cols = ref.pick_rows(ipt, count=count, seed=1)
        pos, local = ref.edges_of_rows(ipt, cols)
        dst = sh.indices_t.index_select(0, pos).to(th.int64)
        uniq, inv = th.unique(dst, return_inverse=True)
        g_rows = hashed_normal(uniq, d, 13).to(th.float64)
        w = hashed_uniform(sh.eid_t.index_select(0, pos).to(th.int64), 1, 7).view(-1).to(th.float64)
        want_dx = th.zeros(cols.numel(), d, dtype=th.float64, device=dev)
        for lo in range(0, pos.numel(), 1 << 20):
            sl = slice(lo, lo + (1 << 20))
            want_dx.index_add_(0, local[sl], w[sl].view(-1, 1) * g_rows.index_select(0, inv[sl]))
        errs["dx"] = ref.max_err(dx.index_select(0, cols), want_dx)[0]
        return dict(errs, max_err=max(errs.values()),
                    what="%d sampled rows of y (and their edges' dedata) and of dx per rank, incl. the 32 longest rows, "
                         "empty rows and the last row, float64 reference rebuilt from the inputs' generating function, "
                         "|x - ref| / (1 + |ref|)" % count)

    def collectives(self, reps=3):
        """Milliseconds of the two exchanges of one step, each timed alone on this rank (all ranks call this
        together), and the bytes every rank receives from its peers per step."""
        from custom_op_benchmark_b200 import sharding
        if self.world == 1:
            return None
        xb = sharding.even_bounds(self.n_src, self.world)
        if self.peer:
            legs = (("x", lambda: self.px.pull(self.ex.x)), ("dy", lambda: self.pdy.pull(self.ex.dy)))
        elif self.ex is not None:
            from custom_op_benchmark_b200 import graphop
            legs = (("x", lambda: sharding.exchange_rows(self.x_shard, self.ex.x, gather=graphop.gather_rows)),
                    ("dy", lambda: sharding.exchange_rows(self.dy_local, self.ex.dy, gather=graphop.gather_rows)))
        else:
            legs = (("x", lambda: sharding.all_gather_rows(self.x_shard, xb)),
                    ("dy", lambda: sharding.all_gather_rows(self.dy_local, self.sh.dst_bounds)))
        out = {"kind": "referenced rows pulled from the peers' memory by one kernel per rank" if self.peer else
               ("all-to-all of the referenced rows" if self.ex is not None else "all-gather of every row")}
        if self.peer_note:
            out["note_peer"] = self.peer_note
        for name, leg in legs:
            leg()
            th.cuda.synchronize()
            a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                leg()
            b.record()
            th.cuda.synchronize()
            out[name + "_ms"] = a.elapsed_time(b) / reps
        row = self.d * 4
        if self.ex is not None:
            rows = sum(self.ex.x.recv_counts) + sum(self.ex.dy.recv_counts)
            out["rows_referenced"] = {"x": self.ex.x.needed.numel(), "of": self.n_src,
                                      "dy": self.ex.dy.needed.numel(), "of_dst": self.n_dst}
        else:
            rows = (self.n_src - self.x_shard.shape[0]) + (self.n_dst - self.sh.rows)
        out["bytes_received_per_step"] = rows * row
        return out


class HaloAttentionWorkload:
    """Fused attention forward + backward over ONE banded graph cut by rows over the ranks (halo.py): every step
    exchanges the K / V halo rows forward and the dK / dV halo rows backward."""
    name = "fused attention forward + backward, one banded graph cut by rows over the ranks, K / V halo exchanged"
    resident = "graph shard and its plans; e2e copies this rank's Q, K, V, dO rows in and O, dQ, dK, dV rows out"
    scaling = "strong"

    def __init__(self, spec, rank, dev, world):
        from custom_op_benchmark_b200 import halo
        self.spec, self.dev, self.world, self.rank = spec, dev, world, rank
        self.h, self.d, self.dtype = spec["heads"], spec["dim"], DTYPES[spec["dtype"]]
        g = make_graph(spec, seed=0, device=dev)          # the same graph on every rank
        self.g, self.e, self.n_dst, self.n_src = g, g.n_edges, g.n_dst, g.n_src
        self.sh = sh = halo.shard_band(g.indptr, g.indices, rank, world)
        self.plan_r, self.plan_t = halo._plans(sh)
        self.scale = self.d ** -0.5
        # inputs are functions of the global node id, so any rank can rebuild any row for checking
        ids = th.arange(sh.lo, sh.hi, device=dev, dtype=th.int64)
        hd = self.h * self.d
        mk = lambda seed: hashed_normal(ids, hd, seed).view(-1, self.h, self.d).to(self.dtype)
        self.Q, self.K, self.V, self.dO = mk(21), mk(22), mk(23), mk(24)
        self.host = [_pinned(t.cpu()) for t in (self.Q, self.K, self.V, self.dO)]
        self.outs = [_pinned(th.empty_like(t, device="cpu")) for t in (self.Q, self.Q, self.K, self.V)]
        s = 2
        F = lambda n: n * hd * s
        rows, win = sh.rows, sh.window_rows
        self.alg = {
            "attention_fwd_banded": 2 * F(rows) + 2 * F(win) + 2 * rows * 4 + rows * self.h * 4,
            "attention_bwd_dst_banded": 4 * F(rows) + 2 * F(win) + 2 * rows * 4 + 3 * rows * self.h * 4,
            "attention_bwd_src_banded": 4 * F(win) + 2 * F(rows) + 2 * win * 4 + 2 * rows * self.h * 4,
        }
        self.alg_step = 6 * F(rows) + 6 * F(win)

    def units(self):
        return float(self.sh.indices.numel()) * self.h    # this rank's edges: the sum over ranks is E * H

    def forward(self):
        from custom_op_benchmark_b200 import halo
        self.o, self.lse, self.saved = halo.band_attention_forward(self.sh, self.Q, self.K, self.V, self.scale)

    def backward(self):
        from custom_op_benchmark_b200 import halo
        return halo.band_attention_backward(self.sh, self.Q, self.saved, self.o, self.lse, self.dO, self.scale)

    def e2e_compute(self, stage):
        from custom_op_benchmark_b200 import halo
        q, k, v, g_o = stage
        o, lse, saved = halo.band_attention_forward(self.sh, q, k, v, self.scale)
        dq, dk, dv = halo.band_attention_backward(self.sh, q, saved, o, lse, g_o, self.scale)
        return [o, dq, dk, dv]

    def e2e_bytes(self):
        return _nbytes(self.host), _nbytes(self.outs)

    def max_err(self):
        """This rank's rows of O, lse, dQ, dK, dV against the float64 reference of the WHOLE layer, its inputs
        rebuilt from their generating function (so the exchanged halo rows and returned gradients are checked)."""
        from oracle import edge_list_f64 as ref
        self.forward()
        got = [self.o, self.lse] + list(self.backward())
        ids = th.arange(self.n_dst, device=self.dev, dtype=th.int64)
        hd = self.h * self.d
        mk = lambda seed: hashed_normal(ids, hd, seed).view(-1, self.h, self.d).to(self.dtype)
        want = ref.attention_f64(self.g.indptr, self.g.indices, mk(21), mk(22), mk(23), self.scale, mk(24))
        out = {}
        for name, a, b in zip(("o", "lse", "dq", "dk", "dv"), got, want):
            b = b[self.sh.lo:self.sh.hi]
            keep = th.isfinite(b)
            out[name] = ref.max_err(a[keep], b[keep])[0]
        return dict(out, max_err=max(out.values()),
                    what="every element of this rank's rows of O, lse, dQ, dK, dV against the float64 edge-list "
                         "reference of the whole layer, |x - ref| / (1 + |ref|)")

    def collectives(self, reps=5):
        from custom_op_benchmark_b200 import halo
        if self.world == 1:
            return None
        kv = th.cat([self.K, self.V], dim=-1)
        halo.halo_gather(self.sh, kv)
        th.cuda.synchronize()
        a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            halo.halo_gather(self.sh, kv)
        b.record()
        th.cuda.synchronize()
        row = 2 * self.h * self.d * 2
        return {"kind": "all-to-all of the halo rows (K and V in one message per neighbour), forward; the same rows of "
                        "dK and dV travel back in the backward",
                "halo_gather_ms": a.elapsed_time(b) / reps, "halo_rows": sum(self.sh.recv_counts),
                "bytes_received_per_step": 2 * sum(self.sh.recv_counts) * row}


WORKLOAD_CLASSES = {"attention": AttentionWorkload, "attention_bias": AttentionBiasWorkload, "gat": GatWorkload, "sddmm_softmax": SddmmSoftmaxWorkload,
                    "sharded_spmm": ShardedSpmmWorkload, "halo_attention": HaloAttentionWorkload}


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
def replay_from_graph(step, steps):
    """Milliseconds per step of `step()` captured once into a CUDA graph and replayed `steps` times, or
    {"error": ...} when the capture is refused."""
    try:
        side = th.cuda.Stream()
        side.wait_stream(th.cuda.current_stream())
        with th.cuda.stream(side):
            for _ in range(3):
                step()
        th.cuda.current_stream().wait_stream(side)
        th.cuda.synchronize()
        graph = th.cuda.CUDAGraph()
        with th.cuda.graph(graph):
            keep = step()
        for _ in range(3):
            graph.replay()
        th.cuda.synchronize()
        a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            graph.replay()
        b.record()
        th.cuda.synchronize()
        del keep
        return a.elapsed_time(b) / steps
    except Exception as exc:  # a capture that the runtime refuses is reported, not fatal
        th.cuda.synchronize()
        return {"error": "%s: %s" % (type(exc).__name__, str(exc)[:200])}


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


def build_workload(args, spec, rank, dev, world):
    if args.scale and spec["kind"] == "rmat":
        spec["scale"] = args.scale
    if spec["ops"] == "sharded_spmm":
        spec["exchange"] = args.exchange
        return ShardedSpmmWorkload(spec, rank, dev, world)
    if spec["ops"] == "halo_attention":
        return HaloAttentionWorkload(spec, rank, dev, world)
    return WORKLOAD_CLASSES[spec["ops"]](spec, rank, dev)


def time_steps(wl, steps, world):
    """K steps with inputs resident, CUDA events on the launching stream, a barrier and a device
    synchronisation on both sides.  Returns (total ms, mean forward ms, mean backward ms, wall t0, wall t1)."""
    if world > 1:
        dist.barrier()
    th.cuda.synchronize()
    ev = [th.cuda.Event(enable_timing=True) for _ in range(2 * steps + 1)]
    t0 = time.time()
    ev[0].record()
    for i in range(steps):
        wl.forward()
        ev[2 * i + 1].record()
        wl.backward()
        ev[2 * i + 2].record()
    th.cuda.synchronize()
    t1 = time.time()
    if world > 1:
        dist.barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    fwd_ms = statistics.mean(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(steps))
    bwd_ms = statistics.mean(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(steps))
    return total_ms, fwd_ms, bwd_ms, t0, t1


class EndToEnd:
    """The step through the public API with host buffers: every step copies all of its inputs from pinned host
    memory to the device and all of its results back.  Three streams: the copies in, the compute (the stream the
    autograd Functions are called on) and the copies out, with two sets of device staging buffers, so that step
    i + 1's inputs travel while step i computes and step i - 1's results travel back (PCIe is full duplex).
    Nothing is skipped and nothing is reused between steps."""

    def __init__(self, wl, dev):
        self.wl = wl
        self.stage = [[th.empty(h.shape, dtype=h.dtype, device=dev) for h in wl.host] for _ in range(2)]
        self.s_in, self.s_out = th.cuda.Stream(dev), th.cuda.Stream(dev)
        self.free = [None, None]

    def run(self, steps):
        wl, cur = self.wl, th.cuda.current_stream()
        self.s_in.wait_stream(cur)
        for i in range(steps):
            b = i & 1
            with th.cuda.stream(self.s_in):
                if self.free[b] is not None:
                    self.s_in.wait_event(self.free[b])      # the step that last used these buffers is done
                for dst, src in zip(self.stage[b], wl.host):
                    dst.copy_(src, non_blocking=True)
                arrived = th.cuda.Event()
                arrived.record(self.s_in)
            cur.wait_event(arrived)
            outs = wl.e2e_compute(self.stage[b])
            done = th.cuda.Event()
            done.record(cur)
            self.free[b] = done
            for t in outs:
                t.record_stream(self.s_out)
            with th.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for dst, src in zip(wl.outs, outs):
                    dst.copy_(src, non_blocking=True)
            del outs
        cur.wait_stream(self.s_out)

    def time(self, steps, world):
        self.run(2)
        th.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
        a.record()
        self.run(steps)
        b.record()
        th.cuda.synchronize()
        return a.elapsed_time(b) / steps


def kernel_breakdown(wl, twin, prof_steps):
    """Per-kernel device time of the step replayed through the instrumented twin, and its launches per step."""
    def step_device():
        wl.forward()
        return wl.backward()
    with twin.routed():
        step_device()            # settle the allocator before timing
    th.cuda.synchronize()
    n0 = twin.launch_count()

    def profiled():
        for _ in range(prof_steps):   # results dropped at once: kept alive they would force fresh cudaMallocs
            step_device()
    recs = twin.profile(profiled, th.cuda.current_stream().cuda_stream)
    launches = (twin.launch_count() - n0) / prof_steps
    per_kernel = {}
    for name, ms in recs:
        per_kernel.setdefault(name, []).append(ms)
    return {k: {"launches_per_step": len(v) / prof_steps, "ms_per_step": sum(v) / prof_steps}
            for k, v in per_kernel.items()}, launches


def sharded_extra(args, rank, dev, world):
    """The one configuration that is cut over the GPUs (R-MAT scale 24 vector SpMM, rows sharded by destination,
    strong scaling), run beside the headline workload at every N so that a scaling run carries a curve with
    communication in its data path.  Returns a dict on rank 0, None elsewhere."""
    spec = dict(WORKLOADS["rmat24_spmm"])
    if args.sharded_scale:
        spec["scale"] = args.sharded_scale
    spec["exchange"] = args.exchange
    free_b, _ = th.cuda.mem_get_info(dev)
    need = (1 << spec["scale"]) * (spec["edge_factor"] * 40 + 128 * 4 * 5)      # graph build + node tensors, generous
    if free_b < need:
        return {"skipped": "needs about %.0f GB of device memory, %.0f GB free" % (need / 1e9, free_b / 1e9)} \
            if rank == 0 else None
    wl = ShardedSpmmWorkload(spec, rank, dev, world)
    steps = max(2, min(args.steps, 5))
    for _ in range(2):
        wl.forward()
        wl.backward()
    total_ms, fwd_ms, bwd_ms, _, _ = time_steps(wl, steps, world)
    coll = wl.collectives()
    err = wl.max_err()
    stats = th.tensor([total_ms, fwd_ms, bwd_ms, err["max_err"]], dtype=th.float64, device=dev)
    work = th.tensor([wl.units()], dtype=th.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    total_ms, fwd_ms, bwd_ms, worst = stats.tolist()
    out = None
    if rank == 0:
        ms = total_ms / steps
        out = {"workload": "rmat24_spmm" if spec["scale"] == 24 else "rmat%d_spmm" % spec["scale"],
               "ops": wl.name, "scaling": "strong", "n_gpus": world, "nodes": wl.n_dst, "edges": wl.e, "dim": wl.d,
               "steps": steps, "ms_per_step": ms, "forward_ms": fwd_ms, "backward_ms": bwd_ms,
               "value": work.item() / (ms * 1e-3), "unit": UNIT, "max_err": worst, "max_err_what": err["what"],
               "exchange": coll}
    del wl
    th.cuda.empty_cache()
    return out


def run_gpu(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"   # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=th.device("cuda", local))
    dev = th.device("cuda", local)
    th.cuda.set_device(dev)
    spec = dict(WORKLOADS[args.workload])
    wl = build_workload(args, spec, rank, dev, world)

    def step_device():
        wl.forward()
        return wl.backward()

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
        print(json.dumps({"lean": True, "workload": args.workload, "edges": wl.e, "nodes": wl.n_dst, "heads": wl.h,
                          "dim": wl.d, "ms_per_step": a.elapsed_time(b) / args.steps}))
        return
    twin = Twin()

    # -- timed region: K steps through the product library, inputs resident ---------------------
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)
    total_ms, fwd_ms, bwd_ms, t_wall0, t_wall1 = time_steps(wl, args.steps, world)
    if t_wall1 - t_wall0 < 0.6:   # a short timed region: keep the same load up until the sampler has a few rows
        t_end = time.time() + 0.7
        while time.time() < t_end:
            step_device()
        th.cuda.synchronize()
        t_wall1 = time.time()
    sampler.stop()
    clocks = sampler.summary(t_wall0, t_wall1)

    # -- the same steps through the chunk-table entry points (the reference's argument lists: no plan) ----------
    chunk_api = None
    if getattr(wl, "planned", False):
        wl.planned = False
        step_device()
        cms, cf, cb, _, _ = time_steps(wl, max(2, min(args.steps, 5)), world)
        wl.planned = True
        chunk_api = {"ms_per_step": cms / max(2, min(args.steps, 5)), "forward_ms": cf, "backward_ms": cb,
                     "what": "the same step through the entry points that take (row, indptr, eid, indices): the owner "
                             "table is rebuilt from the chunk table in every call"}

    # -- end to end: the autograd Functions a user calls, host buffers copied in and out every step
    e2e_ms = EndToEnd(wl, dev).time(max(3, min(args.steps, 6)), world)
    th.cuda.empty_cache()

    # -- per-kernel times and launch count of the same step, through the instrumented twin -------
    kernels, launches_per_step = kernel_breakdown(wl, twin, max(2, min(args.steps, 5)))

    # -- the same step replayed from a CUDA graph (what is left when launch latency is taken out) --
    graph_ms = None
    if args.cuda_graph and world == 1:
        graph_ms = replay_from_graph(step_device, args.steps)

    # -- the gathers alone, same index streams and tables (a floor for the walker kernels) ------
    floors = wl.gather_floor(twin) if rank == 0 and hasattr(wl, "gather_floor") else {}
    # -- the collectives of a sharded step, timed alone (per-kernel events count them with the kernel after them)
    coll = wl.collectives() if hasattr(wl, "collectives") else None

    # -- the timed step's results against the float64 edge-list reference, every rank its own (worst one reported);
    #    a sharded workload's check runs its step, collectives included, so every rank takes part
    err = None
    if not args.no_cpu_baseline:
        err = wl.max_err()
        if world > 1:
            worst = th.tensor([err["max_err"]], dtype=th.float64, device=dev)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            err = dict(err, max_err=worst.item(), over_ranks=world)

    # -- reduce over ranks ---------------------------------------------------------------------
    stats = th.tensor([total_ms, e2e_ms, fwd_ms, bwd_ms], dtype=th.float64, device=dev)
    work = th.tensor([wl.units()], dtype=th.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    total_ms, e2e_ms, fwd_ms, bwd_ms = stats.tolist()
    units = work.item()  # edges*heads of all ranks, per step

    out = None
    if rank == 0:
        alg = wl.alg
        top = max((k for k in kernels if k in alg), key=lambda k: kernels[k]["ms_per_step"])
        top_ms = kernels[top]["ms_per_step"] / max(1.0, kernels[top]["launches_per_step"])
        peak, peak_kind = measured_peak()
        achieved = alg[top] / (top_ms * 1e-3) / 1e9
        ms_per_step = total_ms / args.steps
        h2d, d2h = wl.e2e_bytes()
        in_bytes = _nbytes(wl.host)
        out = {
            "metric": METRIC, "value": units / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": getattr(wl, "scaling", "weak"), "vs_baseline": None,
            "dtype": spec["dtype"], "data": "synthetic",
            "config": {"workload": args.workload, "ops": wl.name, "graph": describe(spec), "nodes": wl.n_dst,
                       "edges": wl.e, "heads": wl.h, "dim": wl.d,
                       "index": "int32 CSR, chunk tables of partition_csr(32)",
                       "per_rank": "a row shard of one graph" if spec["ops"] in ("sharded_spmm", "halo_attention") else "own graph",
                       "l2": "inputs (%.2f GB) %s the 126 MB L2" % (
                           in_bytes / 1e9, "larger than" if in_bytes > 2 * 126e6 else "NOT larger than"),
                       "resident": wl.resident,
                       "plans": ("graph plans built once per graph beside the chunk tables (%.1f ms for both CSR "
                                 "orientations), not per step" % wl.plan_build_ms) if getattr(wl, "planned", False)
                       else "none"},
            "e2e": {"value": units / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "pinned host buffers, copies in / compute / copies out on three streams, two staging sets"},
            "gpu_launches": int(round(launches_per_step * args.steps)),
            "gpu_launches_per_step": launches_per_step,
            "clocks": clocks,
            "phases": {"forward_ms": fwd_ms, "backward_ms": bwd_ms},
            "roofline": {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_source": peak_kind, "algorithmic_bytes": alg[top],
                         "frac_of_spec_8000": achieved / 8000.0,
                         "ms": top_ms, "traffic": traffic_for(top, args.workload),
                         "gather_bytes": wl.gather_bytes(top) if hasattr(wl, "gather_bytes") else None,
                         "step_algorithmic_bytes": wl.alg_step,
                         "step_frac": wl.alg_step / (ms_per_step * 1e-3) / 1e9 / peak},
            "kernels": kernels,
        }
        traffic_step = sum(traffic_for(k, args.workload) or 0 for k in kernels)
        if traffic_step:
            out["roofline"]["step_dram_traffic"] = traffic_step
            out["roofline"]["step_dram_frac"] = traffic_step / (ms_per_step * 1e-3) / 1e9 / peak
        if chunk_api:
            out["chunk_table_api"] = chunk_api
        if graph_ms is not None:
            out["cuda_graph"] = graph_ms if isinstance(graph_ms, dict) else {
                "ms_per_step": graph_ms, "value": units / (graph_ms * 1e-3), "unit": UNIT,
                "note": "one forward + backward captured with torch.cuda.graph and replayed; same kernels, no host "
                        "launch latency"}
        if coll:
            out["exchange"] = dict(coll, note="the exchanges of the sharded step timed alone on rank 0; inside the "
                                              "step the per-kernel events charge them to the kernel that follows, "
                                              "and the dy exchange overlaps the dedata kernel")
        if floors:
            out["gather_floor"] = {
                "what": "graphop_bench_gather_probe_i32: one row per edge per operand read through the kernel's own "
                        "index stream, nothing done with the rows",
                "ms": floors,
                "kernel_over_floor": {k: kernels[k]["ms_per_step"] / max(1.0, kernels[k]["launches_per_step"]) / v
                                      for k, v in floors.items() if k in kernels}}
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline(spec, args.cpu_sample_scale)
        if err is not None:
            out["max_err"] = err
    # -- the sharded configuration beside the headline one (strong scaling, communication in the data path)
    if args.sharded != "off" and spec["ops"] not in ("sharded_spmm", "halo_attention"):
        del wl
        th.cuda.empty_cache()
        extra = sharded_extra(args, rank, dev, world)
        if rank == 0:
            out["sharded"] = extra
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# the CPU baseline and the reference arm
# --------------------------------------------------------------------------------------------
def cpu_baseline(spec, sample_scale):
    """The torch CPU port of the workload's ops (oracle/cpu_baseline.py) timed on a bounded sample."""
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
    ops = spec["ops"] if spec["ops"] in ("gat", "sddmm_softmax", "attention_bias") else "attention"
    sec = cb.time_workload(ops, g, h, d)
    return {"value": g.n_edges * h / sec, "unit": UNIT, "cores": th.get_num_threads(), "host_cpus": os.cpu_count(),
            "kind": "port", "seconds": sec,
            "sample": sample + "; torch CPU fp32, forward + backward through autograd"}


def reference_cuda(spec, graph, steps=3):
    """The reference's own CUDA extension (oracle/_ref, built unmodified from graphop/graphop.cpp and
    graphop/graphop_kernel.cu) timed on this box's GPU: the same ops on the same graph, int64 chunk tables of
    partition_csr(32) as its contract wants, CUDA events, one untimed step first.  Sizes are limited to what its
    32-bit index arithmetic allows (graphop_kernel.cu:49, 144: (h * d) * n must stay below 2^31)."""
    if not th.cuda.is_available():
        return {"unavailable": "no CUDA device"}
    try:
        from oracle.build_reference import load_reference
        ref = load_reference()
    except Exception as exc:  # a build made for another torch
        return {"unavailable": "oracle/_ref does not load: %s" % str(exc)[:120]}
    if ref is None:
        return {"unavailable": "oracle/_ref holds no build of the reference"}
    from custom_op_benchmark_b200.part_csr import partition_csr
    h, d, ops = spec["heads"], spec["dim"], spec["ops"]
    if ops not in ("attention", "attention_bias", "gat", "sddmm_softmax"):
        return {"unavailable": "not run on this workload"}
    if spec["dtype"] != "f32":
        return {"unavailable": "the reference has no %s kernels (AT_DISPATCH_FLOATING_TYPES)" % spec["dtype"]}
    dev = th.device("cuda", 0)
    g = graph.to(device=dev, dtype=th.int64)
    n, m, e = g.n_dst, g.n_src, g.n_edges
    if h * d * max(n, m) >= 2 ** 31 or n != m:
        return {"unavailable": "(h * d) * n overflows the reference's int arithmetic at this size"}
    row, ptr = partition_csr(g.indptr, 32)
    col, ptr_t = partition_csr(g.indptr_t, 32)
    R, C = [row, ptr, g.eid, g.indices], [col, ptr_t, g.eid_t, g.indices_t]
    gen = th.Generator(device=dev).manual_seed(1)
    rn = lambda *s: th.randn(*s, generator=gen, device=dev)
    times = {}

    def timed(name, fn):
        a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
        a.record()
        out = fn()
        b.record()
        times.setdefault(name, []).append((a, b))
        return out

    if ops == "attention":
        Q, K, V, dO, scale = rn(n, h, d), rn(m, h, d), rn(m, h, d), rn(n, h, d), d ** -0.5

        def step():
            s = timed("maskedmm_fwd", lambda: ref.maskedmm_csr_forward(*R, Q, K))
            p = timed("softmax_fwd", lambda: ref.sparse_softmax_forward(*R[:3], s * scale))
            timed("spmm_fwd", lambda: ref.vector_spmm_forward(*R, p, V))
            dp, _ = timed("spmm_bwd", lambda: ref.vector_spmm_backward(*R, *C, p, dO, V))
            ds = timed("softmax_bwd", lambda: ref.sparse_softmax_backward(*R[:3], p, dp))
            timed("maskedmm_bwd", lambda: ref.maskedmm_csr_backward(*R, *C, Q, K, ds * scale))
    elif ops == "attention_bias":
        Q, K, V, dO, scale = rn(n, h, d), rn(m, h, d), rn(m, h, d), rn(n, h, d), d ** -0.5
        rel = rn(e, d) * 0.5

        def step():     # the layer as the reference's ops compose it: two score tensors, then the chain
            s = timed("maskedmm_fwd", lambda: ref.maskedmm_csr_forward(*R, Q, K))
            b = timed("node_mul_edge_fwd", lambda: ref.node_mul_edge_forward(*R[:3], Q, rel))
            p = timed("softmax_fwd", lambda: ref.sparse_softmax_forward(*R[:3], (s + b) * scale))
            timed("spmm_fwd", lambda: ref.vector_spmm_forward(*R, p, V))
            dp, _ = timed("spmm_bwd", lambda: ref.vector_spmm_backward(*R, *C, p, dO, V))
            ds = timed("softmax_bwd", lambda: ref.sparse_softmax_backward(*R[:3], p, dp)) * scale
            timed("maskedmm_bwd", lambda: ref.maskedmm_csr_backward(*R, *C, Q, K, ds))
            timed("node_mul_edge_bwd", lambda: ref.node_mul_edge_backward(*R[:3], Q, rel, ds))
    elif ops == "gat":
        X, Be, w, dY1, dY2 = rn(n, h, d), rn(e, d), th.rand(e, h, generator=gen, device=dev), rn(e, h), rn(n, h, d)

        def step():
            timed("node_mul_edge_fwd", lambda: ref.node_mul_edge_forward(*R[:3], X, Be))
            timed("spmm_fwd", lambda: ref.vector_spmm_forward(*R, w, X))
            timed("node_mul_edge_bwd", lambda: ref.node_mul_edge_backward(*R[:3], X, Be, dY1))
            timed("spmm_bwd", lambda: ref.vector_spmm_backward(*R, *C, w, dY2, X))
    else:
        Q, K, dP = rn(n, h, d) * 3, rn(m, h, d) * 3, rn(e, h)

        def step():
            s = timed("maskedmm_fwd", lambda: ref.maskedmm_csr_forward(*R, Q, K))
            p = timed("softmax_fwd", lambda: ref.sparse_softmax_forward(*R[:3], s))
            ds = timed("softmax_bwd", lambda: ref.sparse_softmax_backward(*R[:3], p, dP))
            timed("maskedmm_bwd", lambda: ref.maskedmm_csr_backward(*R, *C, Q, K, ds))
    step()
    th.cuda.synchronize()
    times.clear()
    a, b = th.cuda.Event(enable_timing=True), th.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    th.cuda.synchronize()
    ms = a.elapsed_time(b) / steps
    per_op = {k: sum(x.elapsed_time(y) for x, y in v) / len(v) for k, v in times.items()}
    return {"ms_per_step": ms, "value": e * h / (ms * 1e-3), "unit": UNIT, "steps": steps, "per_op_ms": per_op,
            "what": "the reference's CUDA ops, compiled unmodified for sm_100a, on the same graph (int64 chunk "
                    "tables, chunk_size 32), forward + backward, CUDA events",
            "note": "its dx kernel is launched with the row CSR's chunk count (graphop_kernel.cu:566, 588): on a graph "
                    "whose transposed CSR has more chunks it leaves the last ones out, so its time is a lower bound"}


def run_reference(args):
    """Reference arm.  The reference is a CUDA-only extension with no CPU implementation of its own, so `value`
    times the torch CPU restatement of its chain on all host cores, on the workload's own graph (the same
    generator and seed as rank 0 of the GPU arm).  Beside it, under `reference_cuda`, the reference's own CUDA ops
    are timed on this box's GPU."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    th.set_num_threads(cores)     # torch.distributed.run exports OMP_NUM_THREADS=1: use every host core anyway
    from oracle import cpu_baseline as cb
    spec = dict(WORKLOADS[args.workload])
    if args.scale and spec["kind"] == "rmat":
        spec["scale"] = args.scale
    world = int(os.environ.get("WORLD_SIZE", "1"))
    h, d = spec["heads"], spec["dim"]
    note = "the reference has no CPU code path; this is the torch CPU restatement of its chain, all host cores"
    if spec["ops"] == "sharded_spmm":
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one device and its index "
                          "arithmetic overflows at R-MAT scale 24 (graphop_kernel.cu:49, 144)"}))
        return
    t0 = time.time()
    g = make_graph(spec, seed=0, device="cuda" if th.cuda.is_available() else "cpu").to(device="cpu")
    ops = "attention" if spec["ops"] == "halo_attention" else spec["ops"]   # the host cores see one whole graph
    secs = []
    budget_s = 150.0
    planned = max(1, args.steps)
    for k in range(1 + planned):               # one untimed step first
        t = cb.time_workload(ops, g, h, d)
        if k:
            secs.append(t)
        if time.time() - t0 + t > budget_s and secs:
            break
    sec = statistics.mean(secs)
    value = g.n_edges * h / sec
    base = {"value": value, "unit": UNIT, "cores": th.get_num_threads(), "host_cpus": cores, "kind": "port",
            "seconds": sec, "sample": "the whole workload graph, %d steps of the %d asked for (bounded to ~%d s of "
                                      "CPU work); torch CPU fp32, forward + backward through autograd" % (
                                          len(secs), planned, int(budget_s))}
    out = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
           "steps": len(secs), "warmup": 1, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": spec["dtype"], "data": "synthetic",
           "config": {"workload": args.workload, "ops": WORKLOAD_CLASSES[ops].name, "graph": describe(spec),
                      "nodes": g.n_dst, "edges": g.n_edges, "heads": h, "dim": d,
                      "index": "int32 CSR, chunk tables of partition_csr(32)", "note": note},
           "cpu_baseline": base,
           "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    if world == 1 or rank == 0:
        out["reference_cuda"] = reference_cuda(spec, g)
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="graphop_b200", choices=["graphop_b200", "reference"])
    ap.add_argument("--workload", default="rmat21_attention", choices=sorted(WORKLOADS))
    ap.add_argument("--scale", type=int, default=0, help="override the R-MAT scale (smaller runs)")
    ap.add_argument("--cpu-sample-scale", type=int, default=19)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="peer", choices=["needed", "all", "peer"],
                    help="sharded workload: fetch only the node rows a shard references (all-to-all), all-gather every "
                         "row, or pull the referenced rows out of the peers' memory with a kernel (symmetric memory)")
    ap.add_argument("--sharded", default="auto", choices=["auto", "off"],
                    help="also run the row-sharded R-MAT scale-24 SpMM at this GPU count and attach it as `sharded`")
    ap.add_argument("--sharded-scale", type=int, default=0, help="override the R-MAT scale of the sharded extra")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="also replay the step from a CUDA graph and report it (1 GPU)")
    ap.add_argument("--lean", action="store_true",
                    help="warm-up and timed steps only (for ncu captures); prints a reduced line")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
