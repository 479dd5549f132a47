"""Graph plans: the planned ops agree with the chunk-table ops (per-edge outputs and the softmax to the bit; row
reductions to rounding, because a plan's work tiles end on row starts), the shape analysis finds dense bands, and a
dense-band graph's bfloat16 attention (tensor-core kernels) matches the float64 reference."""
import pytest
import torch as th

from helpers import assert_close, chunked, graph_zoo
from custom_op_benchmark_b200 import graphop, graphs, wrapper
from oracle import edge_list_f64 as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ZOO = graph_zoo()


def _plans(g, cs, idt):
    r, c = chunked(g, cs, dtype=idt), chunked(g, cs, transposed=True, dtype=idt)
    rc, cc = [t.to(DEV) for t in r], [t.to(DEV) for t in c]
    return rc, cc, graphop.GraphPlan(*rc, g.n_dst), graphop.GraphPlan(*cc, g.n_src)


@pytest.mark.parametrize("name,g", ZOO, ids=[z[0] for z in ZOO])
@pytest.mark.parametrize("cs,idt", [(32, th.int32), (7, th.int64), (None, th.int32)])
def test_planned_ops_equal_chunk_table_ops(name, g, cs, idt):
    rc, cc, pr, pt = _plans(g, cs, idt)
    h, d, e = 4, 32, g.n_edges
    gen = th.Generator(device=DEV).manual_seed(11)
    rn = lambda *s: th.randn(*s, generator=gen, device=DEV)
    A, B, dY = rn(g.n_dst, h, d), rn(g.n_src, h, d), rn(g.n_dst, h, d)
    w, ds, Be = th.rand(e, h, generator=gen, device=DEV), rn(e, h), rn(e, d)
    def same_sums(a, b, what):   # the same terms, added row by row instead of tile piece by tile piece
        assert_close(a, b, 2e-5, 2e-5 * max(1.0, float(b.abs().max())), what)

    assert th.equal(graphop.maskedmm_csr_forward_planned(pr, A, B), graphop.maskedmm_csr_forward(*rc, A, B))
    for a, b in zip(graphop.maskedmm_csr_backward_planned(pr, pt, A, B, ds),
                    graphop.maskedmm_csr_backward(*rc, *cc, A, B, ds)):
        same_sums(a, b, "maskedmm backward")
    same_sums(graphop.vector_spmm_forward_planned(pr, w, B, num_dst=g.n_dst),
              graphop.vector_spmm_forward(*rc, w, B, num_dst=g.n_dst), "spmm forward")
    if g.n_dst == g.n_src:
        got = graphop.vector_spmm_backward_planned(pr, pt, w, dY, B)
        want = graphop.vector_spmm_backward(*rc, *cc, w, dY, B)
        assert th.equal(got[0], want[0])
        same_sums(got[1], want[1], "spmm backward dx")
    p = graphop.sparse_softmax_forward_planned(pr, ds)
    assert th.equal(p, graphop.sparse_softmax_forward(*rc[:3], ds))
    assert th.equal(graphop.sparse_softmax_backward_planned(pr, p, w), graphop.sparse_softmax_backward(*rc[:3], p, w))
    assert th.equal(graphop.node_mul_edge_forward_planned(pr, A, Be), graphop.node_mul_edge_forward(*rc[:3], A, Be))
    got = graphop.node_mul_edge_backward_planned(pr, A, Be, ds)
    want = graphop.node_mul_edge_backward(*rc[:3], A, Be, ds)
    same_sums(got[0], want[0], "node_mul_edge backward dA")
    assert th.equal(got[1], want[1])
    o, lse = graphop.attention_forward_planned(pr, A, B, B * 0.5, 0.2)
    o2, lse2 = graphop.attention_forward(rc[0], rc[1], rc[3], A, B, B * 0.5, 0.2)
    has = th.isfinite(lse2)
    same_sums(o, o2, "attention o")
    assert th.equal(th.isfinite(lse), has)
    same_sums(lse[has], lse2[has], "attention lse")
    got = graphop.attention_backward_planned(pr, pt, A, B, B * 0.5, o2, lse2, dY, 0.2)
    want = graphop.attention_backward(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], A, B, B * 0.5, o2, lse2, dY, 0.2,
                                      eid_t=cc[2])
    for a, b, what in zip(got, want, ("dq", "dk", "dv")):
        same_sums(a, b, "attention " + what)
    # and twice the same answer
    again = graphop.attention_backward_planned(pr, pt, A, B, B * 0.5, o2, lse2, dY, 0.2)
    for a, b in zip(got, again):
        assert th.equal(a, b)


def test_row_aligned_tiles_need_no_carry_levels():
    """A graph whose rows are all shorter than a work tile: the plan says so, and the fused step is 3 launches."""
    g = graphs.er_graph(4096, 15, seed=0)
    rc, cc, pr, pt = _plans(g, 32, th.int32)
    assert pr.no_carry and pt.no_carry
    long_rows = ZOO[3][1]
    _, _, pl, _ = _plans(long_rows, 32, th.int32)
    assert not pl.no_carry


def test_planned_autograd_function():
    g = ZOO[3][1]
    rc, cc, pr, pt = _plans(g, 32, th.int32)
    gen = th.Generator(device=DEV).manual_seed(12)
    Q, dO = (th.randn(g.n_dst, 4, 32, generator=gen, device=DEV) for _ in range(2))
    K, V = (th.randn(g.n_src, 4, 32, generator=gen, device=DEV) for _ in range(2))
    q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
    wrapper.GraphAttentionPlanned.apply(pr, pt, q, k, v, 0.3).backward(dO)
    q2, k2, v2 = (t.clone().requires_grad_(True) for t in (Q, K, V))
    wrapper.GraphAttention.apply(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], q2, k2, v2, 0.3, cc[2]).backward(dO)
    for a, b in ((q, q2), (k, k2), (v, v2)):
        assert_close(a.grad, b.grad, 2e-5, 2e-5 * max(1.0, float(b.grad.abs().max())), "grad")


def test_shape_analysis_finds_dense_bands():
    band = graphs.banded_graph(2, 1024, 128)
    rc, _, pr, pt = _plans(band, 32, th.int32)
    assert pr.dense_band and pr.band_span == 128 + 2 * 128 and pt.dense_band
    blocks = graphs.block_diagonal_graph(16, 30, index_dtype=th.int32)
    _, _, pb, _ = _plans(blocks, None, th.int32)
    assert pb.dense_band and pb.band_span <= 180
    wide = graphs.banded_graph(1, 2048, 200)           # 128 rows reach 128 + 400 > 384 keys: a band, but too wide
    _, _, pw, _ = _plans(wide, 32, th.int32)
    assert not pw.dense_band and pw.band_span == 528
    er = graphs.er_graph(512, 6, seed=2)
    _, _, pe, _ = _plans(er, 32, th.int32)
    assert not pe.dense_band


def _band_with_gaps(n, window, seed):
    """A band whose rows have ragged widths and a few rows no edge at all."""
    gen = th.Generator().manual_seed(seed)
    i = th.arange(n)
    left = th.randint(0, window + 1, (n,), generator=gen)
    right = th.randint(0, window + 1, (n,), generator=gen)
    lo, hi = (i - left).clamp_(min=0), (i + right).clamp_(max=n - 1)
    deg = hi - lo + 1
    deg[th.rand(n, generator=gen) < 0.05] = 0
    dst = th.repeat_interleave(i, deg)
    start = th.cumsum(deg, 0) - deg
    src = th.arange(int(deg.sum())) - start[dst] + lo[dst]
    return graphs.coo_to_graph(dst, src, n)


@pytest.mark.parametrize("make,h", [
    (lambda: graphs.banded_graph(2, 1024, 128), 8),          # the benchmark's band, two short sequences
    (lambda: graphs.banded_graph(1, 1000, 17), 2),            # node count not a multiple of the 128-row tile
    (lambda: graphs.block_diagonal_graph(20, 30, index_dtype=th.int32), 8),   # the reference's own test graph
    (lambda: _band_with_gaps(777, 100, 3), 3),                # ragged widths, rows without edges
])
def test_dense_band_attention_forward_on_tensor_cores(make, h):
    g = make()
    rc, cc, pr, pt = _plans(g, 32, th.int32)
    assert pr.dense_band
    d, scale = 64, 0.125
    gen = th.Generator(device=DEV).manual_seed(13)
    Q, K, V = (th.randn(g.n_dst, h, d, generator=gen, device=DEV).to(th.bfloat16) for _ in range(3))
    o, lse = graphop.attention_forward_planned(pr, Q, K, V, scale)
    want_o, want_lse = ref.attention_f64(g.indptr.to(DEV), g.indices.to(DEV), Q, K, V, scale)
    deg = (g.indptr[1:] - g.indptr[:-1]).to(DEV)
    assert bool((lse[deg == 0] == -float("inf")).all()) and bool((o[deg == 0] == 0).all())
    assert_close(o, want_o, 2e-2, 2e-2, "o")
    assert_close(lse[deg > 0], want_lse[deg > 0], 1e-3, 2e-3, "lse")
    # and the walker's answer on the same graph (chunk-table entry point)
    o2, lse2 = graphop.attention_forward(rc[0], rc[1], rc[3], Q, K, V, scale)
    assert_close(o, o2.double(), 2e-2, 2e-2, "o vs walker")
    # the backward (walker kernels, through the plans) takes the tensor-core forward's O and lse
    dO = th.randn(g.n_dst, h, d, generator=gen, device=DEV).to(th.bfloat16)
    dq, dk, dv = graphop.attention_backward_planned(pr, pt, Q, K, V, o, lse, dO, scale)
    _, _, wq, wk, wv = ref.attention_f64(g.indptr.to(DEV), g.indices.to(DEV), Q, K, V, scale, dO)
    for got, want, what in ((dq, wq, "dq"), (dk, wk, "dk"), (dv, wv, "dv")):
        assert_close(got, want, 2e-2, 5e-2 * max(1.0, float(want.abs().max())), what)


def test_per_call_signature_runs_on_cached_plans():
    """wrapper.GraphAttention takes the graph tensors per call (the reference's convention); their plans are built
    once and found again, so a dense band in bfloat16 reaches the tensor-core kernels through that signature too."""
    g = graphs.banded_graph(1, 640, 64)
    rc, cc, pr, pt = _plans(g, 32, th.int32)
    gen = th.Generator(device=DEV).manual_seed(14)
    Q, K, V, dO = (th.randn(g.n_dst, 4, 64, generator=gen, device=DEV).to(th.bfloat16) for _ in range(4))
    graphop._PLAN_CACHE.clear()
    outs = []
    for _ in range(2):
        q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
        o = wrapper.GraphAttention.apply(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], q, k, v, 0.125, cc[2])
        o.backward(dO)
        outs.append((o.detach(), q.grad, k.grad, v.grad))
    assert len(graphop._PLAN_CACHE) == 2                       # one plan per orientation, built once
    assert all(p.dense_band for p in graphop._PLAN_CACHE.values())
    q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
    wrapper.GraphAttentionPlanned.apply(pr, pt, q, k, v, 0.125).backward(dO)
    for a, b, c in zip(outs[0][1:], outs[1][1:], (q.grad, k.grad, v.grad)):
        assert th.equal(a, b) and th.equal(a, c)
    # a graph tensor modified in place gets a new plan
    rc[3].add_(0)
    assert graphop.cached_plan(rc[0], rc[1], None, rc[3], g.n_dst) not in list(graphop._PLAN_CACHE.values())[:2]
    # and the cache can be switched off
    old, graphop.plan_cache_size = graphop.plan_cache_size, 0
    try:
        q2 = Q.clone().requires_grad_(True)
        o2 = wrapper.GraphAttention.apply(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], q2, K, V, 0.125, cc[2])
        assert_close(o2, outs[0][0].double(), 2e-2, 2e-2, "walker against tensor cores")
    finally:
        graphop.plan_cache_size = old


def test_plan_entry_points_report_bad_arguments():
    import ctypes
    from custom_op_benchmark_b200 import _capi
    lib = _capi.lib()
    g = ZOO[0][1]
    r = [t.to(DEV) for t in chunked(g, 32, dtype=th.int32)]
    need = lib.graphop_plan_bytes(r[0].numel(), g.n_edges, g.n_dst, 4)
    mem = th.empty(need + 256, dtype=th.uint8, device=DEV)
    base = (mem.data_ptr() + 255) // 256 * 256
    plan = _capi.Plan()
    args = [r[0].data_ptr(), r[1].data_ptr(), r[2].data_ptr(), r[3].data_ptr(), r[0].numel(), g.n_edges, g.n_dst]
    stream = th.cuda.current_stream().cuda_stream
    assert lib.graphop_plan_build_i32(*args, base, 64, ctypes.byref(plan), stream) == _capi.ERR_WORKSPACE
    assert lib.graphop_plan_build_i32(*args, base + 4, need, ctypes.byref(plan), stream) == _capi.ERR_WORKSPACE
    assert lib.graphop_plan_build_i32(*args, base, need, None, stream) == _capi.ERR_INVALID_ARGUMENT
    assert lib.graphop_plan_build_i32(*args[:4], -1, g.n_edges, g.n_dst, base, need, ctypes.byref(plan),
                                      stream) == _capi.ERR_INVALID_ARGUMENT
    assert lib.graphop_plan_build_i32(*args, base, need, ctypes.byref(plan), stream) == _capi.OK
    x = th.randn(g.n_edges, 2, device=DEV)
    y = th.empty_like(x)
    ws = th.empty(1 << 20, dtype=th.uint8, device=DEV)
    # a planned op without a plan
    assert lib.graphop_sparse_softmax_forward_planned_f32(None, x.data_ptr(), y.data_ptr(), 2, ws.data_ptr(), ws.numel(),
                                                          stream) == _capi.ERR_INVALID_ARGUMENT
    th.cuda.synchronize()
