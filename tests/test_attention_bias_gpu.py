"""The fused attention layer with an edge term in the scores (graphop_attention_bias_*): scores are
scale * q . (k + rel[edge]), i.e. the reference's maskedmm plus its node_mul_edge ("designed for relative positional
encoding", graphop_kernel.cu:16-34) before the softmax.  Checked against the float64 edge-list reference and against
the same layer composed from the unfused ops through autograd."""
import pytest
import torch as th

from helpers import assert_close, assert_rows_close, chunked, graph_zoo
from custom_op_benchmark_b200 import graphop, wrapper
from oracle import edge_list_f64 as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ZOO = [z for z in graph_zoo() if z[1].n_dst == z[1].n_src]
TOL = {th.float32: (2e-5, 2e-5), th.float64: (1e-11, 1e-11), th.bfloat16: (3e-2, 3e-2)}


def _inputs(g, h, d, dt, seed):
    gen = th.Generator(device=DEV).manual_seed(seed)
    rn = lambda *s: th.randn(*s, generator=gen, device=DEV).to(dt)
    return rn(g.n_dst, h, d), rn(g.n_src, h, d), rn(g.n_src, h, d), rn(g.n_edges, d) * 0.5, rn(g.n_dst, h, d)


@pytest.mark.parametrize("name,g", ZOO, ids=[z[0] for z in ZOO])
@pytest.mark.parametrize("dt,idt,h,d", [(th.float32, th.int32, 4, 32), (th.float32, th.int64, 1, 64),
                                        (th.float64, th.int64, 2, 16), (th.bfloat16, th.int32, 8, 64)])
def test_against_float64_reference(name, g, dt, idt, h, d):
    r = [t.to(DEV) for t in chunked(g, 32, dtype=idt)]
    c = [t.to(DEV) for t in chunked(g, 32, transposed=True, dtype=idt)]
    assert th.equal(r[2].long(), th.arange(g.n_edges, device=DEV))    # rel is indexed by row-CSR position
    Q, K, V, rel, dO = _inputs(g, h, d, dt, 41)
    scale = d ** -0.5
    o, lse = graphop.attention_bias_forward(r[0], r[1], r[3], Q, K, V, rel, scale)
    dq, dk, dv, dr = graphop.attention_bias_backward(r[0], r[1], r[3], c[0], c[1], c[2], c[3], Q, K, V, rel, o, lse,
                                                     dO, scale)
    wo, wl, wq, wk, wv, wr = ref.attention_f64(g.indptr.to(DEV), g.indices.to(DEV), Q, K, V, scale, dO, rel=rel)
    rt, at = TOL[dt]
    deg = (g.indptr[1:] - g.indptr[:-1])
    deg_t = (g.indptr_t[1:] - g.indptr_t[:-1])
    assert_close(o, wo, rt, at, "o")
    has = (deg > 0).to(DEV)
    assert_close(lse[has], wl[has], rt, at * 10, "lse")
    assert bool((lse[~has] == -float("inf")).all()) and bool((o[~has] == 0).all())
    mag = lambda w: max(1.0, float(w.abs().max()))
    assert_rows_close(dq, wq, deg, rt, 4 * at * mag(wq), "dq")
    assert_rows_close(dk, wk, deg_t, rt, 4 * at * mag(wk), "dk")
    assert_rows_close(dv, wv, deg_t, rt, 4 * at * mag(wv), "dv")
    assert_close(dr, wr, rt, 4 * at * mag(wr), "d_rel")


def test_against_the_layer_composed_from_the_unfused_ops():
    """MaskedMMCSR + NodeMulEdge -> scale -> SparseSoftmax -> VectorSPMM (the reference's ops, wrapper.py:8-55) through
    autograd gives the same output and gradients."""
    g = ZOO[3][1]
    r = [t.to(DEV) for t in chunked(g, 32)]
    c = [t.to(DEV) for t in chunked(g, 32, transposed=True)]
    h, d, scale = 4, 32, 0.2
    Q, K, V, rel, dO = _inputs(g, h, d, th.float32, 42)
    leaves = [t.clone().requires_grad_(True) for t in (Q, K, V, rel)]
    q, k, v, b = leaves
    s = (wrapper.MaskedMMCSR.apply(*r, *c, q, k) + wrapper.NodeMulEdge.apply(*r[:3], q, b)) * scale
    p = wrapper.SparseSoftmax.apply(*r[:3], s)
    wrapper.VectorSPMM.apply(*r, *c, p, v).backward(dO)
    fused = [t.clone().requires_grad_(True) for t in (Q, K, V, rel)]
    out = wrapper.GraphAttentionBias.apply(r[0], r[1], r[3], c[0], c[1], c[2], c[3], *fused, scale)
    out.backward(dO)
    for a, b_, what in zip(fused, leaves, ("dq", "dk", "dv", "d_rel")):
        assert_close(a.grad, b_.grad, 1e-4, 1e-4 * max(1.0, float(b_.grad.abs().max())), what)


def test_without_edges_and_bad_arguments():
    n, h, d = 5, 2, 16
    row = th.zeros(0, dtype=th.int32, device=DEV)
    ptr = th.zeros(1, dtype=th.int32, device=DEV)
    idx = th.zeros(0, dtype=th.int32, device=DEV)
    Q = th.randn(n, h, d, device=DEV)
    o, lse = graphop.attention_bias_forward(row, ptr, idx, Q, Q, Q, th.zeros(0, d, device=DEV), 1.0)
    assert bool((o == 0).all()) and bool((lse == -float("inf")).all())
    g = ZOO[0][1]
    r = [t.to(DEV) for t in chunked(g, 32, dtype=th.int32)]
    Q = th.randn(g.n_dst, h, d, device=DEV)
    with pytest.raises(RuntimeError, match="rel must be"):
        graphop.attention_bias_forward(r[0], r[1], r[3], Q, Q, Q, th.zeros(g.n_edges, d + 1, device=DEV), 1.0)


def test_backward_needs_the_transposed_edge_ids():
    from custom_op_benchmark_b200 import _capi
    lib = _capi.lib()
    g = ZOO[0][1]
    r = [t.to(DEV) for t in chunked(g, 32, dtype=th.int32)]
    c = [t.to(DEV) for t in chunked(g, 32, transposed=True, dtype=th.int32)]
    h, d = 2, 16
    Q, K, V, rel, dO = _inputs(g, h, d, th.float32, 43)
    o, lse = graphop.attention_bias_forward(r[0], r[1], r[3], Q, K, V, rel, 0.25)
    outs = [th.empty_like(t) for t in (Q, K, V, rel)]
    n = lib.graphop_workspace_bytes(_capi.OP_ATTENTION_BWD_PAIRS, g.n_edges, g.n_dst, h, d, 4, 4)
    ws = th.empty(n + 256, dtype=th.uint8, device=DEV)
    base = (ws.data_ptr() + 255) // 256 * 256
    p = lambda t: t.data_ptr()
    rc = lib.graphop_attention_bias_backward_f32_i32(
        p(r[0]), p(r[1]), p(r[3]), r[0].numel(), p(c[0]), p(c[1]), None, p(c[3]), c[0].numel(), p(Q), p(K), p(V), p(rel),
        p(o), p(lse), p(dO), 0.25, p(outs[0]), p(outs[1]), p(outs[2]), p(outs[3]), g.n_edges, g.n_dst, g.n_src, h, d, base,
        n, th.cuda.current_stream().cuda_stream)
    assert rc == _capi.ERR_INVALID_ARGUMENT
    th.cuda.synchronize()
