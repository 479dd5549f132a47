"""The fused attention kernels against the op-by-op oracle chain and the dense-masked
float64 attention, and the autograd wiring of every Function against torch autograd."""
import pytest
import torch as th

from helpers import assert_close, assert_rows_close, chunked, graph_zoo
from custom_op_benchmark_b200 import graphop, graphs, wrapper
from oracle import graphop_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ZOO = graph_zoo()
# relative / absolute tolerance on outputs of size O(1): fp32 as the specification states it (rel 1e-5 / abs 1e-6)
TOL = {th.float64: (1e-9, 1e-11), th.float32: (1e-5, 1e-6), th.bfloat16: (2e-2, 2e-2)}


def _qkv(g, h, d, dtype, seed, mag=1.0):
    gen = th.Generator().manual_seed(seed)
    mk = lambda n: (th.randn(n, h, d, generator=gen, dtype=th.float64) * mag).to(dtype)
    return mk(g.n_dst), mk(g.n_src), mk(g.n_src), mk(g.n_dst)


@pytest.mark.parametrize("name,g", ZOO, ids=[z[0] for z in ZOO])
@pytest.mark.parametrize("cs", [32, 11, None])
@pytest.mark.parametrize("h,d,dtype,idt,mag", [
    (4, 32, th.float32, th.int32, 1.0), (8, 64, th.float32, th.int64, 1.0), (4, 32, th.float64, th.int32, 3.0),
    (2, 64, th.float32, th.int32, 3.0), (1, 128, th.float32, th.int32, 1.0), (8, 64, th.bfloat16, th.int32, 1.0),
    (8, 64, th.float64, th.int64, 1.0), (1, 1024, th.float32, th.int32, 0.5), (16, 4, th.float32, th.int32, 1.0),
    # odd head counts: the packed (lse, delta) rows are padded to an even number of heads for fp32
    (3, 8, th.float32, th.int32, 1.0), (5, 16, th.float64, th.int32, 1.0), (3, 16, th.bfloat16, th.int32, 1.0),
])
def test_fused_attention_matches_oracle_chain(name, g, cs, h, d, dtype, idt, mag):
    r, c = chunked(g, cs, dtype=idt), chunked(g, cs, transposed=True, dtype=idt)
    Q, K, V, dO = _qkv(g, h, d, dtype, 1, mag)
    scale = d ** -0.5
    assert graphop.attention_supported(Q.to(DEV))
    rc, cc = [t.to(DEV) for t in r], [t.to(DEV) for t in c]
    o, lse = graphop.attention_forward(rc[0], rc[1], rc[3], Q.to(DEV), K.to(DEV), V.to(DEV), scale)
    want_o, want_dq, want_dk, want_dv = orc.attention_chain(r, c, Q, K, V, scale, dO)
    rt, at = TOL[dtype]
    # logits grow with mag**2 and the softmax amplifies their rounding error by their size
    rt, at = rt * mag ** 2, at * mag ** 2
    assert_close(o, want_o, rt, at, "o")
    # lse against the scores themselves
    s = orc.maskedmm_csr_forward(*r, Q, K) * scale
    dst = g.dst_of_edge()
    want_lse = th.full((g.n_dst, h), -float("inf"), dtype=th.float64)
    mx = th.full((g.n_dst, h), -float("inf"), dtype=th.float64).scatter_reduce_(
        0, dst.view(-1, 1).expand(-1, h), s.view(-1, h), reduce="amax")
    sm = th.zeros(g.n_dst, h, dtype=th.float64).index_add_(0, dst, th.exp(s.view(-1, h) - mx[dst]))
    deg = g.indptr[1:] - g.indptr[:-1]
    want_lse[deg > 0] = (mx + th.log(sm))[deg > 0]
    got_lse = lse.cpu().double()
    assert bool((got_lse[deg == 0] == -float("inf")).all())
    assert_close(got_lse[deg > 0], want_lse[deg > 0], rt if dtype != th.bfloat16 else 1e-5, 1e-5, "lse")
    dq, dk, dv = graphop.attention_backward(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], Q.to(DEV), K.to(DEV),
                                            V.to(DEV), o, lse, dO.to(DEV), scale)
    if dtype == th.bfloat16:
        # o was rounded to bf16 before the backward read it: compare with a looser absolute floor
        at = 5e-2
    # Gradients are sums of products of two or three inputs: their absolute tolerance scales with the size of those
    # products (4x for dO . v against delta, two sums that cancel), and only rows above 256 edges get the
    # degree allowance of assert_rows_close.
    deg, deg_t = g.indptr[1:] - g.indptr[:-1], g.indptr_t[1:] - g.indptr_t[:-1]
    for got, want, dd, what in ((dq, want_dq, deg, "dq"), (dk, want_dk, deg_t, "dk"), (dv, want_dv, deg_t, "dv")):
        assert_rows_close(got, want, dd, rt, 4 * at * max(1.0, float(want.abs().max())), what)
    # the same backward with the transposed CSR's edge ids: (p, ds) handed from the destination pass to the
    # source pass instead of recomputed (valid when the row CSR's edge ids are its positions)
    assert th.equal(r[2].long(), th.arange(g.n_edges))
    dq2, dk2, dv2 = graphop.attention_backward(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], Q.to(DEV), K.to(DEV),
                                               V.to(DEV), o, lse, dO.to(DEV), scale, eid_t=cc[2])
    assert th.equal(dq2, dq)
    for got, want, what in ((dk2, want_dk, "dk (pairs)"), (dv2, want_dv, "dv (pairs)")):
        assert_rows_close(got, want, deg_t, rt, 4 * at * max(1.0, float(want.abs().max())), what)


def test_fused_attention_matches_dense_masked_config1():
    """The ER-small configuration: N=4096, 15 in-neighbours + self-loop, 8 heads x 64, fp32."""
    g = graphs.er_graph(4096, 15, seed=0)
    Q, K, V, dO = _qkv(g, 8, 64, th.float32, 1)
    r, c = chunked(g, 32, dtype=th.int32), chunked(g, 32, transposed=True, dtype=th.int32)
    rc, cc = [t.to(DEV) for t in r], [t.to(DEV) for t in c]
    want = orc.attention_dense_masked(g.indptr, g.indices, Q, K, V, 0.125, dO)
    o, lse = graphop.attention_forward(rc[0], rc[1], rc[3], Q.to(DEV), K.to(DEV), V.to(DEV), 0.125)
    got = [o] + graphop.attention_backward(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], Q.to(DEV), K.to(DEV), V.to(DEV),
                                           o, lse, dO.to(DEV), 0.125)
    for a, b, what in zip(got, want, ("o", "dq", "dk", "dv")):
        assert_close(a, b, 1e-5, 2e-6, what)


def test_fused_attention_is_bit_reproducible_and_matches_unfused_ops():
    g = ZOO[3][1]
    r, c = chunked(g, 32, dtype=th.int32), chunked(g, 32, transposed=True, dtype=th.int32)
    rc, cc = [t.to(DEV) for t in r], [t.to(DEV) for t in c]
    Q, K, V, dO = [t.to(DEV) for t in _qkv(g, 4, 32, th.float32, 2)]
    scale = 32 ** -0.5
    o1, l1 = graphop.attention_forward(rc[0], rc[1], rc[3], Q, K, V, scale)
    o2, l2 = graphop.attention_forward(rc[0], rc[1], rc[3], Q, K, V, scale)
    assert th.equal(o1, o2) and th.equal(l1, l2)
    b1 = graphop.attention_backward(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], Q, K, V, o1, l1, dO, scale)
    b2 = graphop.attention_backward(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], Q, K, V, o1, l1, dO, scale)
    for a, b in zip(b1, b2):
        assert th.equal(a, b)
    b3 = graphop.attention_backward(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], Q, K, V, o1, l1, dO, scale, eid_t=cc[2])
    b4 = graphop.attention_backward(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], Q, K, V, o1, l1, dO, scale, eid_t=cc[2])
    for a, b, c_ in zip(b3, b4, b1):
        assert th.equal(a, b)
        assert_close(a, c_.cpu().double(), 1e-5, 1e-5, "pairs vs recomputed")
    s = graphop.maskedmm_csr_forward(*rc, Q, K) * scale
    p = graphop.sparse_softmax_forward(*rc[:3], s)
    o3 = graphop.vector_spmm_forward(*rc, p, V, num_dst=g.n_dst)
    assert_close(o1, o3, 1e-5, 1e-6, "fused vs unfused")


# ------------------------------------------------------------------------------------------
# autograd wiring
# ------------------------------------------------------------------------------------------
def _leaf(t):
    return t.to(DEV).requires_grad_(True)


def test_autograd_functions_match_torch_autograd_float64():
    g = graphs.er_graph(40, 4, seed=3, index_dtype=th.int64)
    r, c = chunked(g, 3), chunked(g, 3, transposed=True)
    rc, cc = [t.to(DEV) for t in r], [t.to(DEV) for t in c]
    h, d, e, n = 2, 4, g.n_edges, g.n_dst
    gen = th.Generator().manual_seed(4)
    A0, B0 = th.randn(n, h, d, generator=gen, dtype=th.float64), th.randn(n, h, d, generator=gen, dtype=th.float64)
    Be0, w0 = th.randn(e, d, generator=gen, dtype=th.float64), th.rand(e, h, generator=gen, dtype=th.float64)
    dst, src = g.dst_of_edge().to(DEV), g.indices.to(DEV)

    # MaskedMMCSR
    A, B = _leaf(A0), _leaf(B0)
    y = wrapper.MaskedMMCSR.apply(*rc, *cc, A, B)
    A2, B2 = _leaf(A0), _leaf(B0)
    y2 = (A2[dst] * B2[src]).sum(-1)
    gy = th.randn_like(y)
    y.backward(gy), y2.backward(gy)
    assert_close(y, y2, 1e-12, 1e-12, "mm y")
    assert_close(A.grad, A2.grad, 1e-11, 1e-12, "mm dA")
    assert_close(B.grad, B2.grad, 1e-11, 1e-12, "mm dB")

    # SparseSoftmax
    x = _leaf(w0)
    p = wrapper.SparseSoftmax.apply(*rc[:3], x)
    x2 = _leaf(w0)
    ex = th.exp(x2 - x2.max())
    p2 = ex / th.zeros(n, h, dtype=th.float64, device=DEV).index_add(0, dst, ex)[dst]
    gp = th.randn_like(p)
    p.backward(gp), p2.backward(gp)
    assert_close(p, p2, 1e-12, 1e-14, "softmax y")
    assert_close(x.grad, x2.grad, 1e-10, 1e-13, "softmax dx")

    # NodeMulEdge
    A, Be = _leaf(A0), _leaf(Be0)
    y = wrapper.NodeMulEdge.apply(*rc[:3], A, Be)
    A2, Be2 = _leaf(A0), _leaf(Be0)
    y2 = (A2[dst] * Be2.unsqueeze(1)).sum(-1)
    y.backward(gy), y2.backward(gy)
    assert_close(y, y2, 1e-12, 1e-12, "nme y")
    assert_close(A.grad, A2.grad, 1e-11, 1e-12, "nme dA")
    assert_close(Be.grad, Be2.grad, 1e-11, 1e-12, "nme dB")

    # VectorSPMM
    w, xx = _leaf(w0), _leaf(A0)
    o = wrapper.VectorSPMM.apply(*rc, *cc, w, xx)
    w2, xx2 = _leaf(w0), _leaf(A0)
    o2 = th.zeros(n, h, d, dtype=th.float64, device=DEV).index_add(0, dst, w2.unsqueeze(-1) * xx2[src])
    go = th.randn_like(o)
    o.backward(go), o2.backward(go)
    assert_close(o, o2, 1e-12, 1e-12, "spmm y")
    assert_close(w.grad, w2.grad, 1e-11, 1e-12, "spmm dedata")
    assert_close(xx.grad, xx2.grad, 1e-11, 1e-12, "spmm dx")

    # GraphAttention and the dispatching helper
    Q, K, V = _leaf(A0), _leaf(B0), _leaf(A0 * 0.5 + B0)
    out = wrapper.graph_attention(*rc, *cc, Q, K, V, 0.5)
    Q2, K2, V2 = _leaf(A0), _leaf(B0), _leaf(A0 * 0.5 + B0)
    s = (Q2[dst] * K2[src]).sum(-1) * 0.5
    ex = th.exp(s - s.max())
    pp = ex / th.zeros(n, h, dtype=th.float64, device=DEV).index_add(0, dst, ex)[dst]
    out2 = th.zeros(n, h, d, dtype=th.float64, device=DEV).index_add(0, dst, pp.unsqueeze(-1) * V2[src])
    out.backward(go), out2.backward(go)
    assert_close(out, out2, 1e-11, 1e-12, "attn o")
    for a, b, what in ((Q, Q2, "dq"), (K, K2, "dk"), (V, V2, "dv")):
        assert_close(a.grad, b.grad, 1e-10, 1e-12, "attn " + what)


def test_gradcheck_on_a_tiny_graph():
    g = graphs.er_graph(6, 2, seed=5, index_dtype=th.int64)
    r, c = chunked(g, 2), chunked(g, 2, transposed=True)
    rc, cc = [t.to(DEV) for t in r], [t.to(DEV) for t in c]
    gen = th.Generator().manual_seed(6)
    mk = lambda *s: th.randn(*s, generator=gen, dtype=th.float64).to(DEV).requires_grad_(True)
    n, e = g.n_dst, g.n_edges
    assert th.autograd.gradcheck(lambda a, b: wrapper.MaskedMMCSR.apply(*rc, *cc, a, b), (mk(n, 2, 4), mk(n, 2, 4)))
    assert th.autograd.gradcheck(lambda x: wrapper.SparseSoftmax.apply(*rc[:3], x), (mk(e, 2),))
    assert th.autograd.gradcheck(lambda a, b: wrapper.NodeMulEdge.apply(*rc[:3], a, b), (mk(n, 2, 4), mk(e, 4)))
    assert th.autograd.gradcheck(lambda w, x: wrapper.VectorSPMM.apply(*rc, *cc, w, x), (mk(e, 2), mk(n, 2, 4)))
    assert th.autograd.gradcheck(
        lambda q, k, v: wrapper.GraphAttention.apply(rc[0], rc[1], rc[3], cc[0], cc[1], cc[3], q, k, v, 0.7),
        (mk(n, 2, 4), mk(n, 2, 4), mk(n, 2, 4)))


def test_unfused_fallback_of_graph_attention():
    g = graphs.er_graph(50, 3, seed=7, index_dtype=th.int64)
    r, c = chunked(g, 32), chunked(g, 32, transposed=True)
    rc, cc = [t.to(DEV) for t in r], [t.to(DEV) for t in c]
    Q, K, V, dO = _qkv(g, 3, 5, th.float64, 8)   # D = 5: outside the fused kernels' shapes
    assert not graphop.attention_supported(Q.to(DEV))
    q, k, v = _leaf(Q), _leaf(K), _leaf(V)
    o = wrapper.graph_attention(*rc, *cc, q, k, v, 0.4)
    o.backward(dO.to(DEV))
    want = orc.attention_chain(r, c, Q, K, V, 0.4, dO)
    for a, b, what in zip((o, q.grad, k.grad, v.grad), want, ("o", "dq", "dk", "dv")):
        assert_close(a, b, 1e-10, 1e-12, what)
