"""Pins the CPU oracle against the formulas the reference's own test script asserts against
(wrapper.py:155-481): dense bmm for the masked matmul, th.softmax over each block for the
sparse softmax (row and column direction), a sparse-dense product for the SpMM, the
copy-to-edge broadcast for node_mul_edge, all with autograd for the backward halves; and
against the float64 dense-masked attention.  Same graph family as the reference (fully
connected blocks of l nodes) plus chunk tables the reference never exercised."""
import pytest
import torch as th

from helpers import chunked, graph_zoo, assert_close
from custom_op_benchmark_b200 import graphs
from oracle import graphop_oracle as orc

B, L = 4, 30
F64 = th.float64


@pytest.fixture(scope="module")
def blocks():
    return graphs.block_diagonal_graph(B, L)


def _rand(*shape, seed=0):
    return th.rand(*shape, generator=th.Generator().manual_seed(seed), dtype=F64)


@pytest.mark.parametrize("h,d", [(1, 16), (8, 8)])
@pytest.mark.parametrize("cs", [32, 7, None])
def test_maskedmm_matches_dense_bmm(blocks, h, d, cs):
    g, n, e = blocks, B * L, B * L * L
    shape = (n, d) if h == 1 else (n, h, d)
    A = _rand(*shape, seed=1).requires_grad_(True)
    Bm = _rand(*shape, seed=2).requires_grad_(True)
    grad = _rand(*((e,) if h == 1 else (e, h)), seed=3)
    # wrapper.py:185 (h = 1) and wrapper.py:364 (h = 8): batched dense product over each block
    a4 = A.view(B, L, h, d).transpose(1, 2)
    b4 = Bm.view(B, L, h, d).permute(0, 2, 3, 1)
    y_ref = (a4 @ b4).permute(0, 2, 3, 1).reshape(e, h)
    y_ref = y_ref.view(-1) if h == 1 else y_ref
    y_ref.backward(grad)
    r, c = chunked(g, cs), chunked(g, cs, transposed=True)
    y = orc.maskedmm_csr_forward(*r, A, Bm)
    assert_close(y, y_ref, 1e-12, 1e-12, "y")
    dA, dB = orc.maskedmm_csr_backward(*r, *c, A, Bm, grad)
    assert_close(dA, A.grad, 1e-12, 1e-12, "dA")
    assert_close(dB, Bm.grad, 1e-12, 1e-12, "dB")


@pytest.mark.parametrize("h", [1, 8])
@pytest.mark.parametrize("transposed", [False, True])
def test_softmax_matches_dense_softmax(blocks, h, transposed):
    g, e = blocks, B * L * L
    x = _rand(*((e,) if h == 1 else (e, h)), seed=4).requires_grad_(True)
    grad = _rand(*x.shape, seed=5)
    # wrapper.py:219, 246 (h = 1: softmax over dim -1 / -2 of the (B, l, l) block view) and
    # wrapper.py:395, 422 (h = 8: dims -2 / -3 of (B, l, l, h)); edge id = b*l*l + x*l + y
    xv = x.view(B, L, L, h)
    y_ref = th.softmax(xv, 1 if transposed else 2).reshape(x.shape)
    y_ref.backward(grad)
    r = chunked(g, 32, transposed=transposed)[:3]
    y = orc.sparse_softmax_forward(*r, x)
    assert_close(y, y_ref, 1e-12, 1e-14, "y")
    dx = orc.sparse_softmax_backward(*r, y, grad)
    assert_close(dx, x.grad, 1e-11, 1e-14, "dx")


@pytest.mark.parametrize("h,d", [(1, 16), (8, 8)])
def test_spmm_matches_sparse_mm(blocks, h, d):
    g, n, e = blocks, B * L, B * L * L
    x = _rand(*((n, d) if h == 1 else (n, h, d)), seed=6).requires_grad_(True)
    w = _rand(*((e,) if h == 1 else (e, h)), seed=7).requires_grad_(True)
    grad = _rand(*x.shape, seed=8)
    # wrapper.py:277, 459-462: one weighted adjacency product per head
    dst = g.dst_of_edge()
    src = g.indices.to(th.int64)
    w2, x3 = w.view(e, h), x.view(n, h, d)
    y_ref = th.zeros(n, h, d, dtype=F64).index_add(0, dst, w2.unsqueeze(-1) * x3[src]).view(x.shape)
    y_ref.backward(grad)
    r, c = chunked(g, 32), chunked(g, 32, transposed=True)
    y = orc.vector_spmm_forward(*r, w, x)
    assert_close(y, y_ref, 1e-12, 1e-12, "y")
    dw, dx = orc.vector_spmm_backward(*r, *c, w, grad, x)
    assert_close(dw, w.grad, 1e-12, 1e-12, "dedata")
    assert_close(dx, x.grad, 1e-12, 1e-12, "dx")


def test_node_mul_edge_matches_copy_to_edge(blocks):
    g, n, e, h, d = blocks, B * L, B * L * L, 8, 8
    A = _rand(n, h, d, seed=9).requires_grad_(True)
    Be = _rand(e, d, seed=10).requires_grad_(True)
    grad = _rand(e, h, seed=11)
    # wrapper.py:314-316: copy the destination row onto each edge, multiply, reduce over d
    y_ref = (A[g.dst_of_edge()] * Be.view(e, 1, d)).sum(-1)
    y_ref.backward(grad)
    r = chunked(g, 32)[:3]
    y = orc.node_mul_edge_forward(*r, A, Be)
    assert_close(y, y_ref, 1e-12, 1e-12, "y")
    dA, dB = orc.node_mul_edge_backward(*r, A, Be, grad)
    assert_close(dA, A.grad, 1e-12, 1e-12, "dA")
    assert_close(dB, Be.grad, 1e-12, 1e-12, "dB")


@pytest.mark.parametrize("name,g", [z for z in graph_zoo() if z[0] in ("er64", "blockdiag")], ids=lambda v: v if isinstance(v, str) else "")
def test_chain_matches_dense_masked(name, g):
    h, d = 2, 8
    gen = th.Generator().manual_seed(12)
    Q = th.randn(g.n_dst, h, d, generator=gen, dtype=F64)
    K = th.randn(g.n_src, h, d, generator=gen, dtype=F64)
    V = th.randn(g.n_src, h, d, generator=gen, dtype=F64)
    dO = th.randn(g.n_dst, h, d, generator=gen, dtype=F64)
    want = orc.attention_dense_masked(g.indptr, g.indices, Q, K, V, 0.35, dO)
    got = orc.attention_chain(chunked(g, 5), chunked(g, 5, transposed=True), Q, K, V, 0.35, dO)
    for a, b, what in zip(got, want, ("o", "dq", "dk", "dv")):
        assert_close(a, b, 1e-10, 1e-12, what)


def test_chunking_does_not_change_results():
    for name, g in graph_zoo():
        h, d = 2, 4
        gen = th.Generator().manual_seed(13)
        A = th.randn(g.n_dst, h, d, generator=gen, dtype=F64)
        Bm = th.randn(g.n_src, h, d, generator=gen, dtype=F64)
        w = th.rand(g.n_edges, h, generator=gen, dtype=F64)
        base = None
        for cs in (None, 32, 3):
            r = chunked(g, cs)
            out = (orc.maskedmm_csr_forward(*r, A, Bm), orc.sparse_softmax_forward(*r[:3], w),
                   orc.vector_spmm_forward(*r, w, Bm)[: g.n_dst] if g.n_dst <= g.n_src else None)
            if base is None:
                base = out
            else:
                for a, b in zip(out, base):
                    if a is not None:
                        assert_close(a, b, 1e-13, 1e-13, name)


def test_uncovered_edges_and_empty_rows_are_zero():
    g = graph_zoo()[2][1]  # sparse_empty_rows
    row, ptr, eid, idx = chunked(g, 4)
    # drop the last two chunks: their positions are covered by no chunk any more
    row2, ptr2 = row[:-2], ptr[:-2]
    x = th.rand(g.n_edges, 2, dtype=F64)
    y = orc.sparse_softmax_forward(row2, ptr2, eid, x)
    uncovered = eid[int(ptr2[-1]):]
    assert bool((y[uncovered] == 0).all()) and bool((y[eid[: int(ptr2[-1])]] > 0).all())
    deg = g.indptr[1:] - g.indptr[:-1]
    out = orc.vector_spmm_forward(row, ptr, eid, idx, x, th.rand(g.n_dst, 2, 3, dtype=F64))
    assert bool((out[deg == 0] == 0).all())
