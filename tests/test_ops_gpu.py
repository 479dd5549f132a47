"""Parity of the CUDA ops with the CPU oracle, through the C ABI (ctypes -> libgraphop_b200.so).

Tolerances: float64 1e-10 relative (the kernels and the oracle differ only in summation
order); float32 rel 1e-5 / abs 1e-6 on inputs scaled so that outputs are O(1); bfloat16
inputs with fp32 accumulation rel 2e-2 against the oracle run on the bf16-rounded inputs.
"""
import ctypes

import pytest
import torch as th

from helpers import assert_close, chunked, graph_zoo, random_graph
from custom_op_benchmark_b200 import _capi, graphop, graphs
from custom_op_benchmark_b200.part_csr import partition_csr
from oracle import graphop_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ZOO = graph_zoo()
TOL = {th.float64: (1e-10, 1e-12), th.float32: (1e-5, 1e-6), th.bfloat16: (2e-2, 2e-2)}


def _gen(seed):
    return th.Generator().manual_seed(seed)


def _nodes(n, h, d, dtype, seed, scale=1.0):
    t = th.randn(n, h, d, generator=_gen(seed), dtype=th.float64) * scale
    t = t.to(dtype)
    return t.view(n, d) if h == 1 else t


def _edges(e, h, dtype, seed, uniform=True):
    g = _gen(seed)
    t = th.rand(e, h, generator=g, dtype=th.float64) if uniform else th.randn(e, h, generator=g, dtype=th.float64)
    t = t.to(dtype)
    return t.view(e) if h == 1 else t


def _cuda(ts):
    return [t.to(DEV) for t in ts]


def _atol(g, dtype):
    """Absolute tolerance of a per-node sum: the stated one up to 256 edges per node; beyond
    that fp32 round-off of a sum grows with sqrt(degree) and the tolerance follows it."""
    at = TOL[dtype][1]
    deg = int((g.indptr[1:] - g.indptr[:-1]).max()) if g.n_edges else 1
    degt = int((g.indptr_t[1:] - g.indptr_t[:-1]).max()) if g.n_edges else 1
    return at * max(1.0, (max(deg, degt) / 256.0) ** 0.5)


def _row_weights(g, h, dtype, seed):
    """U(0,1) edge weights divided by the in-degree of the edge's node: sums stay O(1)."""
    deg = (g.indptr[1:] - g.indptr[:-1]).to(th.float64).clamp(min=1)
    w = th.rand(g.n_edges, h, generator=_gen(seed), dtype=th.float64) / deg[g.dst_of_edge()].sqrt().unsqueeze(1)
    w = w.to(dtype)
    return w.view(-1) if h == 1 else w


SHAPES = [(1, 16), (4, 32), (8, 64), (2, 64), (1, 128), (3, 5), (1, 1), (2, 12), (1, 1024), (8, 160)]


# ------------------------------------------------------------------------------------------
# vector_spmm
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,g", ZOO, ids=[z[0] for z in ZOO])
@pytest.mark.parametrize("cs", [32, 7, None])
@pytest.mark.parametrize("h,d,dtype,idt", [
    (4, 32, th.float64, th.int64), (4, 32, th.float32, th.int32), (8, 64, th.float32, th.int64),
    (1, 128, th.float32, th.int32), (3, 5, th.float64, th.int32), (1, 1, th.float32, th.int64),
    (8, 64, th.bfloat16, th.int32), (1, 1024, th.float32, th.int32), (8, 160, th.float64, th.int64),
    # weight rows that are not a whole number of 16-byte pieces (12, 8 and 6 bytes), vectorised features
    (3, 8, th.float32, th.int32), (2, 16, th.float32, th.int64), (3, 16, th.bfloat16, th.int32),
    # 2-byte weights that travel as 4-byte words (an even number of heads: 4, 8 and 12 bytes per edge)
    (2, 16, th.bfloat16, th.int32), (4, 32, th.bfloat16, th.int64), (6, 8, th.bfloat16, th.int32),
    # ... and as the words that cover an odd number of them (rows start in either half of a word)
    (1, 32, th.bfloat16, th.int32), (5, 8, th.bfloat16, th.int64), (1, 128, th.bfloat16, th.int32),
])
def test_vector_spmm(name, g, cs, h, d, dtype, idt):
    if g.n_dst > g.n_src:
        pytest.skip("the reference signature returns y with x's row count")
    r, c = chunked(g, cs, dtype=idt), chunked(g, cs, transposed=True, dtype=idt)
    w = _row_weights(g, h, dtype, 1)
    x = _nodes(g.n_src, h, d, dtype, 2)
    dy = _nodes(g.n_src, h, d, dtype, 3)
    rt, at = TOL[dtype][0], _atol(g, dtype)
    y = graphop.vector_spmm_forward(*_cuda(r), w.to(DEV), x.to(DEV))
    assert_close(y, orc.vector_spmm_forward(*r, w, x), rt, at, "y")
    ded, dx = graphop.vector_spmm_backward(*_cuda(r), *_cuda(c), w.to(DEV), dy.to(DEV), x.to(DEV))
    want_ded, want_dx = orc.vector_spmm_backward(*r, *c, w, dy, x)
    scale = max(1.0, float(want_ded.abs().max()))
    assert_close(ded, want_ded, rt, at * scale, "dedata")
    assert_close(dx, want_dx, rt, at * max(1.0, float(want_dx.abs().max())), "dx")
    assert ded.shape == w.shape and dx.shape == x.shape


@pytest.mark.parametrize("h", [1, 2, 3, 4])
@pytest.mark.parametrize("lead,tail", [(1, 0), (1, 1), (2, 1), (0, 1)])
def test_vector_spmm_bf16_weights_at_any_2_byte_alignment(h, lead, tail):
    """bfloat16 edge weights in a view that starts `lead` elements into its allocation and stops `tail` elements
    before its end: rows begin in either half of an aligned 4-byte word, and the words at the tensor's two ends
    are only half inside it.  The elements around the view hold NaN: a weight read from outside would show."""
    g = ZOO[0][1]
    r = chunked(g, 32, dtype=th.int32)
    w = _row_weights(g, h, th.bfloat16, 1)
    x = _nodes(g.n_src, h, 32, th.bfloat16, 2)
    box = th.full((lead + w.numel() + tail,), float("nan"), dtype=th.bfloat16, device=DEV)
    view = box[lead:lead + w.numel()].view(w.shape)
    view.copy_(w)
    assert view.is_contiguous() and view.data_ptr() % 4 == (2 * lead) % 4
    y = graphop.vector_spmm_forward(*_cuda(r), view, x.to(DEV))
    assert_close(y, orc.vector_spmm_forward(*r, w, x), TOL[th.bfloat16][0], _atol(g, th.bfloat16), "y")


def test_vector_spmm_rectangular_num_dst():
    g = ZOO[2][1]  # 200 destinations, 150 sources
    r = chunked(g, 32, dtype=th.int32)
    w, x = _row_weights(g, 4, th.float32, 1), _nodes(g.n_src, 4, 32, th.float32, 2)
    y = graphop.vector_spmm_forward(*_cuda(r), w.to(DEV), x.to(DEV), num_dst=g.n_dst)
    assert y.shape == (g.n_dst, 4, 32)
    assert_close(y, orc.vector_spmm_forward(*r, w, x, num_dst=g.n_dst), 1e-5, 1e-6, "y")


# ------------------------------------------------------------------------------------------
# maskedmm_csr
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,g", ZOO, ids=[z[0] for z in ZOO])
@pytest.mark.parametrize("cs", [32, 5, None])
@pytest.mark.parametrize("h,d,dtype,idt", [
    (8, 64, th.float64, th.int64), (8, 64, th.float32, th.int32), (4, 32, th.float32, th.int64),
    (2, 64, th.float32, th.int32), (1, 1024, th.float32, th.int64), (3, 5, th.float32, th.int32),
    (2, 12, th.float64, th.int32), (1, 1, th.float64, th.int64), (4, 32, th.bfloat16, th.int32),
    (8, 160, th.float32, th.int32),
])
def test_maskedmm(name, g, cs, h, d, dtype, idt):
    r, c = chunked(g, cs, dtype=idt), chunked(g, cs, transposed=True, dtype=idt)
    s = d ** -0.25
    A = _nodes(g.n_dst, h, d, dtype, 4, s)
    B = _nodes(g.n_src, h, d, dtype, 5, s)
    deg = (g.indptr[1:] - g.indptr[:-1]).to(th.float64).clamp(min=1)
    dy = (th.randn(g.n_edges, h, generator=_gen(6), dtype=th.float64) / deg[g.dst_of_edge()].sqrt().unsqueeze(1))
    dy = dy.to(dtype)
    dy = dy.view(-1) if h == 1 else dy
    rt, at = TOL[dtype]
    y = graphop.maskedmm_csr_forward(*_cuda(r), A.to(DEV), B.to(DEV))
    assert y.shape == ((g.n_edges,) if h == 1 else (g.n_edges, h))
    assert_close(y, orc.maskedmm_csr_forward(*r, A, B), rt, at, "y")
    dA, dB = graphop.maskedmm_csr_backward(*_cuda(r), *_cuda(c), A.to(DEV), B.to(DEV), dy.to(DEV))
    want_dA, want_dB = orc.maskedmm_csr_backward(*r, *c, A, B, dy)
    assert_close(dA, want_dA, rt, at * max(1.0, float(want_dA.abs().max())), "dA")
    assert_close(dB, want_dB, rt, at * max(1.0, float(want_dB.abs().max())), "dB")


# ------------------------------------------------------------------------------------------
# node_mul_edge
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,g", ZOO, ids=[z[0] for z in ZOO])
@pytest.mark.parametrize("cs", [32, 9, None])
@pytest.mark.parametrize("h,d,dtype,idt", [
    (8, 64, th.float32, th.int64), (4, 32, th.float32, th.int32), (4, 32, th.float64, th.int32),
    (1, 16, th.float32, th.int32), (3, 5, th.float64, th.int64), (8, 64, th.bfloat16, th.int32),
    (2, 12, th.float32, th.int32), (4, 32, th.bfloat16, th.int32), (2, 64, th.bfloat16, th.int64),
])
def test_node_mul_edge(name, g, cs, h, d, dtype, idt):
    r = chunked(g, cs, dtype=idt)[:3]
    s = d ** -0.25
    A = _nodes(g.n_dst, h, d, dtype, 7, s)
    Be = (th.randn(g.n_edges, d, generator=_gen(8), dtype=th.float64) * s).to(dtype)
    deg = (g.indptr[1:] - g.indptr[:-1]).to(th.float64).clamp(min=1)
    dy = (th.randn(g.n_edges, h, generator=_gen(9), dtype=th.float64) / deg[g.dst_of_edge()].sqrt().unsqueeze(1))
    dy = dy.to(dtype)
    dy = dy.view(-1) if h == 1 else dy
    rt, at = TOL[dtype]
    y = graphop.node_mul_edge_forward(*_cuda(r), A.to(DEV), Be.to(DEV))
    assert_close(y, orc.node_mul_edge_forward(*r, A, Be), rt, at, "y")
    dA, dB = graphop.node_mul_edge_backward(*_cuda(r), A.to(DEV), Be.to(DEV), dy.to(DEV))
    want_dA, want_dB = orc.node_mul_edge_backward(*r, A, Be, dy)
    assert_close(dA, want_dA, rt, at * max(1.0, float(want_dA.abs().max())), "dA")
    assert_close(dB, want_dB, rt, at * max(1.0, float(want_dB.abs().max())), "dB")


# ------------------------------------------------------------------------------------------
# sparse_softmax
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,g", ZOO, ids=[z[0] for z in ZOO])
@pytest.mark.parametrize("cs", [32, 6, None])
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("h,dtype,idt,mag", [
    (1, th.float32, th.int64, 1.0), (2, th.float32, th.int32, 30.0), (4, th.float32, th.int32, 1.0),
    (8, th.float32, th.int64, 5.0), (4, th.float64, th.int32, 30.0), (3, th.float32, th.int32, 1.0),
    (16, th.float64, th.int64, 1.0), (8, th.bfloat16, th.int32, 1.0),
])
def test_sparse_softmax(name, g, cs, transposed, h, dtype, idt, mag):
    r = chunked(g, cs, transposed=transposed, dtype=idt)[:3]
    x = (th.randn(g.n_edges, h, generator=_gen(10), dtype=th.float64) * mag).to(dtype)
    dy = th.randn(g.n_edges, h, generator=_gen(11), dtype=th.float64).to(dtype)
    if h == 1:
        x, dy = x.view(-1), dy.view(-1)
    rt, at = TOL[dtype]
    y = graphop.sparse_softmax_forward(*_cuda(r), x.to(DEV))
    want_y = orc.sparse_softmax_forward(*r, x)
    assert_close(y, want_y, rt, at, "y")
    dx = graphop.sparse_softmax_backward(*_cuda(r), y, dy.to(DEV))
    # the backward is checked on the forward's own (rounded) output, as the reference test does
    want_dx = orc.sparse_softmax_backward(*r, y.cpu(), dy)
    assert_close(dx, want_dx, rt if dtype != th.float32 else 1e-4, at, "dx")


def test_softmax_large_magnitude_rows_sum_to_one():
    g = ZOO[3][1]  # long rows
    r = chunked(g, 32, dtype=th.int32)[:3]
    x = th.randn(g.n_edges, 2, generator=_gen(12)) * 200.0
    y = graphop.sparse_softmax_forward(*_cuda(r), x.to(DEV)).cpu().double()
    assert bool(th.isfinite(y).all())
    sums = th.zeros(g.n_dst, 2, dtype=th.float64).index_add_(0, g.dst_of_edge(), y)
    deg = g.indptr[1:] - g.indptr[:-1]
    assert_close(sums[deg > 0], th.ones_like(sums[deg > 0]), 1e-5, 1e-6, "row sums")


# ------------------------------------------------------------------------------------------
# partial coverage, permuted edge ids, determinism, medium scale
# ------------------------------------------------------------------------------------------
def test_uncovered_edges_get_zero_and_eid_permutation_is_honoured():
    g = ZOO[3][1]
    row, ptr, eid, idx = chunked(g, 32, dtype=th.int64)
    perm = th.randperm(g.n_edges, generator=_gen(13))
    eid = perm  # position k -> edge id perm[k]
    row2, ptr2 = row[3:-4], ptr[3:-4]  # leading and trailing positions are covered by no chunk
    A, B = _nodes(g.n_dst, 4, 32, th.float32, 14, 0.4), _nodes(g.n_src, 4, 32, th.float32, 15, 0.4)
    y = graphop.maskedmm_csr_forward(*_cuda([row2, ptr2, eid, idx]), A.to(DEV), B.to(DEV))
    want = orc.maskedmm_csr_forward(row2, ptr2, eid, idx, A, B)
    assert_close(y, want, 1e-5, 1e-6, "maskedmm")
    assert int((want == 0).all(1).sum()) >= 7
    x = _edges(g.n_edges, 4, th.float32, 16, uniform=False)
    s = graphop.sparse_softmax_forward(*_cuda([row2, ptr2, eid]), x.to(DEV))
    assert_close(s, orc.sparse_softmax_forward(row2, ptr2, eid, x), 1e-5, 1e-6, "softmax")
    w = _row_weights(g, 4, th.float32, 17)
    xs = _nodes(max(g.n_src, g.n_dst), 4, 32, th.float32, 18)
    o = graphop.vector_spmm_forward(*_cuda([row2, ptr2, eid, idx]), w.to(DEV), xs.to(DEV))
    assert_close(o, orc.vector_spmm_forward(row2, ptr2, eid, idx, w, xs), 1e-5, _atol(g, th.float32), "spmm")


def test_results_are_bit_reproducible():
    g = ZOO[3][1]
    r, c = _cuda(chunked(g, 32, dtype=th.int32)), _cuda(chunked(g, 32, transposed=True, dtype=th.int32))
    w = _row_weights(g, 4, th.float32, 19).to(DEV)
    n = max(g.n_src, g.n_dst)
    x, dy = _nodes(n, 4, 32, th.float32, 20).to(DEV), _nodes(n, 4, 32, th.float32, 21).to(DEV)
    first = [graphop.vector_spmm_forward(*r, w, x)] + graphop.vector_spmm_backward(*r, *c, w, dy, x)
    first.append(graphop.sparse_softmax_forward(*r[:3], w))
    for _ in range(3):
        again = [graphop.vector_spmm_forward(*r, w, x)] + graphop.vector_spmm_backward(*r, *c, w, dy, x)
        again.append(graphop.sparse_softmax_forward(*r[:3], w))
        for a, b in zip(first, again):
            assert th.equal(a, b)


@pytest.mark.parametrize("maker", ["rmat", "zipf", "er", "banded"])
def test_medium_graphs_all_ops(maker):
    if maker == "rmat":
        g, h, d = graphs.rmat_graph(13, 16, seed=0), 4, 32
    elif maker == "zipf":
        g, h, d = graphs.zipf_graph(4000, 400_000, 1.1, cap=100_000, seed=0), 2, 64
    elif maker == "er":
        g, h, d = graphs.er_graph(4096, 15, seed=0), 8, 64
    else:
        g, h, d = graphs.banded_graph(2, 1024, 128), 8, 64
    r, c = chunked(g, 32), chunked(g, 32, transposed=True)
    rc, cc = _cuda(r), _cuda(c)
    Q, K, V = (_nodes(g.n_dst, h, d, th.float32, s) for s in (22, 23, 24))
    s = graphop.maskedmm_csr_forward(*rc, Q.to(DEV), K.to(DEV)) * (d ** -0.5)
    assert_close(s, orc.maskedmm_csr_forward(*r, Q, K) * (d ** -0.5), 1e-5, 1e-5, "scores")
    p = graphop.sparse_softmax_forward(*rc[:3], s)
    want_p = orc.sparse_softmax_forward(*r[:3], s.cpu())
    assert_close(p, want_p, 1e-5, 1e-7, "softmax")
    o = graphop.vector_spmm_forward(*rc, p, V.to(DEV))
    assert_close(o, orc.vector_spmm_forward(*r, p.cpu(), V), 1e-5, 1e-6, "spmm")
    dO = _nodes(g.n_dst, h, d, th.float32, 25)
    dp, dV = graphop.vector_spmm_backward(*rc, *cc, p, dO.to(DEV), V.to(DEV))
    want_dp, want_dV = orc.vector_spmm_backward(*r, *c, p.cpu(), dO, V)
    assert_close(dp, want_dp, 1e-5, 1e-5, "dp")
    assert_close(dV, want_dV, 1e-5, 1e-5, "dV")
    ds = graphop.sparse_softmax_backward(*rc[:3], p, dp)
    assert_close(ds, orc.sparse_softmax_backward(*r[:3], p.cpu(), dp.cpu()), 1e-4, 1e-6, "ds")
    dQ, dK = graphop.maskedmm_csr_backward(*rc, *cc, Q.to(DEV), K.to(DEV), ds)
    want_dQ, want_dK = orc.maskedmm_csr_backward(*r, *c, Q, K, ds.cpu())
    assert_close(dQ, want_dQ, 1e-5, 1e-5, "dQ")
    assert_close(dK, want_dK, 1e-5, 1e-5, "dK")


# ------------------------------------------------------------------------------------------
# the boundary itself
# ------------------------------------------------------------------------------------------
def test_input_checks_match_the_reference_messages():
    g = ZOO[0][1]
    r = chunked(g, 32)
    A = _nodes(g.n_dst, 2, 8, th.float32, 26)
    with pytest.raises(RuntimeError, match="row must be a CUDA tensor"):
        graphop.maskedmm_csr_forward(*r, A.to(DEV), A.to(DEV))
    rc = _cuda(r)
    with pytest.raises(RuntimeError, match="A must be a CUDA tensor"):
        graphop.maskedmm_csr_forward(*rc, A, A.to(DEV))
    with pytest.raises(RuntimeError, match="B must be contiguous"):
        graphop.maskedmm_csr_forward(*rc, A.to(DEV), A.to(DEV).transpose(1, 2).contiguous().transpose(1, 2))
    with pytest.raises(RuntimeError, match="not implemented for 'Half'"):
        graphop.maskedmm_csr_forward(*rc, A.to(DEV).half(), A.to(DEV).half())
    with pytest.raises(RuntimeError, match="share dtype"):
        graphop.maskedmm_csr_forward(rc[0].int(), *rc[1:], A.to(DEV), A.to(DEV))


def test_raw_c_abi_status_codes():
    lib = _capi.lib()
    g = ZOO[0][1]
    row, ptr, eid, idx = _cuda(chunked(g, 32, dtype=th.int32))
    w = _row_weights(g, 4, th.float32, 27).to(DEV)
    x = _nodes(g.n_src, 4, 32, th.float32, 28).to(DEV)
    y = th.empty_like(x)
    need = lib.graphop_workspace_bytes(_capi.OP_SPMM_FWD, g.n_edges, g.n_src, 4, 32, 4, 4)
    ws = th.empty(need + 256, dtype=th.uint8, device=DEV)
    base = (ws.data_ptr() + 255) // 256 * 256
    stream = th.cuda.current_stream().cuda_stream
    args = [row.data_ptr(), ptr.data_ptr(), eid.data_ptr(), idx.data_ptr(), w.data_ptr(), x.data_ptr(), y.data_ptr(),
            row.numel(), g.n_edges, g.n_dst, g.n_src, 4, 32]
    fn = lib.graphop_vector_spmm_forward_f32_i32
    assert fn(*args, base, need, stream) == _capi.OK
    th.cuda.synchronize()
    want = orc.vector_spmm_forward(*[t.cpu() for t in (row, ptr, eid, idx)], w.cpu(), x.cpu())
    assert_close(y, want, 1e-5, 1e-6, "raw call")
    # eid = NULL means the identity, which it is for the row CSR
    y2 = th.empty_like(x)
    args2 = list(args)
    args2[2], args2[6] = None, y2.data_ptr()
    assert fn(*args2, base, need, stream) == _capi.OK
    th.cuda.synchronize()
    assert th.equal(y, y2)
    assert fn(*args, base, 1024, stream) == _capi.ERR_WORKSPACE
    assert fn(*args, base + 8, need, stream) == _capi.ERR_WORKSPACE
    bad = list(args)
    bad[11] = 0  # H = 0
    assert fn(*bad, base, need, stream) == _capi.ERR_INVALID_ARGUMENT
    bad = list(args)
    bad[0] = None
    assert fn(*bad, base, need, stream) == _capi.ERR_INVALID_ARGUMENT
    th.cuda.synchronize()


def test_check_graph_reports_contract_violations():
    g = ZOO[0][1]
    row, ptr, eid, idx = _cuda(chunked(g, 32, dtype=th.int32))
    assert graphop.check_graph(row, ptr, eid, idx, g.n_dst, g.n_src) == 0
    bad_row = row.clone()
    bad_row[5] = bad_row[4] - 1 if int(bad_row[4]) > 0 else 3
    bad_row[6:] = bad_row[6:].clamp(min=int(bad_row[5]))
    swapped = row.flip(0).contiguous()
    assert graphop.check_graph(swapped, ptr, eid, idx, g.n_dst, g.n_src) & 2
    bad_idx = idx.clone()
    bad_idx[7] = g.n_src + 5
    assert graphop.check_graph(row, ptr, eid, bad_idx, g.n_dst, g.n_src) & 4
    bad_ptr = ptr.clone()
    bad_ptr[3] = bad_ptr[4] + 1
    assert graphop.check_graph(row, bad_ptr, eid, idx, g.n_dst, g.n_src) & 1


def test_empty_graph_and_empty_edges():
    z = lambda *s, dt=th.int64: th.zeros(*s, dtype=dt, device=DEV)
    row, ptr, eid, idx = z(0), z(1), z(0), z(0)
    x = th.randn(5, 2, 8, device=DEV)
    y = graphop.vector_spmm_forward(row, ptr, eid, idx, th.empty(0, 2, device=DEV), x)
    assert y.shape == x.shape and bool((y == 0).all())
    s = graphop.maskedmm_csr_forward(row, ptr, eid, idx, x, x)
    assert s.shape == (0, 2)
    assert graphop.sparse_softmax_forward(row, ptr, eid, th.empty(0, 2, device=DEV)).shape == (0, 2)
    # rows exist but none has an edge chunk: the un-chunked form of an edgeless graph
    row, ptr = th.arange(5, device=DEV), z(6)
    y = graphop.vector_spmm_forward(row, ptr, eid, idx, th.empty(0, 2, device=DEV), x)
    assert bool((y == 0).all())


# ------------------------------------------------------------------------------------------
# gather_rows (packs rows for the sharded exchange)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape,dtype,idt", [
    ((1000, 128), th.float32, th.int32), ((777, 4, 32), th.float32, th.int64), ((513, 8), th.bfloat16, th.int32),
    ((300, 2, 1024), th.float64, th.int64), ((64, 3), th.float32, th.int32), ((50, 4), th.float32, th.int64),
])
def test_gather_rows_is_an_exact_copy(shape, dtype, idt):
    gen = _gen(31)
    table = th.randn(*shape, generator=gen, dtype=th.float64).to(dtype).to(DEV)
    for count in (0, 1, 5, 4099):
        idx = th.randint(0, shape[0], (count,), generator=gen).to(idt).to(DEV)
        got = graphop.gather_rows(table, idx)
        assert got.shape == (count,) + tuple(shape[1:]) and th.equal(got, table[idx.long()])
    # into a slice of a larger buffer, as the exchange does
    idx = th.randint(0, shape[0], (37,), generator=gen).to(idt).to(DEV)
    buf = th.zeros((50,) + tuple(shape[1:]), dtype=dtype, device=DEV)
    graphop.gather_rows(table, idx, out=buf[13:])
    assert th.equal(buf[13:], table[idx.long()]) and not bool(buf[:13].any())


def test_gather_probe_status_codes():
    """The benchmark's gather probe (instrumented twin of the library): runs on valid arguments (it has no output
    to compare), refuses the rest."""
    import bench
    from custom_op_benchmark_b200 import _capi
    lib = bench.Twin().h
    probe = lib.graphop_bench_gather_probe_i32
    table = th.randn(100, 128, device=DEV)
    narrow = th.randn(100, 12, device=DEV)      # 48-byte rows: allowed (a multiple of 16)
    idx = th.randint(0, 100, (1000,), dtype=th.int32, device=DEV)
    sink = th.zeros(1, dtype=th.int32, device=DEV)
    st = th.cuda.current_stream().cuda_stream
    assert probe(idx.data_ptr(), 1000, table.data_ptr(), table.data_ptr(), 512, sink.data_ptr(), st) == _capi.OK
    assert probe(idx.data_ptr(), 1000, table.data_ptr(), None, 512, sink.data_ptr(), st) == _capi.OK
    assert probe(idx.data_ptr(), 1000, narrow.data_ptr(), None, 48, sink.data_ptr(), st) == _capi.OK
    assert probe(idx.data_ptr(), 0, table.data_ptr(), None, 512, sink.data_ptr(), st) == _capi.OK
    assert probe(idx.data_ptr(), 1000, table.data_ptr(), None, 24, sink.data_ptr(), st) == _capi.ERR_UNSUPPORTED
    assert probe(idx.data_ptr(), 1000, table.data_ptr(), None, 1024, sink.data_ptr(), st) == _capi.ERR_UNSUPPORTED
    assert probe(None, 1000, table.data_ptr(), None, 512, sink.data_ptr(), st) == _capi.ERR_INVALID_ARGUMENT
    th.cuda.synchronize()
    assert int(sink.item()) == 0


def test_pull_rows_reads_each_segment_from_its_own_table():
    """graphop_pull_rows_i32 with both tables on this GPU (on several GPUs the tables are peer mappings): rows of
    segment p come from table p, empty segments and segments of odd sizes included."""
    gen = th.Generator(device=DEV).manual_seed(77)
    tabs = [th.randn(n, 128, generator=gen, device=DEV) for n in (50, 1, 300)]
    counts = [37, 0, 1001]
    idx = [th.randint(0, t.size(0), (c,), generator=gen, device=DEV, dtype=th.int32) for t, c in zip(tabs, counts)]
    seg = [0, 37, 37, 1038]
    out = th.full((1038, 128), float("nan"), device=DEV)
    graphop.pull_rows([t.data_ptr() for t in tabs], seg, th.cat(idx), 512, out)
    want = th.cat([t[i.long()] for t, i in zip(tabs, idx)])
    assert th.equal(out, want)
    with pytest.raises(RuntimeError, match="seg"):
        graphop.pull_rows([tabs[0].data_ptr()], seg, th.cat(idx), 512, out)
    with pytest.raises(RuntimeError, match="not supported"):
        graphop.pull_rows([t.data_ptr() for t in tabs], seg, th.cat(idx), 500, out)      # rows must be 16-byte multiples
