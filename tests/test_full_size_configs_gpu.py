"""Every BASELINE configuration at its real size against an independent float64 reference.

The reference is oracle/edge_list_f64.py: plain torch index ops in float64 on the GPU, none of this package's
kernels.  Configurations 2, 3 and 5 are compared element by element (the float64 copies fit); configuration 4
(R-MAT scale 24, an 8 GiB node tensor) on ~4000 sampled rows per side: the 32 longest rows, rows without edges,
the first and the last row, the rest random, so rows beyond the 4 GiB byte offset of the node tensor are
among them.  Tolerances: rel 1e-5 / abs 1e-6 for fp32 on rows of at most 256 edges, the absolute part growing
with degree / 256 on longer rows (an fp32 sum of n signed terms of size s carries a rounding error of the order
eps * n * s in any summation order) and with the magnitude of the summed terms; rel 2e-2 for bf16 inputs."""
import pytest
import torch as th

from custom_op_benchmark_b200 import graphop, graphs
from custom_op_benchmark_b200.part_csr import partition_csr
from oracle import edge_list_f64 as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
RTOL, ATOL = 1e-5, 1e-6


def _tables(g):
    row, ptr = partition_csr(g.indptr, 32)
    col, ptr_t = partition_csr(g.indptr_t, 32)
    return [row.int(), ptr.int(), g.eid, g.indices], [col.int(), ptr_t.int(), g.eid_t, g.indices_t]


def _deg(indptr):
    ip = indptr.to(th.int64)
    return ip[1:] - ip[:-1]


def assert_rows(got, want, deg, what, rtol=RTOL, atol=ATOL, mag=1.0):
    """Row r of `got` against `want`: |diff| <= rtol |want| + atol * mag * max(1, deg[r] / 256)."""
    g, w = got.to(th.float64), want.to(th.float64)
    assert g.shape == w.shape, (what, g.shape, w.shape)
    allow = (deg.to(th.float64).clamp(min=256.0) / 256.0).view(-1, *([1] * (w.dim() - 1)))
    excess = (g - w).abs() - (rtol * w.abs() + atol * mag * allow)
    worst = float(excess.max()) if excess.numel() else 0.0
    if worst > 0:
        i = int(th.argmax(excess.view(-1)))
        r = i // max(1, w[0].numel())
        raise AssertionError("%s: worst excess %.3g at row %d (degree %d): got %.9g want %.9g" % (
            what, worst, r, int(deg[r]), float(g.view(-1)[i]), float(w.view(-1)[i])))


def test_config2_banded_bf16_fused_chain_full_size():
    g = graphs.banded_graph(4, 8192, 128, device=DEV)
    assert g.n_edges == 4 * 2_088_832
    R, C = _tables(g)
    h, d, scale = 8, 64, 0.125
    gen = th.Generator(device=DEV).manual_seed(2)
    Q, K, V, dO = (th.randn(g.n_dst, h, d, generator=gen, device=DEV).to(th.bfloat16) for _ in range(4))
    o, lse = graphop.attention_forward(R[0], R[1], R[3], Q, K, V, scale)
    dq, dk, dv = graphop.attention_backward(R[0], R[1], R[3], C[0], C[1], C[3], Q, K, V, o, lse, dO, scale, eid_t=C[2])
    # the backward reads the bf16-rounded O: give the reference the same O for delta by comparing against gradients
    # computed from the float64 O; the difference is within the bf16 tolerance
    wo, wl, wq, wk, wv = ref.attention_f64(g.indptr, g.indices, Q, K, V, scale, dO)
    deg, deg_t = _deg(g.indptr), _deg(g.indptr_t)
    assert_rows(o, wo, deg, "o", rtol=2e-2, atol=2e-2)
    assert_rows(lse, wl, deg, "lse", rtol=1e-5, atol=1e-4)
    assert_rows(dq, wq, deg, "dq", rtol=2e-2, atol=5e-2)
    assert_rows(dk, wk, deg_t, "dk", rtol=2e-2, atol=5e-2)
    assert_rows(dv, wv, deg_t, "dv", rtol=2e-2, atol=5e-2)
    # the same step through graph plans: a dense band in bfloat16 with 64 features runs on the tensor-core kernels
    plan_r = graphop.GraphPlan(*R, g.n_dst)
    plan_t = graphop.GraphPlan(*C, g.n_src)
    assert plan_r.dense_band and plan_t.dense_band and plan_r.band_span == 128 + 2 * 128
    o2, lse2 = graphop.attention_forward_planned(plan_r, Q, K, V, scale)
    dq2, dk2, dv2 = graphop.attention_backward_planned(plan_r, plan_t, Q, K, V, o2, lse2, dO, scale)
    assert_rows(o2, wo, deg, "o (tensor cores)", rtol=2e-2, atol=2e-2)
    assert_rows(lse2, wl, deg, "lse (tensor cores)", rtol=1e-5, atol=2e-3)
    assert_rows(dq2, wq, deg, "dq (tensor cores)", rtol=2e-2, atol=5e-2)
    assert_rows(dk2, wk, deg_t, "dk (tensor cores)", rtol=2e-2, atol=5e-2)
    assert_rows(dv2, wv, deg_t, "dv (tensor cores)", rtol=2e-2, atol=5e-2)
    assert not bool(th.isnan(o2).any() | th.isnan(dq2).any() | th.isnan(dk2).any() | th.isnan(dv2).any())


@pytest.fixture(scope="module")
def rmat21():
    g = graphs.rmat_graph(21, 16, seed=0, device=DEV)
    return g, _tables(g)


def test_config3_rmat21_fused_chain_every_element(rmat21):
    g, (R, C) = rmat21
    h, d, scale = 4, 32, 32 ** -0.5
    gen = th.Generator(device=DEV).manual_seed(3)
    Q, K, V, dO = (th.randn(g.n_dst, h, d, generator=gen, device=DEV) for _ in range(4))
    o, lse = graphop.attention_forward(R[0], R[1], R[3], Q, K, V, scale)
    dq, dk, dv = graphop.attention_backward(R[0], R[1], R[3], C[0], C[1], C[3], Q, K, V, o, lse, dO, scale, eid_t=C[2])
    wo, wl, wq, wk, wv = ref.attention_f64(g.indptr, g.indices, Q, K, V, scale, dO)
    deg, deg_t = _deg(g.indptr), _deg(g.indptr_t)
    assert int(deg.max()) > 10_000 and int((deg == 1).sum()) > 100_000     # hubs and self-loop-only rows are there
    assert_rows(o, wo, deg, "o")
    assert_rows(lse, wl, deg, "lse")
    # gradients sum products of O(|dO| |v|) ~ 10 magnitude terms: the absolute part scales with that
    assert_rows(dq, wq, deg, "dq", mag=10.0)
    assert_rows(dk, wk, deg_t, "dk", mag=10.0)
    assert_rows(dv, wv, deg_t, "dv", mag=10.0)


def test_config3_rmat21_node_mul_edge_and_spmm_every_element(rmat21):
    g, (R, C) = rmat21
    n, e, h, d = g.n_dst, g.n_edges, 4, 32
    gen = th.Generator(device=DEV).manual_seed(4)
    X = th.randn(n, h, d, generator=gen, device=DEV)
    Be = th.randn(e, d, generator=gen, device=DEV)
    w = graphop.sparse_softmax_forward(*R[:3], th.rand(e, h, generator=gen, device=DEV))
    dY1 = th.randn(e, h, generator=gen, device=DEV)
    dY2 = th.randn(n, h, d, generator=gen, device=DEV)
    y1 = graphop.node_mul_edge_forward(*R[:3], X, Be)
    y2 = graphop.vector_spmm_forward(*R, w, X)
    da, dbe = graphop.node_mul_edge_backward(*R[:3], X, Be, dY1)
    dw, dx = graphop.vector_spmm_backward(*R, *C, w, dY2, X)
    wy1, wy2, wdx, wdbe, wdw = ref.gat_f64(g.indptr, g.indices, X, Be, w, dY1, dY2)
    deg, deg_t = _deg(g.indptr), _deg(g.indptr_t)
    one = th.ones(e, dtype=th.int64, device=DEV)
    assert_rows(y1, wy1, one, "node_mul_edge y", mag=10.0)          # a dot product of 32 O(1) terms
    assert_rows(y2, wy2, deg, "vector_spmm y")
    assert_rows(dbe, wdbe, one, "node_mul_edge dB", mag=4.0)
    assert_rows(dw, wdw, one, "vector_spmm dedata", mag=10.0)
    # dX sums, per node, products dY1 * B_edge of two N(0, 1) factors (up to ~16 each) over its in-edges plus weighted dY2
    # rows over its out-edges: an fp32 sum of 256 such terms already carries ~256 * eps * 1 = 1.5e-5 of rounding
    assert_rows(da + dx, wdx, th.maximum(deg, deg_t), "dX (both ops)", mag=40.0)


def test_config5_zipf_sddmm_softmax_every_element():
    g = graphs.zipf_graph(1_000_000, 50_000_000, 1.1, seed=0, device=DEV)
    R, C = _tables(g)
    n, e, h, d = g.n_dst, g.n_edges, 2, 64
    deg, deg_t = _deg(g.indptr), _deg(g.indptr_t)
    assert int(deg.max()) == 1_000_000
    gen = th.Generator(device=DEV).manual_seed(5)
    Q, K = (th.randn(n, h, d, generator=gen, device=DEV) * 3 for _ in range(2))
    dP = th.randn(e, h, generator=gen, device=DEV)
    s = graphop.maskedmm_csr_forward(*R, Q, K)
    p = graphop.sparse_softmax_forward(*R[:3], s)
    ds = graphop.sparse_softmax_backward(*R[:3], p, dP)
    dq, dk = graphop.maskedmm_csr_backward(*R, *C, Q, K, ds)
    ws, wp, wq, wk = ref.sddmm_softmax_f64(g.indptr, g.indices, Q, K, dP)
    one = th.ones(e, dtype=th.int64, device=DEV)
    assert_rows(s, ws, one, "scores", mag=100.0)                    # 64 terms of magnitude ~9 each
    # the probabilities see the fp32 rounding of scores of magnitude up to ~600: exp amplifies an absolute score
    # error of ~3e-5 into a relative one of that size
    assert_rows(p, wp, one, "probabilities", rtol=2e-4, atol=1e-7)
    # gradients flow through p and ds of the same accuracy
    assert_rows(dq, wq, deg, "dq", rtol=2e-4, atol=1e-4)
    assert_rows(dk, wk, deg_t, "dk", rtol=2e-4, atol=1e-4)


def test_node_tensor_above_4gib_sampled_rows():
    """A 4.6 GB source tensor whose referenced rows lie mostly beyond the 4 GiB byte offset: the 64-bit row
    offsets (the reference multiplies 32-bit ints there, graphop_kernel.cu:49, 144)."""
    free_b, _ = th.cuda.mem_get_info()
    if free_b < 24e9:
        pytest.skip("needs ~20 GB of free device memory")
    n_src, n_dst, d = 9_000_000, 200_000, 128                        # 9e6 * 128 * 4 B = 4.6 GB
    gen = th.Generator(device=DEV).manual_seed(6)
    deg = th.randint(0, 12, (n_dst,), generator=gen, device=DEV)
    deg[7] = 40_000
    dst = th.repeat_interleave(th.arange(n_dst, device=DEV), deg)
    src = th.randint(8_400_000, n_src, (dst.numel(),), generator=gen, device=DEV)   # byte offsets > 4.3e9
    src[:1000] = th.randint(0, 1000, (1000,), generator=gen, device=DEV)
    g = graphs.coo_to_graph(dst, src, n_dst, n_src)
    R, C = _tables(g)
    x = th.randn(n_src, d, generator=gen, device=DEV)
    w = th.rand(g.n_edges, generator=gen, device=DEV)
    dy = th.randn(n_dst, d, generator=gen, device=DEV)
    assert x.numel() * 4 > 1 << 32
    y = graphop.vector_spmm_forward(*R, w, x, num_dst=n_dst)
    dw, dx = graphop.vector_spmm_backward(*R, *C, w, dy, x)
    rows = ref.pick_rows(g.indptr, 4000)
    want = ref.spmm_rows_f64(g.indptr, g.indices, None, w.view(-1, 1), x.view(n_src, 1, d), rows)
    assert_rows(y.index_select(0, rows).view(-1, 1, d), want, _deg(g.indptr)[rows], "y")
    pos, val = ref.sddmm_rows_f64(g.indptr, g.indices, dy.view(n_dst, 1, d), x.view(n_src, 1, d), rows)
    assert_rows(dw.index_select(0, pos).view(-1, 1), val, th.ones_like(pos), "dedata", mag=20.0)
    cols = th.unique(th.cat([ref.pick_rows(g.indptr_t, 2000, seed=1),
                             src[th.randint(0, src.numel(), (2000,), generator=gen, device=DEV)]]))
    want = ref.spmm_rows_f64(g.indptr_t, g.indices_t, g.eid_t, w.view(-1, 1), dy.view(n_dst, 1, d), cols)
    assert_rows(dx.index_select(0, cols).view(-1, 1, d), want, _deg(g.indptr_t)[cols], "dx")
    assert int(cols.max()) * d * 4 > 1 << 32


def test_config4_rmat24_spmm_sampled_rows():
    free_b, _ = th.cuda.mem_get_info()
    if free_b < 120e9:
        pytest.skip("needs ~100 GB of free device memory")
    g = graphs.rmat_graph(24, 32, seed=0, device=DEV)
    R, C = _tables(g)
    n, e, d = g.n_dst, g.n_edges, 128
    gen = th.Generator(device=DEV).manual_seed(7)
    x = th.randn(n, d, generator=gen, device=DEV)
    w = th.rand(e, generator=gen, device=DEV)
    dy = th.randn(n, d, generator=gen, device=DEV)
    assert x.numel() * 4 == 1 << 33
    y = graphop.vector_spmm_forward(*R, w, x)
    dw, dx = graphop.vector_spmm_backward(*R, *C, w, dy, x)
    rows = ref.pick_rows(g.indptr, 4000)
    assert int(rows.max()) == n - 1                                  # the last row: 8 GiB - 512 B into the tensor
    want = ref.spmm_rows_f64(g.indptr, g.indices, None, w.view(-1, 1), x.view(n, 1, d), rows)
    assert_rows(y.index_select(0, rows).view(-1, 1, d), want, _deg(g.indptr)[rows], "y")
    pos, val = ref.sddmm_rows_f64(g.indptr, g.indices, dy.view(n, 1, d), x.view(n, 1, d), rows)
    assert_rows(dw.index_select(0, pos).view(-1, 1), val, th.ones_like(pos), "dedata", mag=20.0)
    cols = ref.pick_rows(g.indptr_t, 4000, seed=1)
    want = ref.spmm_rows_f64(g.indptr_t, g.indices_t, g.eid_t, w.view(-1, 1), dy.view(n, 1, d), cols)
    assert_rows(dx.index_select(0, cols).view(-1, 1, d), want, _deg(g.indptr_t)[cols], "dx")
