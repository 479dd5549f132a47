"""Full-size checks on the BASELINE configurations, where the CPU oracle would take minutes:
size-independent properties instead of element-wise comparison.

* adjoint identities: <y, dy> == <x, dx> for (vector_spmm forward, its dx), <s, ds> == <A, dA> for
  (maskedmm forward, its dA) and the same for dB; these tie each backward kernel to its forward at
  34.5 M edges;
* softmax rows sum to one (also with logits scaled to +-600 on the Zipf graph, rows up to 10^6 edges);
* the fused chain equals the chain of the three unfused ops, forward and backward;
* bit-identical results on a second run.
Inner products are accumulated in float64 on the device."""
import pytest
import torch as th

from custom_op_benchmark_b200 import graphop, graphs
from custom_op_benchmark_b200.part_csr import partition_csr

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tables(g):
    row, ptr = partition_csr(g.indptr, 32)
    col, ptr_t = partition_csr(g.indptr_t, 32)
    return [row.int(), ptr.int(), g.eid, g.indices], [col.int(), ptr_t.int(), g.eid_t, g.indices_t]


def _dot(a, b):
    return float((a.double() * b.double()).sum())


def _rel(a, b):
    return abs(a - b) / max(abs(a), abs(b), 1e-30)


@pytest.fixture(scope="module")
def rmat21():
    g = graphs.rmat_graph(21, 16, seed=0, device=DEV)
    return g, _tables(g)


def test_rmat21_adjoint_identities_and_softmax_rows(rmat21):
    g, (R, C) = rmat21
    n, e, h, d = g.n_dst, g.n_edges, 4, 32
    gen = th.Generator(device=DEV).manual_seed(1)
    rn = lambda *s: th.randn(*s, generator=gen, device=DEV)
    x, dy, A, B = rn(n, h, d), rn(n, h, d), rn(n, h, d), rn(n, h, d)
    raw, ds = th.rand(e, h, generator=gen, device=DEV), rn(e, h)
    w = graphop.sparse_softmax_forward(*R[:3], raw)
    dst = g.dst_of_edge()
    sums = th.zeros(n, h, dtype=th.float64, device=DEV).index_add_(0, dst, w.double())
    assert float((sums - 1).abs().max()) < 1e-5           # every node has its self-loop: every row sums to 1
    y = graphop.vector_spmm_forward(*R, w, x)
    dw, dx = graphop.vector_spmm_backward(*R, *C, w, dy, x)
    assert _rel(_dot(y, dy), _dot(x, dx)) < 1e-5          # <Wx, dy> == <x, W^T dy>
    assert _rel(_dot(y, dy), _dot(w, dw)) < 1e-5          # y is linear in w as well
    s = graphop.maskedmm_csr_forward(*R, A, B)
    dA, dB = graphop.maskedmm_csr_backward(*R, *C, A, B, ds)
    assert _rel(_dot(s, ds), _dot(A, dA)) < 1e-5          # s is bilinear in (A, B)
    assert _rel(_dot(s, ds), _dot(B, dB)) < 1e-5
    assert th.equal(y, graphop.vector_spmm_forward(*R, w, x))
    assert th.equal(dA, graphop.maskedmm_csr_backward(*R, *C, A, B, ds)[0])


def test_rmat21_fused_chain_equals_unfused_ops(rmat21):
    g, (R, C) = rmat21
    n, h, d = g.n_dst, 4, 32
    gen = th.Generator(device=DEV).manual_seed(2)
    Q, K, V, dO = (th.randn(n, h, d, generator=gen, device=DEV) for _ in range(4))
    scale = d ** -0.5
    o, lse = graphop.attention_forward(R[0], R[1], R[3], Q, K, V, scale)
    dq, dk, dv = graphop.attention_backward(R[0], R[1], R[3], C[0], C[1], C[3], Q, K, V, o, lse, dO, scale,
                                            eid_t=C[2])
    s = graphop.maskedmm_csr_forward(*R, Q, K) * scale
    p = graphop.sparse_softmax_forward(*R[:3], s)
    o2 = graphop.vector_spmm_forward(*R, p, V)
    dp, dv2 = graphop.vector_spmm_backward(*R, *C, p, dO, V)
    dsc = graphop.sparse_softmax_backward(*R[:3], p, dp) * scale
    dq2, dk2 = graphop.maskedmm_csr_backward(*R, *C, Q, K, dsc)
    for a, b, what in ((o, o2, "o"), (dq, dq2, "dq"), (dk, dk2, "dk"), (dv, dv2, "dv")):
        err = float((a - b).abs().max())
        ref = float(b.abs().max())
        assert err <= 2e-5 * ref + 1e-5, "%s: max abs diff %g against magnitude %g" % (what, err, ref)
    o3, lse3 = graphop.attention_forward(R[0], R[1], R[3], Q, K, V, scale)
    assert th.equal(o, o3) and th.equal(lse, lse3)


def test_zipf_full_size_softmax_under_large_logits():
    g = graphs.zipf_graph(1_000_000, 50_000_000, 1.1, seed=0, device=DEV)
    R, _ = _tables(g)
    n, e, h, d = g.n_dst, g.n_edges, 2, 64
    assert int((g.indptr[1:] - g.indptr[:-1]).max()) == 1_000_000       # the capped rows exist
    gen = th.Generator(device=DEV).manual_seed(3)
    Q, K = (th.randn(n, h, d, generator=gen, device=DEV) * 3 for _ in range(2))
    s = graphop.maskedmm_csr_forward(*R, Q, K)
    assert float(s.abs().max()) > 300                                   # max-subtraction is really needed
    p = graphop.sparse_softmax_forward(*R[:3], s)
    assert bool(th.isfinite(p).all()) and float(p.min()) >= 0
    sums = th.zeros(n, h, dtype=th.float64, device=DEV).index_add_(0, g.dst_of_edge(), p.double())
    assert float((sums - 1).abs().max()) < 1e-4
    dp = th.randn(e, h, generator=gen, device=DEV)
    dx = graphop.sparse_softmax_backward(*R[:3], p, dp)
    # softmax backward is orthogonal to the all-ones direction of every row
    rowsum = th.zeros(n, h, dtype=th.float64, device=DEV).index_add_(0, g.dst_of_edge(), dx.double())
    assert float(rowsum.abs().max()) < 1e-4
    assert th.equal(p, graphop.sparse_softmax_forward(*R[:3], s))
