"""The reference's own test script (wrapper.py:77-485) restated as a pytest: same graph (512
fully-connected blocks of 30 nodes), same U(0,1) inputs, same dense torch formulas to compare
against, same `allclose` tolerances (default rtol 1e-5 / atol 1e-8; rtol 1e-3 / atol 1e-6 for
the softmax backward), run through this package's ops.  The h = 8 SpMM backward, which the
reference computes but never asserts (wrapper.py:482-485), is asserted here."""
import pytest
import torch as th

from custom_op_benchmark_b200 import graphs
from custom_op_benchmark_b200.part_csr import partition_csr
from custom_op_benchmark_b200.wrapper import MaskedMMCSR, NodeMulEdge, SparseSoftmax, VectorSPMM, chunk_size

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BS, L = 512, 30
N, E = BS * L, BS * L * L


@pytest.fixture(scope="module")
def gr():
    g = graphs.block_diagonal_graph(BS, L, index_dtype=th.int64).to(DEV)
    ROW, INDPTR_R = partition_csr(g.indptr, chunk_size=chunk_size)
    COL, INDPTR_C = partition_csr(g.indptr_t, chunk_size=chunk_size)
    assert ROW.numel() == N  # every row is exactly one chunk, as in the reference run
    return g, ROW, INDPTR_R, COL, INDPTR_C


def _u(*s, seed):
    return th.rand(*s, generator=th.Generator(device=DEV).manual_seed(seed), device=DEV)


def test_single_head_masked_mm(gr):
    g, ROW, IR, COL, IC = gr
    dim = 1024
    A, B = _u(N, dim, seed=1).requires_grad_(True), _u(N, dim, seed=2).requires_grad_(True)
    grad = _u(E, seed=3)
    y_ori = (A.view(BS, L, dim) @ B.view(BS, L, dim).transpose(-1, -2)).view(-1)  # wrapper.py:185
    y_ori.backward(grad)
    A_grad, B_grad = A.grad.clone(), B.grad.clone()
    A.grad.zero_(), B.grad.zero_()
    y = MaskedMMCSR.apply(ROW, IR, g.eid, g.indices, COL, IC, g.eid_t, g.indices_t, A, B)
    assert th.allclose(y, y_ori)
    y.backward(grad)
    assert th.allclose(A.grad, A_grad) and th.allclose(B.grad, B_grad)


@pytest.mark.parametrize("h", [1, 8])
def test_softmax_scatter_and_gather(gr, h):
    g, ROW, IR, COL, IC = gr
    shape = (E,) if h == 1 else (E, h)
    grad = _u(*shape, seed=4)
    for transposed, (row, ptr, eid) in ((False, (ROW, IR, g.eid)), (True, (COL, IC, g.eid_t))):
        x = _u(*shape, seed=5).requires_grad_(True)
        dim = (1 if transposed else 2)
        y_ori = th.softmax(x.view(BS, L, L, h), dim).view(shape)  # wrapper.py:219, 246, 395, 422
        y_ori.backward(grad)
        x_grad = x.grad.clone()
        x.grad.zero_()
        y = SparseSoftmax.apply(row, ptr, eid, x)
        assert th.allclose(y_ori, y)
        y.backward(grad)
        assert th.allclose(x_grad, x.grad, rtol=1e-3, atol=1e-6)


def test_single_head_spmm(gr):
    g, ROW, IR, COL, IC = gr
    dim = 1024
    A = _u(N, dim, seed=6).requires_grad_(True)
    val = _u(E, seed=7).requires_grad_(True)
    grad = _u(N, dim, seed=8)
    dst = g.dst_of_edge()
    adj = th.sparse_coo_tensor(th.stack([dst, g.indices]), val, (N, N)).coalesce()  # wrapper.py:119
    y_ori = th.sparse.mm(adj, A)
    y_ori.backward(grad)
    A_grad, val_grad = A.grad.clone(), val.grad.clone()
    A.grad.zero_(), val.grad.zero_()
    y = VectorSPMM.apply(ROW, IR, g.eid, g.indices, COL, IC, g.eid_t, g.indices_t, val, A)
    assert th.allclose(y_ori, y)
    y.backward(grad)
    assert th.allclose(A_grad, A.grad) and th.allclose(val.grad, val_grad)


def test_multi_head_node_mul_edge(gr):
    g, ROW, IR, COL, IC = gr
    dim, h = 64, 8
    A = _u(N, dim * h, seed=9).requires_grad_(True)
    B = _u(E, dim, seed=10).requires_grad_(True)
    grad = _u(E, h, seed=11)
    A_e = A[g.dst_of_edge()]  # copy to edge, wrapper.py:314
    y_ori = (A_e.view(-1, h, dim) * B.view(-1, 1, dim)).sum(-1)
    y_ori.backward(grad)
    A_grad, B_grad = A.grad.clone(), B.grad.clone()
    A.grad.zero_(), B.grad.zero_()
    y = NodeMulEdge.apply(ROW, IR, g.eid, A.view(-1, h, dim), B.view(-1, dim))
    assert th.allclose(y_ori, y)
    y.backward(grad)
    assert th.allclose(A_grad, A.grad) and th.allclose(B_grad, B.grad)


def test_multi_head_masked_mm(gr):
    g, ROW, IR, COL, IC = gr
    dim, h = 64, 8
    A, B = _u(N, dim * h, seed=12).requires_grad_(True), _u(N, dim * h, seed=13).requires_grad_(True)
    grad = _u(E, h, seed=14)
    y_ori = (A.view(BS, L, h, dim).transpose(1, 2) @ B.view(BS, L, h, dim).permute(0, 2, 3, 1)) \
        .permute(0, 2, 3, 1).contiguous().view(-1, h)  # wrapper.py:364
    y_ori.backward(grad)
    A_grad, B_grad = A.grad.clone(), B.grad.clone()
    A.grad.zero_(), B.grad.zero_()
    y = MaskedMMCSR.apply(ROW, IR, g.eid, g.indices, COL, IC, g.eid_t, g.indices_t, A.view(-1, h, dim),
                          B.view(-1, h, dim))
    assert th.allclose(y, y_ori)
    y.backward(grad)
    assert th.allclose(A.grad, A_grad) and th.allclose(B.grad, B_grad)


def test_multi_head_spmm_forward_and_backward(gr):
    g, ROW, IR, COL, IC = gr
    dim, h = 64, 8
    A = _u(N, h, dim, seed=15).requires_grad_(True)
    val = _u(E, h, seed=16).requires_grad_(True)
    grad = _u(N, h, dim, seed=17)
    dst = g.dst_of_edge()
    y_ori = th.zeros(N, h, dim, device=DEV).index_add(0, dst, val.unsqueeze(-1) * A[g.indices])
    y_ori.backward(grad)
    A_grad, val_grad = A.grad.clone(), val.grad.clone()
    A.grad.zero_(), val.grad.zero_()
    y = VectorSPMM.apply(ROW, IR, g.eid, g.indices, COL, IC, g.eid_t, g.indices_t, val, A)
    assert th.allclose(y_ori, y)
    y.backward(grad)
    assert th.allclose(A_grad, A.grad, rtol=1e-4) and th.allclose(val.grad, val_grad, rtol=1e-4)
