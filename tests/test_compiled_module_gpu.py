"""The compiled Python module `graphop` (csrc/binding/graphop_module.cpp): the reference's eight functions
(graphop/graphop.cpp:216-225) bound with pybind11 on the C ABI.  Same kernels as the ctypes surface, so the results
must be identical bit for bit; the four autograd Functions of the reference's wrapper.py run on top of it."""
import pytest
import torch as th

from helpers import chunked, graph_zoo
import custom_op_benchmark_b200 as pkg
from custom_op_benchmark_b200 import graphop as mirror, wrapper

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ZOO = graph_zoo()


@pytest.fixture(scope="module")
def compiled():
    return pkg.compiled_graphop()


def test_importable_under_the_reference_name(compiled):
    import graphop
    assert graphop is compiled
    for name in ("maskedmm_csr_forward", "maskedmm_csr_backward", "node_mul_edge_forward", "node_mul_edge_backward",
                 "sparse_softmax_forward", "sparse_softmax_backward", "vector_spmm_forward", "vector_spmm_backward"):
        assert callable(getattr(graphop, name))


@pytest.mark.parametrize("name,g", ZOO, ids=[z[0] for z in ZOO])
@pytest.mark.parametrize("dt,idt", [(th.float32, th.int64), (th.float64, th.int64), (th.bfloat16, th.int32)])
def test_eight_functions_equal_the_ctypes_surface(compiled, name, g, dt, idt):
    r = [t.to(DEV) for t in chunked(g, 32, dtype=idt)]
    c = [t.to(DEV) for t in chunked(g, 32, transposed=True, dtype=idt)]
    h, d, e = 2, 16, g.n_edges
    gen = th.Generator(device=DEV).manual_seed(21)
    rn = lambda *s: th.randn(*s, generator=gen, device=DEV).to(dt)
    A, B, dS, Be = rn(g.n_dst, h, d), rn(g.n_src, h, d), rn(e, h), rn(e, d)
    w = th.rand(e, h, generator=gen, device=DEV).to(dt)
    assert th.equal(compiled.maskedmm_csr_forward(*r, A, B), mirror.maskedmm_csr_forward(*r, A, B))
    for a, b in zip(compiled.maskedmm_csr_backward(*r, *c, A, B, dS), mirror.maskedmm_csr_backward(*r, *c, A, B, dS)):
        assert th.equal(a, b)
    assert th.equal(compiled.node_mul_edge_forward(*r[:3], A, Be), mirror.node_mul_edge_forward(*r[:3], A, Be))
    for a, b in zip(compiled.node_mul_edge_backward(*r[:3], A, Be, dS), mirror.node_mul_edge_backward(*r[:3], A, Be, dS)):
        assert th.equal(a, b)
    p = compiled.sparse_softmax_forward(*r[:3], dS)
    assert th.equal(p, mirror.sparse_softmax_forward(*r[:3], dS))
    assert th.equal(compiled.sparse_softmax_backward(*r[:3], p, w), mirror.sparse_softmax_backward(*r[:3], p, w))
    if g.n_dst == g.n_src:     # the reference's y = zeros_like(x) contract (graphop_kernel.cu:527)
        assert th.equal(compiled.vector_spmm_forward(*r, w, B), mirror.vector_spmm_forward(*r, w, B))
        for a, b in zip(compiled.vector_spmm_backward(*r, *c, w, A, B), mirror.vector_spmm_backward(*r, *c, w, A, B)):
            assert th.equal(a, b)
        o, lse = compiled.attention_forward(r[0], r[1], r[3], A, B, B, 0.25)
        o2, lse2 = mirror.attention_forward(r[0], r[1], r[3], A, B, B, 0.25)
        assert th.equal(o, o2) and th.equal(lse, lse2)
        got = compiled.attention_backward(r[0], r[1], r[3], c[0], c[1], None, c[3], A, B, B, o, lse, A, 0.25)
        want = mirror.attention_backward(r[0], r[1], r[3], c[0], c[1], c[3], A, B, B, o, lse, A, 0.25)
        for a, b in zip(got, want):
            assert th.equal(a, b)


def test_two_dimensional_node_tensors_give_one_dimensional_edge_tensors(compiled):
    g = ZOO[0][1]
    r = [t.to(DEV) for t in chunked(g, 32)]
    A, B = th.randn(g.n_dst, 8, device=DEV), th.randn(g.n_src, 8, device=DEV)
    y = compiled.maskedmm_csr_forward(*r, A, B)
    assert y.shape == (g.n_edges,)
    assert th.equal(y, mirror.maskedmm_csr_forward(*r, A, B))


def test_wrapper_functions_run_on_the_compiled_module(compiled, monkeypatch):
    """The four autograd Functions (wrapper.py:8-55) with the compiled module underneath, forward and backward."""
    g = ZOO[3][1]
    r = [t.to(DEV) for t in chunked(g, 32)]
    c = [t.to(DEV) for t in chunked(g, 32, transposed=True)]
    gen = th.Generator(device=DEV).manual_seed(22)
    Q, K = th.randn(g.n_dst, 2, 16, generator=gen, device=DEV), th.randn(g.n_src, 2, 16, generator=gen, device=DEV)

    def chain(q, k):
        s = wrapper.MaskedMMCSR.apply(*r, *c, q, k)
        return wrapper.SparseSoftmax.apply(*r[:3], s)

    results = []
    for backend in (mirror, compiled):
        monkeypatch.setattr(wrapper, "_g", backend)
        q, k = Q.clone().requires_grad_(True), K.clone().requires_grad_(True)
        p = chain(q, k)
        (p * p).sum().backward()
        results.append((p.detach(), q.grad, k.grad))
    for a, b in zip(*results):
        assert th.equal(a, b)


def test_errors_are_runtime_errors(compiled):
    g = ZOO[0][1]
    r = [t.to(DEV) for t in chunked(g, 32)]
    A, B = th.randn(g.n_dst, 2, 8, device=DEV), th.randn(g.n_src, 2, 8, device=DEV)
    with pytest.raises(RuntimeError, match="CUDA"):
        compiled.maskedmm_csr_forward(*r, A.cpu(), B)
    with pytest.raises(RuntimeError, match="contiguous"):
        compiled.maskedmm_csr_forward(*r, A.transpose(0, 1).contiguous().transpose(0, 1), B)
    with pytest.raises(RuntimeError, match="invalid"):
        compiled.maskedmm_csr_forward(*r, A, B.double())           # mixed element types
    with pytest.raises(RuntimeError, match="not implemented"):
        compiled.maskedmm_csr_forward(*r, A.half(), B.half())
