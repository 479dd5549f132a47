"""The DLPack boundary (include/graphop_dlpack.h, dlpack_ops.py): tensors go in as DLPack capsules, types and
sizes are read from the descriptors, outputs and workspace are the caller's.  Same kernels as the typed entry
points: results are identical bit for bit."""
import pytest
import torch as th

from helpers import chunked, graph_zoo
from custom_op_benchmark_b200 import _capi, dlpack_ops as dl, graphop

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ZOO = graph_zoo()


def _ws(op, g, h, d, dt, idt):
    n = dl.workspace_bytes(op, g.n_edges, max(g.n_dst, g.n_src, g.n_edges), h, d, th.empty(0, dtype=dt).element_size(),
                           th.empty(0, dtype=idt).element_size())
    return th.empty(max(n, 256), dtype=th.uint8, device=DEV)


@pytest.mark.parametrize("name,g", ZOO[:5], ids=[z[0] for z in ZOO[:5]])
@pytest.mark.parametrize("dt,idt", [(th.float32, th.int32), (th.float64, th.int64), (th.bfloat16, th.int64)])
def test_dlpack_entry_points_equal_the_typed_ones(name, g, dt, idt):
    r = [t.to(DEV) for t in chunked(g, 32, dtype=idt)]
    c = [t.to(DEV) for t in chunked(g, 32, transposed=True, dtype=idt)]
    h, d, e = 2, 16, g.n_edges
    gen = th.Generator(device=DEV).manual_seed(31)
    rn = lambda *s: th.randn(*s, generator=gen, device=DEV).to(dt)
    A, B, dS, Be, dY = rn(g.n_dst, h, d), rn(g.n_src, h, d), rn(e, h), rn(e, d), rn(g.n_dst, h, d)
    w = th.rand(e, h, generator=gen, device=DEV).to(dt)
    nan = lambda *s: th.full(s, float("nan"), device=DEV, dtype=dt)
    ws = lambda op: _ws(op, g, h, d, dt, idt)

    y = nan(e, h)
    dl.maskedmm_csr_forward(*r, A, B, y, ws(_capi.OP_MASKEDMM_FWD))
    assert th.equal(y, graphop.maskedmm_csr_forward(*r, A, B))
    dA, dB = nan(g.n_dst, h, d), nan(g.n_src, h, d)
    dl.maskedmm_csr_backward(*r, *c, A, B, dS, dA, dB, ws(_capi.OP_MASKEDMM_BWD))
    for a, b in zip((dA, dB), graphop.maskedmm_csr_backward(*r, *c, A, B, dS)):
        assert th.equal(a, b)
    y = nan(e, h)
    dl.node_mul_edge_forward(*r[:3], A, Be, y, ws(_capi.OP_NODE_MUL_EDGE_FWD))
    assert th.equal(y, graphop.node_mul_edge_forward(*r[:3], A, Be))
    dA, dBe = nan(g.n_dst, h, d), nan(e, d)
    dl.node_mul_edge_backward(*r[:3], A, Be, dS, dA, dBe, ws(_capi.OP_NODE_MUL_EDGE_BWD))
    for a, b in zip((dA, dBe), graphop.node_mul_edge_backward(*r[:3], A, Be, dS)):
        assert th.equal(a, b)
    p = nan(e, h)
    dl.sparse_softmax_forward(*r[:3], dS, p, g.n_dst, ws(_capi.OP_SOFTMAX_FWD))
    assert th.equal(p, graphop.sparse_softmax_forward(*r[:3], dS))
    dx = nan(e, h)
    dl.sparse_softmax_backward(*r[:3], p, w, dx, g.n_dst, ws(_capi.OP_SOFTMAX_BWD))
    assert th.equal(dx, graphop.sparse_softmax_backward(*r[:3], p, w))
    out = nan(g.n_dst, h, d)
    dl.vector_spmm_forward(*r, w, B, out, ws(_capi.OP_SPMM_FWD))
    assert th.equal(out, graphop.vector_spmm_forward(*r, w, B, num_dst=g.n_dst))
    if g.n_dst == g.n_src:
        dw, dX = nan(e, h), nan(g.n_src, h, d)
        dl.vector_spmm_backward(*r, *c, w, dY, B, dw, dX, ws(_capi.OP_SPMM_BWD))
        for a, b in zip((dw, dX), graphop.vector_spmm_backward(*r, *c, w, dY, B)):
            assert th.equal(a, b)
    o, lse = nan(g.n_dst, h, d), th.full((g.n_dst, h), float("nan"), device=DEV,
                                         dtype=th.float64 if dt == th.float64 else th.float32)
    dl.attention_forward(r[0], r[1], r[3], A, B, B, 0.25, o, lse, ws(_capi.OP_ATTENTION_FWD))
    o2, lse2 = graphop.attention_forward(r[0], r[1], r[3], A, B, B, 0.25)
    assert th.equal(o, o2) and th.equal(lse, lse2)
    dq, dk, dv = nan(g.n_dst, h, d), nan(g.n_src, h, d), nan(g.n_src, h, d)
    dl.attention_backward(r[0], r[1], r[3], c[0], c[1], None, c[3], A, B, B, o, lse, dY, 0.25, dq, dk, dv,
                          ws(_capi.OP_ATTENTION_BWD))
    for a, b in zip((dq, dk, dv), graphop.attention_backward(r[0], r[1], r[3], c[0], c[1], c[3], A, B, B, o, lse, dY,
                                                              0.25)):
        assert th.equal(a, b)


def test_identity_edge_ids_and_a_side_stream():
    g = ZOO[1][1]
    r = [t.to(DEV) for t in chunked(g, 32, dtype=th.int32)]
    assert th.equal(r[2], th.arange(g.n_edges, device=DEV, dtype=th.int32))   # the row CSR's edge ids are positions
    A, B = th.randn(g.n_dst, 4, 32, device=DEV), th.randn(g.n_src, 4, 32, device=DEV)
    y = th.full((g.n_edges, 4), float("nan"), device=DEV)
    side = th.cuda.Stream()
    side.wait_stream(th.cuda.current_stream())
    with th.cuda.stream(side):
        dl.maskedmm_csr_forward(r[0], r[1], None, r[3], A, B, y, _ws(_capi.OP_MASKEDMM_FWD, g, 4, 32, th.float32,
                                                                      th.int32), stream=side.cuda_stream)
    side.synchronize()
    assert th.equal(y, graphop.maskedmm_csr_forward(*r, A, B))


def test_what_the_descriptors_say_is_checked_before_any_launch():
    g = ZOO[0][1]
    r = [t.to(DEV) for t in chunked(g, 32, dtype=th.int32)]
    A, B = th.randn(g.n_dst, 2, 8, device=DEV), th.randn(g.n_src, 2, 8, device=DEV)
    y = th.empty(g.n_edges, 2, device=DEV)
    ws = _ws(_capi.OP_MASKEDMM_FWD, g, 2, 8, th.float32, th.int32)
    bad = [
        dict(A=A.double()),                                   # mixed element types
        dict(y=th.empty(g.n_edges + 1, 2, device=DEV)),       # edge count disagrees with indices
        dict(B=th.randn(g.n_src, 2, 9, device=DEV)),          # feature width disagrees
        dict(indices=r[3].long()),                            # mixed index types
        dict(A=th.randn(g.n_dst, 2, 16, device=DEV)[:, :, ::2]),   # not compact
        dict(ws=ws.view(th.int16)),                           # the workspace must have 1-byte elements
    ]
    for change in bad:
        a = dict(row=r[0], indptr=r[1], eid=r[2], indices=r[3], A=A, B=B, y=y, ws=ws)
        a.update(change)
        with pytest.raises(RuntimeError, match="invalid argument"):
            dl.maskedmm_csr_forward(a["row"], a["indptr"], a["eid"], a["indices"], a["A"], a["B"], a["y"], a["ws"])
    th.cuda.synchronize()


class _HandMadeProducer:
    """A DLPack producer that is not an array library: it fills a DLManagedTensor by hand (ctypes) over device memory
    it was given, the way a C program would, and hands out the capsule."""

    class _Managed(__import__("ctypes").Structure):
        pass

    def __init__(self, tensor, code, bits):
        import ctypes
        self._owner = tensor                      # keeps the device memory alive
        self._shape = (ctypes.c_int64 * tensor.dim())(*tensor.shape)
        m = self._Managed
        if not hasattr(m, "_fields_"):
            m._fields_ = [("dl_tensor", dl.DLTensor), ("manager_ctx", ctypes.c_void_p), ("deleter", ctypes.c_void_p)]
        self._managed = m()
        t = self._managed.dl_tensor
        t.data = tensor.data_ptr()
        t.device.device_type, t.device.device_id = 2, tensor.device.index or 0
        t.ndim = tensor.dim()
        t.dtype.code, t.dtype.bits, t.dtype.lanes = code, bits, 1
        t.shape = ctypes.cast(self._shape, ctypes.POINTER(ctypes.c_int64))
        t.strides = None
        t.byte_offset = 0
        self._managed.deleter = None

    def __dlpack_device__(self):
        return (2, self._owner.device.index or 0)

    def __dlpack__(self, stream=None):
        import ctypes
        new = ctypes.pythonapi.PyCapsule_New
        new.restype, new.argtypes = ctypes.py_object, [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
        return new(ctypes.addressof(self._managed), b"dltensor", None)


def test_a_producer_that_is_not_an_array_library():
    g = ZOO[1][1]
    r = [t.to(DEV) for t in chunked(g, 32, dtype=th.int32)]
    h, d = 4, 32
    gen = th.Generator(device=DEV).manual_seed(33)
    w = th.rand(g.n_edges, h, generator=gen, device=DEV)
    x = th.randn(g.n_src, h, d, generator=gen, device=DEV)
    out = th.full((g.n_dst, h, d), float("nan"), device=DEV)
    ws = _ws(_capi.OP_SPMM_FWD, g, h, d, th.float32, th.int32)
    wrap = lambda t, code, bits: _HandMadeProducer(t, code, bits)
    idx = [wrap(t, 0, 32) for t in r]
    dl.vector_spmm_forward(idx[0], idx[1], idx[2], idx[3], wrap(w, 2, 32), wrap(x, 2, 32), wrap(out, 2, 32),
                           wrap(ws, 1, 8))
    assert th.equal(out, graphop.vector_spmm_forward(*r, w, x, num_dst=g.n_dst))
    # what the descriptor says is what counts: the same memory declared as float64 is refused
    with pytest.raises(RuntimeError, match="invalid argument"):
        dl.vector_spmm_forward(idx[0], idx[1], idx[2], idx[3], wrap(w, 2, 64), wrap(x, 2, 32), wrap(out, 2, 32),
                               wrap(ws, 1, 8))
