"""The operator set for any array library that speaks DLPack (include/graphop_dlpack.h).

The reference extension takes torch tensors only and lists "switch backend to dlpack" as its open item
(README.md:5-7).  Every function here takes objects with a ``__dlpack__`` method - torch, CuPy or JAX arrays, or
anything else that exports the capsule - and passes the tensor descriptors inside the capsules straight to the
C ABI, which reads element type, index type and shapes from them.  This module imports no array library.

Nothing is allocated: the caller passes the output tensors and a workspace (a 1-byte-element array of at least
``workspace_bytes(...)`` elements), exactly as on the C side.  ``stream`` is the CUDA stream handle the kernels are
enqueued on (0: the default stream); it is also the stream handed to each producer's ``__dlpack__`` so that the
producer can order its pending work before it.  A non-zero status raises ``RuntimeError``, as the reference's
binding does (graphop.cpp:4-6).
"""
import ctypes

from . import _capi


class _DLDevice(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_int32), ("device_id", ctypes.c_int32)]


class _DLDataType(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint8), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16)]


class DLTensor(ctypes.Structure):
    """dlpack.h's DLTensor, the first member of the DLManagedTensor a "dltensor" capsule points to."""
    _fields_ = [("data", ctypes.c_void_p), ("device", _DLDevice), ("ndim", ctypes.c_int32), ("dtype", _DLDataType),
                ("shape", ctypes.POINTER(ctypes.c_int64)), ("strides", ctypes.POINTER(ctypes.c_int64)),
                ("byte_offset", ctypes.c_uint64)]


_T = ctypes.POINTER(DLTensor)
_get_pointer = ctypes.pythonapi.PyCapsule_GetPointer
_get_pointer.restype = ctypes.c_void_p
_get_pointer.argtypes = [ctypes.py_object, ctypes.c_char_p]

# entry point -> argument kinds: t tensor, i int64, d double (the stream comes last everywhere)
DL_SIGNATURES = {
    "graphop_dl_maskedmm_csr_forward": "tttttttt",
    "graphop_dl_maskedmm_csr_backward": "tttttttttttttt",
    "graphop_dl_node_mul_edge_forward": "ttttttt",
    "graphop_dl_node_mul_edge_backward": "ttttttttt",
    "graphop_dl_sparse_softmax_forward": "tttttit",
    "graphop_dl_sparse_softmax_backward": "ttttttit",
    "graphop_dl_vector_spmm_forward": "tttttttt",
    "graphop_dl_vector_spmm_backward": "tttttttttttttt",
    "graphop_dl_attention_forward": "ttttttdttt",
    "graphop_dl_attention_backward": "tttttttttttttdtttt",
}
_KIND = {"t": _T, "i": ctypes.c_int64, "d": ctypes.c_double}
_bound = {}


def _entry(name):
    fn = _bound.get(name)
    if fn is None:
        fn = getattr(_capi.lib(), name)
        fn.argtypes = [_KIND[k] for k in DL_SIGNATURES[name]] + [ctypes.c_void_p]
        fn.restype = ctypes.c_int
        _bound[name] = fn
    return fn


def _capsule(obj, stream):
    """The object's legacy ("dltensor") capsule.  A CUDA producer gets the consumer's stream as the array API
    standard says (1: the default stream; a handle otherwise); anything else, and producers without the keyword,
    get a plain call (the C side then refuses what is not device memory)."""
    device = getattr(obj, "__dlpack_device__", None)
    if device is not None and int(device()[0]) not in (2, 13):
        return obj.__dlpack__()
    try:
        return obj.__dlpack__(stream=stream if stream else 1)
    except TypeError:
        return obj.__dlpack__()


def _call(name, args, stream):
    keep, c_args = [], []
    for kind, a in zip(DL_SIGNATURES[name], args):
        if kind != "t":
            c_args.append(a)
        elif a is None:
            c_args.append(None)
        else:
            cap = _capsule(a, stream)
            keep.append(cap)             # not consumed: the capsule's own destructor releases the export
            c_args.append(ctypes.cast(_get_pointer(cap, b"dltensor"), _T))
    rc = _entry(name)(*c_args, ctypes.c_void_p(stream or 0))
    del keep
    if rc != _capi.OK:
        raise RuntimeError("%s: %s" % (name, _capi.error_message(rc)))


def workspace_bytes(op, n_edges, n_nodes, heads, dim, elem_bytes, index_bytes):
    """graphop_workspace_bytes: a sufficient workspace size for one call of op (the OP_* ids of _capi)."""
    return int(_capi.lib().graphop_workspace_bytes(op, n_edges, n_nodes, heads, dim, elem_bytes, index_bytes))


def maskedmm_csr_forward(row, indptr, eid, indices, A, B, out, workspace, stream=0):
    """out[eid[k], h] = <A[row(k), h], B[indices[k], h]> (graphop.cpp:16-30 with the output passed in)."""
    _call("graphop_dl_maskedmm_csr_forward", (row, indptr, eid, indices, A, B, out, workspace), stream)


def maskedmm_csr_backward(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B, dy, dA, dB,
                          workspace, stream=0):
    """graphop.cpp:108-131: dA over the row CSR, dB over the column CSR."""
    _call("graphop_dl_maskedmm_csr_backward", (row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B,
                                               dy, dA, dB, workspace), stream)


def node_mul_edge_forward(row, indptr, eid, A, B, out, workspace, stream=0):
    """graphop.cpp:39-51: out[eid[k], h] = <A[row(k), h], B[eid[k]]>."""
    _call("graphop_dl_node_mul_edge_forward", (row, indptr, eid, A, B, out, workspace), stream)


def node_mul_edge_backward(row, indptr, eid, A, B, dy, dA, dB, workspace, stream=0):
    """graphop.cpp:141-154."""
    _call("graphop_dl_node_mul_edge_backward", (row, indptr, eid, A, B, dy, dA, dB, workspace), stream)


def sparse_softmax_forward(row, indptr, eid, x, out, num_nodes, workspace, stream=0):
    """graphop.cpp:59-69; num_nodes bounds node id + 1."""
    _call("graphop_dl_sparse_softmax_forward", (row, indptr, eid, x, out, int(num_nodes), workspace), stream)


def sparse_softmax_backward(row, indptr, eid, y, dy, dx, num_nodes, workspace, stream=0):
    """graphop.cpp:163-175."""
    _call("graphop_dl_sparse_softmax_backward", (row, indptr, eid, y, dy, dx, int(num_nodes), workspace), stream)


def vector_spmm_forward(row, indptr, eid, indices, edata, x, out, workspace, stream=0):
    """graphop.cpp:79-93; out has one row per destination node."""
    _call("graphop_dl_vector_spmm_forward", (row, indptr, eid, indices, edata, x, out, workspace), stream)


def vector_spmm_backward(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, edata, dy, x, dedata, dx,
                         workspace, stream=0):
    """graphop.cpp:190-214."""
    _call("graphop_dl_vector_spmm_backward", (row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, edata, dy, x,
                                              dedata, dx, workspace), stream)


def attention_forward(row, indptr, indices, q, k, v, scale, o, lse, workspace, stream=0):
    """The fused chain maskedmm -> scale -> softmax -> spmm (no reference counterpart as one call)."""
    _call("graphop_dl_attention_forward", (row, indptr, indices, q, k, v, float(scale), o, lse, workspace), stream)


def attention_backward(row, indptr, indices, col, indptr_t, eid_t, indices_t, q, k, v, o, lse, d_o, scale, dq, dk,
                       dv, workspace, stream=0):
    """Gradients of the fused chain; eid_t may be None."""
    _call("graphop_dl_attention_backward", (row, indptr, indices, col, indptr_t, eid_t, indices_t, q, k, v, o, lse,
                                            d_o, float(scale), dq, dk, dv, workspace), stream)
