"""The `graphop` module surface: the eight functions the reference extension exports to
Python (PYBIND11_MODULE at graphop/graphop.cpp:216-225), same names, same positional
arguments, same return shapes and order, plus the fused attention pair.

Each function checks its tensors the way the reference wrappers do (CHECK_INPUT,
graphop.cpp:4-6: every tensor must be a CUDA tensor and contiguous, RuntimeError otherwise),
allocates the outputs and the workspace with torch, and calls the C ABI of
libgraphop_b200.so on the current CUDA stream under a device guard (the reference calls
cudaSetDevice and never restores it, graphop_kernel.cu:242).  There is no CPU path.

Differences from the reference, all supersets: index tensors may be int32 as well as int64
(all of one call's index tensors must share a dtype); bfloat16 is accepted next to float32
and float64; ``dy`` is made contiguous instead of being read unchecked
(graphop.cpp:120-130, 148-153); the source and destination node counts may differ.
"""
import collections
import weakref

import torch as th

from . import _capi

__all__ = [
    "maskedmm_csr_forward", "maskedmm_csr_backward", "node_mul_edge_forward", "node_mul_edge_backward",
    "sparse_softmax_forward", "sparse_softmax_backward", "vector_spmm_forward", "vector_spmm_backward",
    "attention_forward", "attention_backward", "attention_supported", "check_graph", "gather_rows",
    "GraphPlan", "maskedmm_csr_forward_planned", "maskedmm_csr_backward_planned", "vector_spmm_forward_planned",
    "vector_spmm_backward_planned", "sparse_softmax_forward_planned", "sparse_softmax_backward_planned",
    "node_mul_edge_forward_planned", "node_mul_edge_backward_planned", "attention_forward_planned",
    "attention_backward_planned",
]

_ELEM = {th.float32: ("f32", 4), th.float64: ("f64", 8), th.bfloat16: ("bf16", 2)}
_INDEX = {th.int32: ("i32", 4), th.int64: ("i64", 8)}


def _check_input(t, name):
    # graphop.cpp:4-6
    if not t.is_cuda:
        raise RuntimeError("%s must be a CUDA tensor" % name)
    if not t.is_contiguous():
        raise RuntimeError("%s must be contiguous" % name)


def _check_all(**tensors):
    for name, t in tensors.items():
        _check_input(t, name)


def _elem(*ts):
    dt = ts[0].dtype
    if dt not in _ELEM:
        # the text AT_DISPATCH_FLOATING_TYPES raises with (graphop_kernel.cu:254)
        names = {th.float16: "Half", th.int64: "Long", th.int32: "Int", th.uint8: "Byte", th.bool: "Bool"}
        raise RuntimeError('"graphop" not implemented for \'%s\'' % names.get(dt, str(dt).replace("torch.", "")))
    for t in ts:
        if t.dtype != dt:
            raise RuntimeError("expected all floating tensors to share dtype %s, got %s" % (dt, t.dtype))
    return _ELEM[dt]


def _index(*ts):
    dt = ts[0].dtype
    if dt not in _INDEX:
        raise RuntimeError("index tensors must be int32 or int64, got %s" % dt)
    for t in ts:
        if t.dtype != dt:
            raise RuntimeError("expected all index tensors to share dtype %s, got %s" % (dt, t.dtype))
    return _INDEX[dt]


def _chunks(row, indptr):
    c = row.size(0)
    if indptr.size(0) != c + 1:
        raise RuntimeError("indptr must hold row.size(0) + 1 entries")
    return c


def _heads(t, node):
    """(h, d) of a node tensor given as (n, d) / (n, h, d), or h of an edge tensor (e,) / (e, h)."""
    if node:
        if t.dim() not in (2, 3):
            raise RuntimeError("node tensors must be (n, d) or (n, h, d)")
        return (1 if t.dim() == 2 else t.size(1)), t.size(-1)
    if t.dim() not in (1, 2):
        raise RuntimeError("edge tensors must be (e,) or (e, h)")
    return 1 if t.dim() == 1 else t.size(1)


def _p(t):
    return None if t is None else t.data_ptr()


def _call(name, elem, index, op_id, n_edges, n_nodes, h, d, device, args):
    """Allocates the workspace, appends (workspace, bytes, stream) and checks the status."""
    lib = _capi.lib()
    need = lib.graphop_workspace_bytes(op_id, n_edges, n_nodes, h, d, elem[1], index[1])
    ws = th.empty(need + 256, dtype=th.uint8, device=device)
    base = ws.data_ptr()
    aligned = (base + 255) // 256 * 256
    fn = getattr(lib, "graphop_%s_%s_%s" % (name, elem[0], index[0]))
    rc = fn(*args, aligned, need, th.cuda.current_stream(device).cuda_stream)
    if rc != _capi.OK:
        raise RuntimeError("graphop_%s: %s" % (name, _capi.error_message(rc)))


def maskedmm_csr_forward(row, indptr, eid, indices, A, B):
    """y[eid[k], h] = A[row(k), h, :] . B[indices[k], h, :]  ->  (e,) if A is 2-D else (e, h)."""
    _check_all(row=row, indptr=indptr, eid=eid, indices=indices, A=A, B=B)
    elem, index = _elem(A, B), _index(row, indptr, eid, indices)
    h, d = _heads(A, True)
    e, c = eid.size(0), _chunks(row, indptr)
    y = th.empty((e,) if h == 1 else (e, h), dtype=A.dtype, device=A.device)
    with th.cuda.device(A.device):
        _call("maskedmm_csr_forward", elem, index, _capi.OP_MASKEDMM_FWD, e, max(A.size(0), B.size(0)), h, d,
              A.device, [_p(row), _p(indptr), _p(eid), _p(indices), _p(A), _p(B), _p(y), c, e, A.size(0), B.size(0),
                         h, d])
    return y


def maskedmm_csr_backward(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B, dy):
    """[dA, dB] of maskedmm_csr_forward; the row CSR serves dA, the column CSR dB."""
    _check_all(row=row, indptr_r=indptr_r, eid_r=eid_r, indices_r=indices_r, col=col, indptr_c=indptr_c,
               eid_c=eid_c, indices_c=indices_c, A=A, B=B)
    dy = dy.contiguous()
    _check_input(dy, "dy")
    elem = _elem(A, B, dy)
    index = _index(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c)
    h, d = _heads(A, True)
    e, cr, cc = eid_r.size(0), _chunks(row, indptr_r), _chunks(col, indptr_c)
    dA, dB = th.empty_like(A), th.empty_like(B)
    with th.cuda.device(A.device):
        _call("maskedmm_csr_backward", elem, index, _capi.OP_MASKEDMM_BWD, e, max(A.size(0), B.size(0)), h, d,
              A.device, [_p(row), _p(indptr_r), _p(eid_r), _p(indices_r), cr, _p(col), _p(indptr_c), _p(eid_c),
                         _p(indices_c), cc, _p(A), _p(B), _p(dy), _p(dA), _p(dB), e, A.size(0), B.size(0), h, d])
    return [dA, dB]


def node_mul_edge_forward(row, indptr, eid, A, B):
    """y[eid[k], h] = A[row(k), h, :] . B[eid[k], :], B an (e, d) edge tensor shared by the heads."""
    _check_all(row=row, indptr=indptr, eid=eid, A=A, B=B)
    elem, index = _elem(A, B), _index(row, indptr, eid)
    h, d = _heads(A, True)
    e, c = eid.size(0), _chunks(row, indptr)
    y = th.empty((e,) if h == 1 else (e, h), dtype=A.dtype, device=A.device)
    with th.cuda.device(A.device):
        _call("node_mul_edge_forward", elem, index, _capi.OP_NODE_MUL_EDGE_FWD, e, A.size(0), h, d, A.device,
              [_p(row), _p(indptr), _p(eid), _p(A), _p(B), _p(y), c, e, A.size(0), h, d])
    return y


def node_mul_edge_backward(row, indptr, eid, A, B, dy):
    """[dA, dB] of node_mul_edge_forward."""
    _check_all(row=row, indptr=indptr, eid=eid, A=A, B=B)
    dy = dy.contiguous()
    _check_input(dy, "dy")
    elem, index = _elem(A, B, dy), _index(row, indptr, eid)
    h, d = _heads(A, True)
    e, c = eid.size(0), _chunks(row, indptr)
    dA, dB = th.empty_like(A), th.empty_like(B)
    with th.cuda.device(A.device):
        _call("node_mul_edge_backward", elem, index, _capi.OP_NODE_MUL_EDGE_BWD, e, A.size(0), h, d, A.device,
              [_p(row), _p(indptr), _p(eid), _p(A), _p(B), _p(dy), _p(dA), _p(dB), c, e, A.size(0), h, d])
    return [dA, dB]


_NODE_BOUNDS = {}   # id(row tensor) -> (weak reference, version counter, bound)


def _softmax_nodes(row, num_nodes=None):
    """Rows of the per-node statistics the softmax kernels index by node id: largest node id + 1.

    The reference sizes that scratch by the edge count (graphop_kernel.cu:420-427), which wastes memory on
    dense graphs and is too small for a graph whose node ids exceed its edge count.  ``row`` is non-decreasing,
    so its last entry is the largest id: it is read back once per chunk table (a small device-to-host copy
    that waits for the stream) and remembered while the tensor object lives unmodified.  Pass ``num_nodes`` to
    skip the read."""
    if num_nodes is not None:
        return int(num_nodes)
    if row.numel() == 0:
        return 0
    hit = _NODE_BOUNDS.get(id(row))
    if hit is not None and hit[0]() is row and hit[1] == row._version:
        return hit[2]
    bound = int(row[-1].item()) + 1
    if len(_NODE_BOUNDS) >= 256:
        _NODE_BOUNDS.clear()
    _NODE_BOUNDS[id(row)] = (weakref.ref(row), row._version, bound)
    return bound


def sparse_softmax_forward(row, indptr, eid, x, num_nodes=None):
    """Softmax of x over the edges of each node, per head; x is (e,) or (e, h).  ``num_nodes`` (an addition):
    a bound on node id + 1 when the caller knows it."""
    _check_all(row=row, indptr=indptr, eid=eid, x=x)
    elem, index = _elem(x), _index(row, indptr, eid)
    h = _heads(x, False)
    e, c = eid.size(0), _chunks(row, indptr)
    y = th.empty_like(x)
    n = _softmax_nodes(row, num_nodes)
    with th.cuda.device(x.device):
        _call("sparse_softmax_forward", elem, index, _capi.OP_SOFTMAX_FWD, e, n, h, 1, x.device,
              [_p(row), _p(indptr), _p(eid), _p(x), _p(y), c, e, n, h])
    return y


def sparse_softmax_backward(row, indptr, eid, y, dy, num_nodes=None):
    """dx = y * (dy - sum over the node of dy * y)."""
    _check_all(row=row, indptr=indptr, eid=eid, y=y, dy=dy)
    elem, index = _elem(y, dy), _index(row, indptr, eid)
    h = _heads(dy, False)
    e, c = eid.size(0), _chunks(row, indptr)
    dx = th.empty_like(dy)
    n = _softmax_nodes(row, num_nodes)
    with th.cuda.device(y.device):
        _call("sparse_softmax_backward", elem, index, _capi.OP_SOFTMAX_BWD, e, n, h, 1, y.device,
              [_p(row), _p(indptr), _p(eid), _p(y), _p(dy), _p(dx), c, e, n, h])
    return dx


def vector_spmm_forward(row, indptr, eid, indices, edata, x, num_dst=None):
    """y[n, h, :] = sum over n's edges of edata[eid[k], h] * x[indices[k], h, :].

    ``y`` has x's shape as in the reference (graphop_kernel.cu:527); ``num_dst`` (an addition)
    gives it that many rows instead, for a shard that owns fewer destinations than sources."""
    _check_all(row=row, indptr=indptr, eid=eid, indices=indices, edata=edata, x=x)
    elem, index = _elem(edata, x), _index(row, indptr, eid, indices)
    h, d = _heads(x, True)
    if _heads(edata, False) != h:
        raise RuntimeError("edata and x disagree on the number of heads")
    e, c = eid.size(0), _chunks(row, indptr)
    n_dst = x.size(0) if num_dst is None else int(num_dst)
    y = th.empty((n_dst,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    with th.cuda.device(x.device):
        _call("vector_spmm_forward", elem, index, _capi.OP_SPMM_FWD, e, max(n_dst, x.size(0)), h, d, x.device,
              [_p(row), _p(indptr), _p(eid), _p(indices), _p(edata), _p(x), _p(y), c, e, n_dst, x.size(0), h, d])
    return y


def vector_spmm_backward(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, edata, dy, x):
    """[dedata, dx] of vector_spmm_forward (this order: graphop_kernel.cu:599)."""
    _check_all(row=row, indptr=indptr, eid=eid, indices=indices, col=col, indptr_t=indptr_t, eid_t=eid_t,
               indices_t=indices_t, edata=edata, dy=dy, x=x)
    elem = _elem(edata, dy, x)
    index = _index(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t)
    h, d = _heads(x, True)
    e, c, ct = eid.size(0), _chunks(row, indptr), _chunks(col, indptr_t)
    dedata, dx = th.empty_like(edata), th.empty_like(x)
    with th.cuda.device(x.device):
        _call("vector_spmm_backward", elem, index, _capi.OP_SPMM_BWD, e, max(dy.size(0), x.size(0)), h, d, x.device,
              [_p(row), _p(indptr), _p(eid), _p(indices), c, _p(col), _p(indptr_t), _p(eid_t), _p(indices_t), ct,
               _p(edata), _p(dy), _p(x), _p(dedata), _p(dx), e, dy.size(0), x.size(0), h, d])
    return [dedata, dx]


# ------------------------------------------------------------------------------------------
# fused attention (an addition: one call for maskedmm -> scale -> sparse_softmax -> vector_spmm)
# ------------------------------------------------------------------------------------------
def attention_supported(q):
    """Shapes the fused kernels take: D * itemsize a power-of-two multiple of 16 bytes, a node
    row of at most 4 KiB, 16-byte aligned storage."""
    if q.dtype not in _ELEM or q.dim() not in (2, 3):
        return False
    h, d = _heads(q, True)
    v = 16 // q.element_size()
    if d % v or (d // v) & (d // v - 1):
        return False
    return h * d // v <= 256 and q.data_ptr() % 16 == 0


def _lse_dtype(q):
    return th.float64 if q.dtype == th.float64 else th.float32


def attention_forward(row, indptr, indices, q, k, v, scale):
    """(o, lse): o[n] = sum_k softmax_k(scale * q[n].k[indices[k]]) v[indices[k]] over n's edges,
    lse[n, h] the log of the softmax denominator (kept for the backward)."""
    _check_all(row=row, indptr=indptr, indices=indices, q=q, k=k, v=v)
    elem, index = _elem(q, k, v), _index(row, indptr, indices)
    h, d = _heads(q, True)
    e, c = indices.size(0), _chunks(row, indptr)
    o = th.empty_like(q)
    lse = th.empty((q.size(0), h), dtype=_lse_dtype(q), device=q.device)
    if e == 0:
        return o.zero_(), lse.fill_(float("-inf"))
    with th.cuda.device(q.device):
        _call("attention_forward", elem, index, _capi.OP_ATTENTION_FWD, e, max(q.size(0), k.size(0)), h, d,
              q.device, [_p(row), _p(indptr), _p(indices), c, _p(q), _p(k), _p(v), float(scale), _p(o), _p(lse), e,
                         q.size(0), k.size(0), h, d])
    return o, lse


def attention_backward(row, indptr, indices, col, indptr_t, indices_t, q, k, v, o, lse, d_o, scale, eid_t=None):
    """[dq, dk, dv] of attention_forward; probabilities are recomputed from q, k and lse.

    ``eid_t`` (optional): for every position of the transposed CSR the position of the same edge in the row
    CSR, i.e. the transposed CSR's edge ids when the row CSR's are 0..e-1.  With it the destination pass
    keeps (p, ds) per edge (2 * e * h accumulator-sized values of workspace) and the source pass does not
    recompute them."""
    d_o = d_o.contiguous()
    _check_all(row=row, indptr=indptr, indices=indices, col=col, indptr_t=indptr_t, indices_t=indices_t, q=q, k=k,
               v=v, o=o, lse=lse, d_o=d_o)
    elem = _elem(q, k, v, o, d_o)
    if eid_t is not None:
        _check_all(eid_t=eid_t)
        index = _index(row, indptr, indices, col, indptr_t, indices_t, eid_t)
    else:
        index = _index(row, indptr, indices, col, indptr_t, indices_t)
    h, d = _heads(q, True)
    e, c, ct = indices.size(0), _chunks(row, indptr), _chunks(col, indptr_t)
    dq, dk, dv = th.empty_like(q), th.empty_like(k), th.empty_like(v)
    if e == 0:
        return [dq.zero_(), dk.zero_(), dv.zero_()]
    with th.cuda.device(q.device):
        op_id = _capi.OP_ATTENTION_BWD if eid_t is None else _capi.OP_ATTENTION_BWD_PAIRS
        _call("attention_backward", elem, index, op_id, e, max(q.size(0), k.size(0)), h, d,
              q.device, [_p(row), _p(indptr), _p(indices), c, _p(col), _p(indptr_t), _p(eid_t), _p(indices_t), ct, _p(q),
                         _p(k), _p(v), _p(o), _p(lse), _p(d_o), float(scale), _p(dq), _p(dk), _p(dv), e, q.size(0),
                         k.size(0), h, d])
    return [dq, dk, dv]


def attention_bias_forward(row, indptr, indices, q, k, v, rel, scale):
    """attention_forward with an edge term in the scores: s = scale * q[n].(k[indices[j]] + rel[j]), rel an (e, d)
    tensor indexed by row-CSR position and shared by the heads - the reference's node_mul_edge ("designed for
    relative positional encoding", graphop_kernel.cu:16-34) added to maskedmm's scores inside the fused pass."""
    _check_all(row=row, indptr=indptr, indices=indices, q=q, k=k, v=v, rel=rel)
    elem, index = _elem(q, k, v, rel), _index(row, indptr, indices)
    h, d = _heads(q, True)
    e, c = indices.size(0), _chunks(row, indptr)
    if rel.dim() != 2 or rel.size(0) != e or rel.size(1) != d:
        raise RuntimeError("rel must be (e, d)")
    o = th.empty_like(q)
    lse = th.empty((q.size(0), h), dtype=_lse_dtype(q), device=q.device)
    if e == 0:
        return o.zero_(), lse.fill_(float("-inf"))
    with th.cuda.device(q.device):
        _call("attention_bias_forward", elem, index, _capi.OP_ATTENTION_FWD, e, max(q.size(0), k.size(0)), h, d,
              q.device, [_p(row), _p(indptr), _p(indices), c, _p(q), _p(k), _p(v), _p(rel), float(scale), _p(o),
                         _p(lse), e, q.size(0), k.size(0), h, d])
    return o, lse


def attention_bias_backward(row, indptr, indices, col, indptr_t, eid_t, indices_t, q, k, v, rel, o, lse, d_o, scale):
    """[dq, dk, dv, d_rel] of attention_bias_forward.  eid_t: for every position of the transposed CSR the position
    of the same edge in the row CSR (required: the row pass hands (p, ds) of every edge to the other passes)."""
    d_o = d_o.contiguous()
    _check_all(row=row, indptr=indptr, indices=indices, col=col, indptr_t=indptr_t, eid_t=eid_t, indices_t=indices_t,
               q=q, k=k, v=v, rel=rel, o=o, lse=lse, d_o=d_o)
    elem = _elem(q, k, v, rel, o, d_o)
    index = _index(row, indptr, indices, col, indptr_t, indices_t, eid_t)
    h, d = _heads(q, True)
    e, c, ct = indices.size(0), _chunks(row, indptr), _chunks(col, indptr_t)
    dq, dk, dv, d_rel = th.empty_like(q), th.empty_like(k), th.empty_like(v), th.empty_like(rel)
    if e == 0:
        return [dq.zero_(), dk.zero_(), dv.zero_(), d_rel]
    with th.cuda.device(q.device):
        _call("attention_bias_backward", elem, index, _capi.OP_ATTENTION_BWD_PAIRS, e, max(q.size(0), k.size(0)), h,
              d, q.device, [_p(row), _p(indptr), _p(indices), c, _p(col), _p(indptr_t), _p(eid_t), _p(indices_t), ct,
                            _p(q), _p(k), _p(v), _p(rel), _p(o), _p(lse), _p(d_o), float(scale), _p(dq), _p(dk),
                            _p(dv), _p(d_rel), e, q.size(0), k.size(0), h, d])
    return [dq, dk, dv, d_rel]


def gather_rows(table, idx, out=None):
    """out[r] = table[idx[r]] (rows of a contiguous CUDA tensor, int32 or int64 row ids; 16-byte multiples go
    through the library's copy kernel, anything else through torch)."""
    _check_all(table=table, idx=idx)
    row_bytes = (table[0].numel() if table.size(0) else 0) * table.element_size()
    if out is None:
        out = th.empty((idx.numel(),) + tuple(table.shape[1:]), dtype=table.dtype, device=table.device)
    if idx.numel() == 0:
        return out
    if row_bytes == 0 or row_bytes % 16 or table.data_ptr() % 16 or out.data_ptr() % 16 or not out.is_contiguous() \
            or table.size(0) >= 2 ** 31:
        return th.index_select(table, 0, idx.long(), out=out)
    idx32 = idx if idx.dtype == th.int32 else idx.to(th.int32)
    with th.cuda.device(table.device):
        rc = _capi.lib().graphop_gather_rows_i32(_p(idx32), idx32.numel(), _p(table), row_bytes, _p(out),
                                                 th.cuda.current_stream(table.device).cuda_stream)
    if rc != _capi.OK:
        raise RuntimeError("graphop_gather_rows: %s" % _capi.error_message(rc))
    return out


def pull_rows(tables, seg, idx, row_bytes, out):
    """out[r] = table_p[idx[r]] for the rows r of segment p (seg[p] <= r < seg[p + 1]); `tables` are device addresses
    (ints) of row blocks on this and on peer GPUs, mapped into this process.  One kernel of plain peer loads
    (graphop_pull_rows_i32); the caller orders it after the owners' writes."""
    import ctypes
    n = len(tables)
    if len(seg) != n + 1:
        raise RuntimeError("seg must hold one more entry than tables")
    _check_all(idx=idx, out=out)
    if idx.dtype != th.int32:
        raise RuntimeError("idx must be int32")
    tabs = (ctypes.c_void_p * n)(*[ctypes.c_void_p(int(t)) for t in tables])
    segs = (ctypes.c_int64 * (n + 1))(*[int(s) for s in seg])
    with th.cuda.device(out.device):
        rc = _capi.lib().graphop_pull_rows_i32(tabs, segs, n, _p(idx), int(row_bytes), _p(out),
                                               th.cuda.current_stream(out.device).cuda_stream)
    if rc != _capi.OK:
        raise RuntimeError("graphop_pull_rows: %s" % _capi.error_message(rc))
    return out


def partition_csr(indptr, chunk_size=32):
    """partition_csr of the reference (part_csr.py:13-27) for an int32 / int64 indptr on a CUDA device, by the
    library's kernels (graphop_partition_csr_count / _fill): (row, indptr_) as int64 tensors on that device."""
    import ctypes
    if chunk_size <= 0:
        raise ValueError("chunk_size must be positive")
    if not indptr.is_cuda or indptr.dtype not in (th.int32, th.int64) or indptr.dim() != 1:
        raise RuntimeError("indptr must be a one-dimensional int32 or int64 CUDA tensor")
    if indptr.numel() < 1:
        raise IndexError("indptr must hold at least one element")
    ip = indptr.contiguous()
    n = ip.numel() - 1
    suffix = "i32" if ip.dtype == th.int32 else "i64"
    lib = _capi.lib()
    with th.cuda.device(ip.device):
        stream = th.cuda.current_stream(ip.device).cuda_stream
        ws = th.empty(lib.graphop_partition_csr_workspace_bytes(n), dtype=th.uint8, device=ip.device)
        count = ctypes.c_int64(0)
        rc = getattr(lib, "graphop_partition_csr_count_" + suffix)(
            _p(ip), n, int(chunk_size), _p(ws), ws.numel(), ctypes.byref(count), stream)
        if rc != _capi.OK:
            raise RuntimeError("graphop_partition_csr_count: %s" % _capi.error_message(rc))
        row = th.empty(count.value, dtype=th.int64, device=ip.device)
        ptr = th.empty(count.value + 1, dtype=th.int64, device=ip.device)
        rc = getattr(lib, "graphop_partition_csr_fill_" + suffix)(
            _p(ip), n, int(chunk_size), _p(ws), count.value, _p(row), _p(ptr), stream)
        if rc != _capi.OK:
            raise RuntimeError("graphop_partition_csr_fill: %s" % _capi.error_message(rc))
    return row, ptr


def transpose_csr(indptr, indices, n_src):
    """(indptr_t, indices_t, eid_t) of a row CSR on a CUDA device whose edge ids are its positions, in the inputs'
    integer type (int32 or int64, the same for both): edges regrouped by source, ties in row-CSR order.  The
    library's kernels (graphop_transpose_csr): a stable radix sort of the positions by source and one fill pass."""
    if not (indptr.is_cuda and indices.is_cuda) or indptr.dtype != indices.dtype or \
            indptr.dtype not in (th.int32, th.int64) or indptr.dim() != 1 or indices.dim() != 1:
        raise RuntimeError("indptr and indices must be one-dimensional CUDA tensors of the same type, int32 or int64")
    if indptr.numel() < 1:
        raise IndexError("indptr must hold at least one element")
    ip, idx = indptr.contiguous(), indices.contiguous()
    n_dst, e, n_src = ip.numel() - 1, idx.numel(), int(n_src)
    suffix, width = ("i32", 4) if ip.dtype == th.int32 else ("i64", 8)
    lib = _capi.lib()
    with th.cuda.device(ip.device):
        ws = th.empty(lib.graphop_transpose_csr_workspace_bytes(e, width), dtype=th.uint8, device=ip.device)
        ptr_t = th.empty(n_src + 1, dtype=ip.dtype, device=ip.device)
        idx_t, eid_t = th.empty_like(idx), th.empty_like(idx)
        rc = getattr(lib, "graphop_transpose_csr_" + suffix)(
            _p(ip), _p(idx), n_dst, n_src, e, _p(ptr_t), _p(idx_t), _p(eid_t), _p(ws), ws.numel(),
            th.cuda.current_stream(ip.device).cuda_stream)
    if rc != _capi.OK:
        raise RuntimeError("graphop_transpose_csr: %s" % _capi.error_message(rc))
    return ptr_t, idx_t, eid_t


def check_graph(row, indptr, eid, indices, n_nodes, n_other):
    """Debug aid: verifies on the device the graph contract the kernels rely on (monotone
    indptr and row, indices and edge ids in range) and returns the violation bit mask
    (0 = fine).  Synchronises the stream."""
    import ctypes
    _check_all(row=row, indptr=indptr)
    index = _index(row, indptr)
    e = eid.size(0) if eid is not None else (indices.size(0) if indices is not None else 0)
    flags = ctypes.c_int(0)
    fn = getattr(_capi.lib(), "graphop_check_graph_%s" % index[0])
    with th.cuda.device(row.device):
        rc = fn(_p(row), _p(indptr), _p(eid), _p(indices), row.size(0), e, n_nodes, n_other, ctypes.byref(flags),
                th.cuda.current_stream(row.device).cuda_stream)
    if rc not in (_capi.OK, _capi.ERR_INVALID_ARGUMENT):
        raise RuntimeError("graphop_check_graph: %s" % _capi.error_message(rc))
    return flags.value


# ------------------------------------------------------------------------------------------
# graph plans (an addition): what the ops rebuild from the index tensors on every call, built once
# ------------------------------------------------------------------------------------------
class GraphPlan:
    """One CSR orientation prepared once: the owner node of every position, 32-bit copies of int64 index tensors,
    per-node ranges and the shape flags (``dense_band``).  The reference prepares its graphs on the host in Python
    loops before any op runs (part_csr.py:18-21, wrapper.py:93-112); this is that step for the kernels here, on
    the device.  Building a plan waits for the device once; the ``*_planned`` ops then take the plan in place
    of ``(row, indptr, eid, indices)`` and skip the per-call expansion.

    ``indices`` may be None for ops without a second endpoint (sparse_softmax, node_mul_edge), ``eid`` None for
    the identity.  The plan keeps the index tensors it refers to alive."""

    def __init__(self, row, indptr, eid, indices, n_nodes):
        import ctypes
        given = dict(row=row, indptr=indptr)
        if eid is not None:
            given["eid"] = eid
        if indices is not None:
            given["indices"] = indices
        _check_all(**given)
        index = _index(*given.values())
        self.n_chunks, self.n_nodes = _chunks(row, indptr), int(n_nodes)
        self.n_edges = int(indices.size(0) if indices is not None else (eid.size(0) if eid is not None else 0))
        if eid is not None and indices is not None and eid.size(0) != indices.size(0):
            raise RuntimeError("eid and indices disagree on the number of edges")
        self.device = row.device
        lib = _capi.lib()
        need = lib.graphop_plan_bytes(self.n_chunks, self.n_edges, self.n_nodes, index[1])
        self._memory = th.empty(need + 256, dtype=th.uint8, device=self.device)
        base = (self._memory.data_ptr() + 255) // 256 * 256
        self._keep = (row, indptr, eid, indices)
        self.c = _capi.Plan()
        fn = getattr(lib, "graphop_plan_build_%s" % index[0])
        with th.cuda.device(self.device):
            rc = fn(_p(row), _p(indptr), _p(eid), _p(indices), self.n_chunks, self.n_edges, self.n_nodes, base, need,
                    ctypes.byref(self.c), th.cuda.current_stream(self.device).cuda_stream)
        if rc != _capi.OK:
            raise RuntimeError("graphop_plan_build: %s" % _capi.error_message(rc))

    @property
    def dense_band(self):
        return bool(self.c.flags & _capi.PLAN_DENSE_BAND)

    @property
    def band_span(self):
        return int(self.c.band_span)

    @property
    def no_carry(self):
        """No node's positions cross a (row-aligned) work-tile boundary: the planned row-reducing ops are one
        launch each on this graph."""
        return bool(self.c.flags & _capi.PLAN_NO_CARRY)

    def ref(self):
        import ctypes
        return ctypes.byref(self.c)


plan_cache_size = 8      # plans kept by cached_plan(); 0 switches the cache off
_PLAN_CACHE = collections.OrderedDict()


def cached_plan(row, indptr, eid, indices, n_nodes):
    """The GraphPlan of these index tensors, built on first use and kept while the same tensor objects come back
    unmodified (identity and torch's version counter; the most recent ``plan_cache_size`` plans are kept).  This is
    what lets the entry points that take (row, indptr, eid, indices) per call - the reference's calling convention -
    run at the speed of the planned ones: a training loop passes the same graph tensors every step."""
    tensors = (row, indptr, eid, indices)
    if plan_cache_size <= 0:
        return GraphPlan(row, indptr, eid, indices, n_nodes)
    key = tuple((id(t), t._version) if t is not None else None for t in tensors) + (int(n_nodes),)
    hit = _PLAN_CACHE.get(key)
    if hit is not None and all(a is b for a, b in zip(hit._keep, tensors)):
        _PLAN_CACHE.move_to_end(key)
        return hit
    plan = GraphPlan(row, indptr, eid, indices, n_nodes)
    _PLAN_CACHE[key] = plan
    while len(_PLAN_CACHE) > plan_cache_size:
        _PLAN_CACHE.popitem(last=False)
    return plan


def _call_planned(name, elem, op_id, plans, n_nodes, h, d, device, args):
    lib = _capi.lib()
    need = lib.graphop_workspace_bytes(op_id, plans[0].n_edges, n_nodes, h, d, elem[1], 4)
    ws = th.empty(need + 256, dtype=th.uint8, device=device)
    aligned = (ws.data_ptr() + 255) // 256 * 256
    fn = getattr(lib, "graphop_%s_planned_%s" % (name, elem[0]))
    rc = fn(*[p.ref() for p in plans], *args, aligned, need, th.cuda.current_stream(device).cuda_stream)
    if rc != _capi.OK:
        raise RuntimeError("graphop_%s_planned: %s" % (name, _capi.error_message(rc)))


def maskedmm_csr_forward_planned(plan, A, B):
    _check_all(A=A, B=B)
    elem = _elem(A, B)
    h, d = _heads(A, True)
    y = th.empty((plan.n_edges,) if h == 1 else (plan.n_edges, h), dtype=A.dtype, device=A.device)
    with th.cuda.device(A.device):
        _call_planned("maskedmm_csr_forward", elem, _capi.OP_MASKEDMM_FWD, [plan], max(A.size(0), B.size(0)), h, d,
                      A.device, [_p(A), _p(B), _p(y), A.size(0), B.size(0), h, d])
    return y


def maskedmm_csr_backward_planned(plan_r, plan_c, A, B, dy):
    dy = dy.contiguous()
    _check_all(A=A, B=B, dy=dy)
    elem = _elem(A, B, dy)
    h, d = _heads(A, True)
    dA, dB = th.empty_like(A), th.empty_like(B)
    with th.cuda.device(A.device):
        _call_planned("maskedmm_csr_backward", elem, _capi.OP_MASKEDMM_BWD, [plan_r, plan_c],
                      max(A.size(0), B.size(0)), h, d, A.device,
                      [_p(A), _p(B), _p(dy), _p(dA), _p(dB), A.size(0), B.size(0), h, d])
    return [dA, dB]


def node_mul_edge_forward_planned(plan, A, B):
    _check_all(A=A, B=B)
    elem = _elem(A, B)
    h, d = _heads(A, True)
    y = th.empty((plan.n_edges,) if h == 1 else (plan.n_edges, h), dtype=A.dtype, device=A.device)
    with th.cuda.device(A.device):
        _call_planned("node_mul_edge_forward", elem, _capi.OP_NODE_MUL_EDGE_FWD, [plan], A.size(0), h, d, A.device,
                      [_p(A), _p(B), _p(y), A.size(0), h, d])
    return y


def node_mul_edge_backward_planned(plan, A, B, dy):
    dy = dy.contiguous()
    _check_all(A=A, B=B, dy=dy)
    elem = _elem(A, B, dy)
    h, d = _heads(A, True)
    dA, dB = th.empty_like(A), th.empty_like(B)
    with th.cuda.device(A.device):
        _call_planned("node_mul_edge_backward", elem, _capi.OP_NODE_MUL_EDGE_BWD, [plan], A.size(0), h, d, A.device,
                      [_p(A), _p(B), _p(dy), _p(dA), _p(dB), A.size(0), h, d])
    return [dA, dB]


def sparse_softmax_forward_planned(plan, x):
    _check_all(x=x)
    elem, h = _elem(x), _heads(x, False)
    y = th.empty_like(x)
    with th.cuda.device(x.device):
        _call_planned("sparse_softmax_forward", elem, _capi.OP_SOFTMAX_FWD, [plan], plan.n_nodes, h, 1, x.device,
                      [_p(x), _p(y), h])
    return y


def sparse_softmax_backward_planned(plan, y, dy):
    _check_all(y=y, dy=dy)
    elem, h = _elem(y, dy), _heads(dy, False)
    dx = th.empty_like(dy)
    with th.cuda.device(y.device):
        _call_planned("sparse_softmax_backward", elem, _capi.OP_SOFTMAX_BWD, [plan], plan.n_nodes, h, 1, y.device,
                      [_p(y), _p(dy), _p(dx), h])
    return dx


def vector_spmm_forward_planned(plan, edata, x, num_dst=None):
    _check_all(edata=edata, x=x)
    elem = _elem(edata, x)
    h, d = _heads(x, True)
    n_dst = x.size(0) if num_dst is None else int(num_dst)
    y = th.empty((n_dst,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    with th.cuda.device(x.device):
        _call_planned("vector_spmm_forward", elem, _capi.OP_SPMM_FWD, [plan], max(n_dst, x.size(0)), h, d, x.device,
                      [_p(edata), _p(x), _p(y), n_dst, x.size(0), h, d])
    return y


def vector_spmm_backward_planned(plan_r, plan_t, edata, dy, x):
    _check_all(edata=edata, dy=dy, x=x)
    elem = _elem(edata, dy, x)
    h, d = _heads(x, True)
    dedata, dx = th.empty_like(edata), th.empty_like(x)
    with th.cuda.device(x.device):
        _call_planned("vector_spmm_backward", elem, _capi.OP_SPMM_BWD, [plan_r, plan_t], max(dy.size(0), x.size(0)),
                      h, d, x.device, [_p(edata), _p(dy), _p(x), _p(dedata), _p(dx), dy.size(0), x.size(0), h, d])
    return [dedata, dx]


def attention_forward_planned(plan, q, k, v, scale):
    """attention_forward on a plan of the row CSR; a dense-band graph with bfloat16 tensors of 64 features per
    head runs on the tensor cores."""
    _check_all(q=q, k=k, v=v)
    elem = _elem(q, k, v)
    h, d = _heads(q, True)
    o = th.empty_like(q)
    lse = th.empty((q.size(0), h), dtype=_lse_dtype(q), device=q.device)
    if plan.n_edges == 0:
        return o.zero_(), lse.fill_(float("-inf"))
    with th.cuda.device(q.device):
        _call_planned("attention_forward", elem, _capi.OP_ATTENTION_FWD, [plan], max(q.size(0), k.size(0)), h, d,
                      q.device, [_p(q), _p(k), _p(v), float(scale), _p(o), _p(lse), q.size(0), k.size(0), h, d])
    return o, lse


def attention_backward_planned(plan_r, plan_t, q, k, v, o, lse, d_o, scale):
    """attention_backward on plans of both CSR orientations (plan_t built with the transposed CSR's edge ids lets
    the row pass hand every edge's probability to the transposed pass)."""
    d_o = d_o.contiguous()
    _check_all(q=q, k=k, v=v, o=o, lse=lse, d_o=d_o)
    elem = _elem(q, k, v, o, d_o)
    h, d = _heads(q, True)
    dq, dk, dv = th.empty_like(q), th.empty_like(k), th.empty_like(v)
    if plan_r.n_edges == 0:
        return [dq.zero_(), dk.zero_(), dv.zero_()]
    with th.cuda.device(q.device):
        op_id = _capi.OP_ATTENTION_BWD_PAIRS if plan_t.c.eid else _capi.OP_ATTENTION_BWD
        _call_planned("attention_backward", elem, op_id, [plan_r, plan_t], max(q.size(0), k.size(0)), h, d, q.device,
                      [_p(q), _p(k), _p(v), _p(o), _p(lse), _p(d_o), float(scale), _p(dq), _p(dk), _p(dv), q.size(0),
                       k.size(0), h, d])
    return [dq, dk, dv]
