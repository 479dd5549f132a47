"""CPU oracle for the graphop sparse graph-attention ops.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this file; only the tests, the smoke
check and the CPU-baseline leg of the benchmark do, and there only as the
checker or the timed baseline.  It restates, in plain torch on the CPU, the
arithmetic of the reference's CUDA kernels (graphop/graphop_kernel.cu) one op
at a time, each function citing the kernel lines it follows.  The kernels'
math is restated, not their scheduling: where the reference accumulates with
atomics in whatever order the hardware picks, the oracle uses `index_add_` in
float64, which is the exact sum up to rounding far below the test tolerance.

Pinning: `partition_csr_loop` is checked against vectors produced by running
the reference's own part_csr.py on the CPU (tests/golden/partition_csr.json),
and the op restatements are checked against (a) the dense torch formulas the
reference's own test script asserts against (wrapper.py:155-481: dense bmm,
th.softmax over the block, th.sparse.mm), and (b) outputs of the reference's
CUDA extension itself, compiled unmodified and run on a B200
(tests/golden/reference_cuda_*.npz, made by oracle/make_reference_golden.py).

Conventions shared with the reference: chunk ``i`` covers CSR positions
``[indptr[i], indptr[i+1])`` of node ``row[i]``; ``eid[k]`` maps a CSR position
to an edge id (the row index into every edge tensor); ``indices[k]`` is the
other endpoint.  ``h == 1`` is spelled as 2-D node tensors ``(n, d)`` and 1-D
edge tensors ``(e,)``.
"""
import torch as th

F64 = th.float64


# ----------------------------------------------------------------------------------------
# integer side
# ----------------------------------------------------------------------------------------
def partition_csr_loop(indptr, chunk_size=32):
    """Pure-Python restatement of partition_csr (part_csr.py:13-27), small inputs only.

    Returns two Python lists ``(row, indptr_)``.
    """
    ip = [int(v) for v in indptr]
    row, out = [], []
    for i in range(len(ip) - 1):
        for j in range(ip[i], ip[i + 1], chunk_size):
            row.append(i)
            out.append(j)
    out.append(ip[-1])
    return row, out


def expand_rows(row, indptr, e):
    """Owner node of every CSR position, -1 where no chunk covers the position.

    Chunk i owns positions [indptr[i], indptr[i+1]) (the loop bounds of every kernel,
    e.g. graphop_kernel.cu:24, 45, 107).
    """
    row = row.to(th.int64).cpu()
    ip = indptr.to(th.int64).cpu()
    out = th.full((e,), -1, dtype=th.int64)
    ln = (ip[1:] - ip[:-1]).clamp(min=0)
    owner = th.repeat_interleave(row, ln)
    start = th.cumsum(ln, 0) - ln
    chunk = th.repeat_interleave(th.arange(row.numel()), ln)
    pos = ip[:-1][chunk] + (th.arange(owner.numel()) - start[chunk])
    out[pos] = owner
    return out


def _covered(row, indptr, eid, e):
    """(positions, owner node, edge id) of every covered CSR position."""
    owner = expand_rows(row, indptr, e)
    pos = th.nonzero(owner >= 0).view(-1)
    return pos, owner[pos], eid.to(th.int64).cpu()[pos]


def _nodes(t):
    """(n, h, d) float64 view of a node tensor given as (n, d) or (n, h, d)."""
    t = t.detach().to("cpu", F64)
    return t.unsqueeze(1) if t.dim() == 2 else t


def _edges(t):
    """(e, h) float64 view of an edge tensor given as (e,) or (e, h)."""
    t = t.detach().to("cpu", F64)
    return t.unsqueeze(1) if t.dim() == 1 else t


def _like_edges(y, h):
    return y.squeeze(1) if h == 1 else y


# ----------------------------------------------------------------------------------------
# the 8 ops
# ----------------------------------------------------------------------------------------
def maskedmm_csr_forward(row, indptr, eid, indices, A, B):
    """y[eid[j], h] = sum_d A[row(j), h, d] * B[indices[j], h, d]  (graphop_kernel.cu:45-53).

    Edge ids no chunk covers keep the zero the launcher allocates (graphop_kernel.cu:284).
    """
    a, b = _nodes(A), _nodes(B)
    e, h = eid.numel(), a.shape[1]
    pos, r, ed = _covered(row, indptr, eid, e)
    c = indices.to(th.int64).cpu()[pos]
    y = th.zeros(e, h, dtype=F64)
    y[ed] = (a[r] * b[c]).sum(-1)
    return _like_edges(y, 1 if A.dim() == 2 else h)


def maskedmm_csr_backward(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B, dy):
    """dA[row] += sum_k dy[eid_r[k]] * B[indices_r[k]] over the row CSR, then the same kernel
    over the column CSR with A in B's place gives dB (graphop_kernel.cu:105-110, 383-407).
    Returns [dA, dB]."""
    a, b, g = _nodes(A), _nodes(B), _edges(dy)
    e = eid_r.numel()
    dA, dB = th.zeros_like(a), th.zeros_like(b)
    pos, r, ed = _covered(row, indptr_r, eid_r, e)
    dA.index_add_(0, r, g[ed].unsqueeze(-1) * b[indices_r.to(th.int64).cpu()[pos]])
    pos, c, ed = _covered(col, indptr_c, eid_c, e)
    dB.index_add_(0, c, g[ed].unsqueeze(-1) * a[indices_c.to(th.int64).cpu()[pos]])
    return [dA.view(A.shape), dB.view(B.shape)]


def node_mul_edge_forward(row, indptr, eid, A, B):
    """y[eid[j], h] = sum_d A[row(j), h, d] * B[eid[j], d]  (graphop_kernel.cu:24-32);
    B is one (e, d) edge tensor shared by all heads."""
    a = _nodes(A)
    be = B.detach().to("cpu", F64)
    e, h = eid.numel(), a.shape[1]
    _, r, ed = _covered(row, indptr, eid, e)
    y = th.zeros(e, h, dtype=F64)
    y[ed] = (a[r] * be[ed].unsqueeze(1)).sum(-1)
    return _like_edges(y, 1 if A.dim() == 2 else h)


def node_mul_edge_backward(row, indptr, eid, A, B, dy):
    """dA[row, h, :] += sum_k dy[eid[k], h] * B[eid[k], :]  (graphop_kernel.cu:66-71) and
    dB[eid[k], :] = sum_h dy[eid[k], h] * A[row, h, :]      (graphop_kernel.cu:84-92).
    Returns [dA, dB]."""
    a, g = _nodes(A), _edges(dy)
    be = B.detach().to("cpu", F64)
    e = eid.numel()
    _, r, ed = _covered(row, indptr, eid, e)
    dA = th.zeros_like(a)
    dA.index_add_(0, r, g[ed].unsqueeze(-1) * be[ed].unsqueeze(1))
    dB = th.zeros_like(be)
    dB[ed] = (g[ed].unsqueeze(-1) * a[r]).sum(1)
    return [dA.view(A.shape), dB]


def sparse_softmax_forward(row, indptr, eid, x):
    """Per (node, head): y = exp(x - max) / sum exp(x - max) over the node's covered
    edges (graphop_kernel.cu:175-176, 186-190, 199-200).  The reference seeds the
    running max with -1e9 (graphop_kernel.cu:428); inputs here stay far above that."""
    xe = _edges(x)
    e, h = xe.shape
    _, r, ed = _covered(row, indptr, eid, e)
    y = th.zeros(e, h, dtype=F64)
    if ed.numel():
        n = int(r.max()) + 1
        xv = xe[ed]
        mx = th.full((n, h), -float("inf"), dtype=F64)
        mx.scatter_reduce_(0, r.view(-1, 1).expand(-1, h), xv, reduce="amax", include_self=True)
        ex = th.exp(xv - mx[r])
        sm = th.zeros(n, h, dtype=F64).index_add_(0, r, ex)
        y[ed] = ex / sm[r]
    return y.view(x.shape)


def sparse_softmax_backward(row, indptr, eid, y, dy):
    """dx = dy*y - (sum_row dy*y) * y  (graphop_kernel.cu:214-217, 226-228)."""
    ye, g = _edges(y), _edges(dy)
    e, h = ye.shape
    _, r, ed = _covered(row, indptr, eid, e)
    dx = th.zeros(e, h, dtype=F64)
    if ed.numel():
        n = int(r.max()) + 1
        agg = th.zeros(n, h, dtype=F64).index_add_(0, r, g[ed] * ye[ed])
        dx[ed] = g[ed] * ye[ed] - agg[r] * ye[ed]
    return dx.view(dy.shape)


def vector_spmm_forward(row, indptr, eid, indices, edata, x, num_dst=None):
    """y[row, h, :] += sum_k edata[eid[k], h] * x[indices[k], h, :]  (graphop_kernel.cu:123-128);
    y has x's shape (graphop_kernel.cu:527), nodes without edges stay zero.  ``num_dst`` gives y
    that many rows instead (destination shards that differ from the source count)."""
    xs, w = _nodes(x), _edges(edata)
    e = eid.numel()
    pos, r, ed = _covered(row, indptr, eid, e)
    n_dst = xs.shape[0] if num_dst is None else num_dst
    y = th.zeros((n_dst,) + tuple(xs.shape[1:]), dtype=F64)
    y.index_add_(0, r, w[ed].unsqueeze(-1) * xs[indices.to(th.int64).cpu()[pos]])
    return y.view((n_dst,) + tuple(x.shape[1:]))


def vector_spmm_backward(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, edata, dy, x):
    """dedata[eid[j], h] = sum_d dy[row(j), h, d] * x[indices[j], h, d]  (graphop_kernel.cu:140-147)
    and dx[col, h, :] += sum_k edata[eid_t[k], h] * dy[indices_t[k], h, :] over the transposed
    CSR (graphop_kernel.cu:156-161).  Every transposed chunk is processed: the reference's
    launch sizes this grid by the row CSR's chunk count (graphop_kernel.cu:566, 588), which
    drops chunks when the transposed CSR has more of them; that defect is not restated.
    Returns [dedata, dx]."""
    xs, g, w = _nodes(x), _nodes(dy), _edges(edata)
    e, h = w.shape
    pos, r, ed = _covered(row, indptr, eid, e)
    ded = th.zeros(e, h, dtype=F64)
    ded[ed] = (g[r] * xs[indices.to(th.int64).cpu()[pos]]).sum(-1)
    pos, c, ed = _covered(col, indptr_t, eid_t, e)
    dx = th.zeros_like(xs)
    dx.index_add_(0, c, w[ed].unsqueeze(-1) * g[indices_t.to(th.int64).cpu()[pos]])
    return [ded.view(edata.shape), dx.view(x.shape)]


# ----------------------------------------------------------------------------------------
# the attention chain
# ----------------------------------------------------------------------------------------
def attention_chain(g_row, g_col, Q, K, V, scale, dO=None):
    """SDDMM(Q, K) * scale -> sparse_softmax -> SpMM(V), composed from the op restatements
    above.  ``g_row = (row, indptr, eid, indices)``, ``g_col`` the same for the transposed
    CSR.  With ``dO`` also returns (dQ, dK, dV) by chaining the backward restatements."""
    row, ip, eid, idx = g_row
    col, ipt, eidt, idxt = g_col
    s = maskedmm_csr_forward(row, ip, eid, idx, Q, K) * scale
    p = sparse_softmax_forward(row, ip, eid, s)
    o = vector_spmm_forward(row, ip, eid, idx, p, V, num_dst=Q.shape[0])
    if dO is None:
        return o
    dp, dV = vector_spmm_backward(row, ip, eid, idx, col, ipt, eidt, idxt, p, dO, V)
    ds = sparse_softmax_backward(row, ip, eid, p, dp) * scale
    dQ, dK = maskedmm_csr_backward(row, ip, eid, idx, col, ipt, eidt, idxt, Q, K, ds)
    return o, dQ, dK, dV


def attention_dense_masked(indptr, indices, Q, K, V, scale, dO=None):
    """Float64 dense-masked attention with autograd: scores on an (h, n, n) grid, -inf
    off the edge set, softmax over sources, matmul with V.  Independent of the edge-list
    code above (it never touches chunks or eid), for graphs without duplicate edges and
    small enough for the dense grid.  Rows with no edge give zero output."""
    q = Q.detach().to("cpu", F64).clone().requires_grad_(True)
    k = K.detach().to("cpu", F64).clone().requires_grad_(True)
    v = V.detach().to("cpu", F64).clone().requires_grad_(True)
    n = q.shape[0]
    ip = indptr.to(th.int64).cpu()
    dst = th.repeat_interleave(th.arange(n), ip[1:] - ip[:-1])
    mask = th.zeros(n, k.shape[0], dtype=th.bool)
    mask[dst, indices.to(th.int64).cpu()] = True
    s = th.einsum("nhd,mhd->hnm", q, k) * scale
    s = s.masked_fill(~mask.unsqueeze(0), -float("inf"))
    p = th.softmax(s, -1)
    p = th.where(mask.unsqueeze(0), p, th.zeros_like(p))  # all-masked rows: nan -> 0
    o = th.einsum("hnm,mhd->nhd", p, v)
    if dO is None:
        return o.detach()
    o.backward(dO.detach().to("cpu", F64))
    return o.detach(), q.grad, k.grad, v.grad
