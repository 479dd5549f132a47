"""Float64 edge-list reference of the graph-attention ops at full size.  TEST / BENCH CHECKER ONLY:
nothing in the product package imports it, and it calls none of the package's kernels.

Same arithmetic as the op-by-op oracle (graphop_oracle.py, which follows graphop_kernel.cu:45-53, 105-110,
123-128, 175-200, 214-228), written with plain torch index ops (index_select, index_add_, scatter_reduce_)
so that it runs on whatever device holds the tensors, in bounded memory: edges are processed in chunks, every
chunk's temporaries are float64 (edges, heads, dim) blocks.  On a GPU the whole R-MAT scale-21 chain, forward
and backward, takes a few seconds; for graphs whose node tensors are too large to hold twice in float64 the
`*_rows` functions compute a sample of rows only.

Graphs are given as plain CSR by destination (indptr, indices) with edge ids equal to CSR positions; the
chunk tables of partition_csr play no role in the arithmetic.
"""
import torch as th

F64 = th.float64


def dst_of_edges(indptr):
    ip = indptr.to(th.int64)
    return th.repeat_interleave(th.arange(ip.numel() - 1, device=ip.device), ip[1:] - ip[:-1])


def _chunks(n, chunk):
    for lo in range(0, n, chunk):
        yield lo, min(n, lo + chunk)


def _edge_scores(Q, K, d, s, scale, rel=None):
    k = K.index_select(0, s).to(F64)
    if rel is not None:              # the node_mul_edge term (graphop_kernel.cu:23-31): one row per edge, all heads
        k = k + rel.to(F64).unsqueeze(1)
    return (Q.index_select(0, d).to(F64) * k).sum(-1) * scale


def attention_f64(indptr, indices, Q, K, V, scale, dO=None, chunk=1 << 20, rel=None):
    """softmax(scale * Q K^T on the edges) V per destination, and its gradients when dO is given.
    rel (E, D), optional: the scores become scale * Q . (K + rel[edge]) - maskedmm plus node_mul_edge.
    Returns (o, lse) or (o, lse, dq, dk, dv) (+ d_rel when rel is given), all float64 on Q's device."""
    dev = Q.device

    def _scores(Q, K, d, s, scale, lo=0, hi=0):   # with the edge term of this chunk, when there is one
        return _edge_scores(Q, K, d, s, scale, None if rel is None else rel[lo:hi])

    n_dst, (h, dd) = Q.shape[0], Q.shape[1:]
    dst = dst_of_edges(indptr.to(dev))
    src = indices.to(dev, th.int64)
    e = src.numel()
    m = th.full((n_dst, h), -float("inf"), dtype=F64, device=dev)
    for lo, hi in _chunks(e, chunk):
        d, s = dst[lo:hi], src[lo:hi]
        m.scatter_reduce_(0, d.view(-1, 1).expand(-1, h), _scores(Q, K, d, s, scale, lo, hi), reduce="amax")
    l = th.zeros(n_dst, h, dtype=F64, device=dev)
    for lo, hi in _chunks(e, chunk):
        d, s = dst[lo:hi], src[lo:hi]
        l.index_add_(0, d, th.exp(_scores(Q, K, d, s, scale, lo, hi) - m.index_select(0, d)))
    lse = m + th.log(l)          # nodes without edges: -inf + log 0 = -inf
    lse_safe = th.where(th.isfinite(lse), lse, th.zeros_like(lse))
    o = th.zeros(n_dst, h, dd, dtype=F64, device=dev)
    for lo, hi in _chunks(e, chunk):
        d, s = dst[lo:hi], src[lo:hi]
        p = th.exp(_scores(Q, K, d, s, scale, lo, hi) - lse_safe.index_select(0, d))
        o.index_add_(0, d, p.unsqueeze(-1) * V.index_select(0, s).to(F64))
    if dO is None:
        return o, lse
    delta = (dO.to(F64) * o).sum(-1)
    dq = th.zeros_like(o)
    dk = th.zeros(K.shape, dtype=F64, device=dev)
    dv = th.zeros(V.shape, dtype=F64, device=dev)
    d_rel = None if rel is None else th.zeros(rel.shape, dtype=F64, device=dev)
    for lo, hi in _chunks(e, chunk):
        d, s = dst[lo:hi], src[lo:hi]
        p = th.exp(_scores(Q, K, d, s, scale, lo, hi) - lse_safe.index_select(0, d))
        g = dO.index_select(0, d).to(F64)
        dp = (g * V.index_select(0, s).to(F64)).sum(-1)
        ds = p * (dp - delta.index_select(0, d)) * scale
        kk = K.index_select(0, s).to(F64)
        qq = Q.index_select(0, d).to(F64)
        if rel is not None:
            kk = kk + rel[lo:hi].to(F64).unsqueeze(1)
            d_rel[lo:hi] = (ds.unsqueeze(-1) * qq).sum(1)     # node_mul_edge's dB (graphop_kernel.cu:79-93)
        dq.index_add_(0, d, ds.unsqueeze(-1) * kk)
        dk.index_add_(0, s, ds.unsqueeze(-1) * qq)
        dv.index_add_(0, s, p.unsqueeze(-1) * g)
    if rel is not None:
        return o, lse, dq, dk, dv, d_rel
    return o, lse, dq, dk, dv


def sddmm_softmax_f64(indptr, indices, Q, K, dP=None, chunk=1 << 20):
    """p = softmax over each destination's edges of (Q . K on the edges), and dQ, dK for an upstream dP.
    Returns (s, p) or (s, p, dq, dk); s and p are (E, H) float64."""
    dev = Q.device
    n_dst, h = Q.shape[0], Q.shape[1]
    dst = dst_of_edges(indptr.to(dev))
    src = indices.to(dev, th.int64)
    e = src.numel()
    s = th.empty(e, h, dtype=F64, device=dev)
    for lo, hi in _chunks(e, chunk):
        s[lo:hi] = _edge_scores(Q, K, dst[lo:hi], src[lo:hi], 1.0)
    m = th.full((n_dst, h), -float("inf"), dtype=F64, device=dev)
    m.scatter_reduce_(0, dst.view(-1, 1).expand(-1, h), s, reduce="amax")
    ex = th.exp(s - m.index_select(0, dst))
    p = ex / th.zeros(n_dst, h, dtype=F64, device=dev).index_add_(0, dst, ex).index_select(0, dst)
    if dP is None:
        return s, p
    g = dP.to(F64)
    agg = th.zeros(n_dst, h, dtype=F64, device=dev).index_add_(0, dst, g * p)
    ds = p * (g - agg.index_select(0, dst))
    dq = th.zeros(Q.shape, dtype=F64, device=dev)
    dk = th.zeros(K.shape, dtype=F64, device=dev)
    for lo, hi in _chunks(e, chunk):
        d, c = dst[lo:hi], src[lo:hi]
        dq.index_add_(0, d, ds[lo:hi].unsqueeze(-1) * K.index_select(0, c).to(F64))
        dk.index_add_(0, c, ds[lo:hi].unsqueeze(-1) * Q.index_select(0, d).to(F64))
    return s, p, dq, dk


def gat_f64(indptr, indices, X, Be, w, dY1, dY2, chunk=1 << 20):
    """node_mul_edge(X, Be) and vector_spmm(w, X) with their gradients.
    Returns (y1 (E,H), y2 (N,H,D), dX (N,H,D), dBe (E,D), dw (E,H)) in float64."""
    dev = X.device
    n, h, dd = X.shape
    dst = dst_of_edges(indptr.to(dev))
    src = indices.to(dev, th.int64)
    e = src.numel()
    y1 = th.empty(e, h, dtype=F64, device=dev)
    dw = th.empty(e, h, dtype=F64, device=dev)
    dbe = th.empty(e, dd, dtype=F64, device=dev)
    y2 = th.zeros(n, h, dd, dtype=F64, device=dev)
    dx = th.zeros(n, h, dd, dtype=F64, device=dev)
    for lo, hi in _chunks(e, chunk):
        d, c = dst[lo:hi], src[lo:hi]
        xd, xs = X.index_select(0, d).to(F64), X.index_select(0, c).to(F64)
        be, ww = Be[lo:hi].to(F64), w[lo:hi].to(F64)
        g1, g2 = dY1[lo:hi].to(F64), dY2.index_select(0, d).to(F64)
        y1[lo:hi] = (xd * be.unsqueeze(1)).sum(-1)
        y2.index_add_(0, d, ww.unsqueeze(-1) * xs)
        dw[lo:hi] = (g2 * xs).sum(-1)
        dbe[lo:hi] = (g1.unsqueeze(-1) * xd).sum(1)
        dx.index_add_(0, d, g1.unsqueeze(-1) * be.unsqueeze(1))      # through node_mul_edge
        dx.index_add_(0, c, ww.unsqueeze(-1) * g2)                   # through vector_spmm
    return y1, y2, dx, dbe, dw


# ------------------------------------------------------------------------------------------------
# sampled rows, for graphs too large for a full float64 copy of the node tensors
# ------------------------------------------------------------------------------------------------
def pick_rows(indptr, count=4000, top=32, seed=0):
    """Row ids to check: the `top` highest-degree rows, up to `top` rows without edges, the first and the
    last row, and random rows up to `count` in all (sorted, unique, int64 on indptr's device)."""
    ip = indptr.to(th.int64)
    n = ip.numel() - 1
    deg = ip[1:] - ip[:-1]
    gen = th.Generator(device="cpu").manual_seed(seed)
    picks = [th.topk(deg, min(top, n)).indices, th.nonzero(deg == 0).flatten()[:top],
             th.tensor([0, n - 1], device=ip.device),
             th.randint(0, n, (count,), generator=gen).to(ip.device)]
    return th.unique(th.cat(picks))[:count]


def edges_of_rows(indptr, rows):
    """(positions, local): CSR positions of all edges of `rows`, and for each the index into `rows`."""
    ip = indptr.to(th.int64)
    lo, deg = ip[rows], ip[rows + 1] - ip[rows]
    local = th.repeat_interleave(th.arange(rows.numel(), device=ip.device), deg)
    start = th.cumsum(deg, 0) - deg
    pos = th.arange(int(deg.sum()), device=ip.device) - start[local] + lo[local]
    return pos, local


def spmm_rows_f64(indptr, indices, eid, w, x, rows, chunk=1 << 20):
    """y[rows] of vector_spmm: sum over a row's positions k of w[eid[k]] * x[indices[k]] (float64).
    `eid` None: the identity."""
    pos, local = edges_of_rows(indptr, rows)
    h, dd = x.shape[1:]
    out = th.zeros(rows.numel(), h, dd, dtype=F64, device=x.device)
    for lo, hi in _chunks(pos.numel(), chunk):
        p = pos[lo:hi]
        e = p if eid is None else eid.index_select(0, p).to(th.int64)
        c = indices.index_select(0, p).to(th.int64)
        out.index_add_(0, local[lo:hi], w.index_select(0, e).to(F64).view(-1, h, 1) * x.index_select(0, c).to(F64))
    return out


def sddmm_rows_f64(indptr, indices, a, b, rows, chunk=1 << 20):
    """(positions, values): a[row] . b[indices[k]] for every position k of `rows` (float64, (n_pos, H))."""
    pos, local = edges_of_rows(indptr, rows)
    h = a.shape[1]
    out = th.empty(pos.numel(), h, dtype=F64, device=a.device)
    for lo, hi in _chunks(pos.numel(), chunk):
        c = indices.index_select(0, pos[lo:hi]).to(th.int64)
        out[lo:hi] = (a.index_select(0, rows[local[lo:hi]]).to(F64) * b.index_select(0, c).to(F64)).sum(-1)
    return pos, out


def max_err(got, want):
    """(largest |got - want| / (1 + |want|), largest |want|) as floats."""
    w = want.to(F64)
    err = ((got.to(F64) - w).abs() / (1.0 + w.abs())).max() if w.numel() else th.zeros((), dtype=F64)
    return float(err), float(w.abs().max()) if w.numel() else 0.0
