"""Torch CPU implementation of the attention chain, the timed CPU baseline.  TEST / BENCH
INFRASTRUCTURE ONLY: nothing in the product package imports it.

Same arithmetic as the op-by-op oracle (graphop_oracle.py), written for speed on the host
cores instead of for float64 exactness: float32, gathers with index_select, per-node
reductions with scatter_reduce / index_add_, the backward through torch autograd, destination
nodes processed in blocks so that the (edges, heads, dim) temporaries stay bounded.
"""
import time

import torch as th


def attention_chain_cpu(indptr, indices, Q, K, V, scale, dO, rows_per_block=1 << 15, rel=None):
    """Forward and backward of SDDMM(Q, K) * scale -> softmax per destination -> SpMM(V) on the
    CPU.  Returns (O, dQ, dK, dV).  rel (edges, dim), optional: the node_mul_edge term added to the scores
    (its gradient is computed and dropped)."""
    ip = indptr.to("cpu", th.int64)
    idx = indices.to("cpu", th.int64)
    n, h, d = Q.shape
    q = Q.detach().float().cpu().requires_grad_(True)
    k = K.detach().float().cpu().requires_grad_(True)
    v = V.detach().float().cpu().requires_grad_(True)
    g = dO.detach().float().cpu()
    b = None if rel is None else rel.detach().float().cpu().requires_grad_(True)
    out = th.empty(n, h, d)
    for r0 in range(0, n, rows_per_block):
        r1 = min(n, r0 + rows_per_block)
        lo, hi = int(ip[r0]), int(ip[r1])
        if hi == lo:
            out[r0:r1] = 0
            continue
        deg = ip[r0 + 1:r1 + 1] - ip[r0:r1]
        dst = th.repeat_interleave(th.arange(r1 - r0), deg)
        src = idx[lo:hi]
        qb = q[r0:r1]
        ke = k.index_select(0, src)
        if b is not None:
            ke = ke + b[lo:hi].unsqueeze(1)
        s = (qb.index_select(0, dst) * ke).sum(-1) * scale
        m = th.full((r1 - r0, h), -float("inf")).scatter_reduce(0, dst.view(-1, 1).expand(-1, h), s.detach(),
                                                                 reduce="amax")
        ex = th.exp(s - m.index_select(0, dst))
        den = th.zeros(r1 - r0, h).index_add(0, dst, ex)
        p = ex / den.index_select(0, dst)
        ob = th.zeros(r1 - r0, h, d).index_add(0, dst, p.unsqueeze(-1) * v.index_select(0, src))
        ob.backward(g[r0:r1])
        out[r0:r1] = ob.detach()
    return out, q.grad, k.grad, v.grad


def time_chain(indptr, indices, Q, K, V, scale, dO, repeats=1, rel=None):
    """Seconds of one forward+backward (best of `repeats`)."""
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        attention_chain_cpu(indptr, indices, Q, K, V, scale, dO, rel=rel)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def _edge_list(indptr, indices):
    ip = indptr.to("cpu", th.int64)
    dst = th.repeat_interleave(th.arange(ip.numel() - 1), ip[1:] - ip[:-1])
    return dst, indices.to("cpu", th.int64)


def gat_cpu(indptr, indices, X, Be, w, dY1, dY2):
    """node_mul_edge(X, Be) and vector_spmm(w, X), forward and backward, on the CPU in float32."""
    dst, src = _edge_list(indptr, indices)
    x = X.detach().float().requires_grad_(True)
    be = Be.detach().float().requires_grad_(True)
    ww = w.detach().float().requires_grad_(True)
    y1 = (x.index_select(0, dst) * be.unsqueeze(1)).sum(-1)
    y2 = th.zeros_like(x).index_add(0, dst, ww.unsqueeze(-1) * x.index_select(0, src))
    th.autograd.backward([y1, y2], [dY1.float(), dY2.float()])
    return y1.detach(), y2.detach(), x.grad, be.grad, ww.grad


def sddmm_softmax_cpu(indptr, indices, Q, K, dP):
    """maskedmm(Q, K) then sparse softmax per destination, forward and backward, on the CPU in float32."""
    dst, src = _edge_list(indptr, indices)
    q = Q.detach().float().requires_grad_(True)
    k = K.detach().float().requires_grad_(True)
    h = q.shape[1]
    s = (q.index_select(0, dst) * k.index_select(0, src)).sum(-1)
    m = th.full((q.shape[0], h), -float("inf")).scatter_reduce(0, dst.view(-1, 1).expand(-1, h), s.detach(), reduce="amax")
    ex = th.exp(s - m.index_select(0, dst))
    p = ex / th.zeros(q.shape[0], h).index_add(0, dst, ex).index_select(0, dst)
    p.backward(dP.float())
    return p.detach(), q.grad, k.grad


def time_workload(ops, g, h, d, seed=1):
    """Seconds of one forward + backward of the named op group on graph `g`."""
    gen = th.Generator().manual_seed(seed)
    r = lambda *s: th.randn(*s, generator=gen)
    n, m, e = g.n_dst, g.n_src, g.n_edges
    if ops == "attention":
        return time_chain(g.indptr, g.indices, r(n, h, d), r(m, h, d), r(m, h, d), d ** -0.5, r(n, h, d))
    if ops == "attention_bias":
        return time_chain(g.indptr, g.indices, r(n, h, d), r(m, h, d), r(m, h, d), d ** -0.5, r(n, h, d),
                          rel=r(e, d) * 0.5)
    t0 = time.perf_counter()
    if ops == "gat":
        gat_cpu(g.indptr, g.indices, r(n, h, d), r(e, d), th.rand(e, h, generator=gen), r(e, h), r(n, h, d))
    elif ops == "sddmm_softmax":
        sddmm_softmax_cpu(g.indptr, g.indices, r(n, h, d) * 3, r(m, h, d) * 3, r(e, h))
    else:
        raise ValueError(ops)
    return time.perf_counter() - t0
