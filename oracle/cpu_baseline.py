"""Torch CPU implementation of the attention chain, the timed CPU baseline.  TEST / BENCH
INFRASTRUCTURE ONLY: nothing in the product package imports it.

Same arithmetic as the op-by-op oracle (graphop_oracle.py), written for speed on the host
cores instead of for float64 exactness: float32, gathers with index_select, per-node
reductions with scatter_reduce / index_add_, the backward through torch autograd, destination
nodes processed in blocks so that the (edges, heads, dim) temporaries stay bounded.
"""
import time

import torch as th


def attention_chain_cpu(indptr, indices, Q, K, V, scale, dO, rows_per_block=1 << 15):
    """Forward and backward of SDDMM(Q, K) * scale -> softmax per destination -> SpMM(V) on the
    CPU.  Returns (O, dQ, dK, dV)."""
    ip = indptr.to("cpu", th.int64)
    idx = indices.to("cpu", th.int64)
    n, h, d = Q.shape
    q = Q.detach().float().cpu().requires_grad_(True)
    k = K.detach().float().cpu().requires_grad_(True)
    v = V.detach().float().cpu().requires_grad_(True)
    g = dO.detach().float().cpu()
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
        s = (qb.index_select(0, dst) * k.index_select(0, src)).sum(-1) * scale
        m = th.full((r1 - r0, h), -float("inf")).scatter_reduce(0, dst.view(-1, 1).expand(-1, h), s.detach(),
                                                                 reduce="amax")
        ex = th.exp(s - m.index_select(0, dst))
        den = th.zeros(r1 - r0, h).index_add(0, dst, ex)
        p = ex / den.index_select(0, dst)
        ob = th.zeros(r1 - r0, h, d).index_add(0, dst, p.unsqueeze(-1) * v.index_select(0, src))
        ob.backward(g[r0:r1])
        out[r0:r1] = ob.detach()
    return out, q.grad, k.grad, v.grad


def time_chain(indptr, indices, Q, K, V, scale, dO, repeats=1):
    """Seconds of one forward+backward (best of `repeats`)."""
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        attention_chain_cpu(indptr, indices, Q, K, V, scale, dO)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best
