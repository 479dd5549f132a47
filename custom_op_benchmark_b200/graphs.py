"""Seeded synthetic graphs and the CSR plumbing around them.

The reference builds one test graph by hand (512 fully-connected blocks of 30
nodes, wrapper.py:79-116) and nothing else.  The workloads measured here are
generated from seeds instead of read from a dataset: Erdos-Renyi in-neighbour
lists, banded local attention, R-MAT power-law graphs and a rank-size (Zipf)
in-degree sequence.  Every generator returns a `Graph` holding both CSR
orientations in the layout the ops consume:

* row CSR, sorted by destination then source: ``indptr`` (N_dst+1),
  ``indices`` (source of each edge), ``eid`` (identity: the edge id of an edge
  IS its position in the row CSR, as in wrapper.py:100);
* transposed CSR, sorted by source then destination: ``indptr_t`` (N_src+1),
  ``indices_t`` (destination of each edge), ``eid_t`` (a true permutation
  mapping a transposed position to its edge id, as ``eid_c`` in wrapper.py:110).

All tensor work is torch, so a generator runs on whatever device it is given;
index dtype is int32 unless asked otherwise.
"""
from dataclasses import dataclass

import numpy as np
import torch as th

__all__ = [
    "Graph", "coo_to_graph", "transpose_csr", "transpose_csr_tensor_ops", "block_diagonal_graph", "er_graph",
    "banded_graph", "rmat_graph", "zipf_graph",
]


@dataclass
class Graph:
    n_dst: int
    n_src: int
    indptr: th.Tensor
    indices: th.Tensor
    eid: th.Tensor
    indptr_t: th.Tensor
    indices_t: th.Tensor
    eid_t: th.Tensor

    @property
    def n_edges(self):
        return int(self.indices.numel())

    def to(self, device=None, dtype=None):
        def cv(t):
            return t.to(device=device if device is not None else t.device,
                        dtype=dtype if dtype is not None else t.dtype)
        return Graph(self.n_dst, self.n_src, cv(self.indptr), cv(self.indices), cv(self.eid),
                     cv(self.indptr_t), cv(self.indices_t), cv(self.eid_t))

    def dst_of_edge(self):
        """Destination node of every edge, by edge id (int64)."""
        deg = (self.indptr[1:] - self.indptr[:-1]).to(th.int64)
        return th.repeat_interleave(th.arange(self.n_dst, device=deg.device), deg)


def _indptr_from_sorted(keys, n):
    counts = th.bincount(keys, minlength=n) if keys.numel() else th.zeros(n, dtype=th.int64, device=keys.device)
    ip = th.zeros(n + 1, dtype=th.int64, device=keys.device)
    th.cumsum(counts, 0, out=ip[1:])
    return ip


def transpose_csr(indptr, indices, n_src):
    """Transposed CSR of a row CSR whose edge ids are its positions.

    Returns ``(indptr_t, indices_t, eid_t)`` as int64: edges regrouped by source,
    ties kept in row-CSR order (a stable sort), so within one source the
    destinations ascend.
    """
    if indptr.is_cuda and indices.is_cuda and indptr.dtype == indices.dtype and \
            indptr.dtype in (th.int32, th.int64) and indices.numel() < 2 ** 31 - 1:
        from . import graphop   # the CUDA library's kernels; raises if it has not been built
        return tuple(t.to(th.int64) for t in graphop.transpose_csr(indptr, indices, n_src))
    return transpose_csr_tensor_ops(indptr, indices, n_src)


def transpose_csr_tensor_ops(indptr, indices, n_src):
    """The same by tensor ops on the inputs' device (the host path, and the checker of the kernels)."""
    ip = indptr.to(th.int64)
    src = indices.to(th.int64)
    n_dst = ip.numel() - 1
    deg = ip[1:] - ip[:-1]
    dst = th.repeat_interleave(th.arange(n_dst, dtype=th.int64, device=ip.device), deg)
    order = th.sort(src, stable=True).indices  # position in transposed CSR -> edge id
    return _indptr_from_sorted(src, n_src), dst[order], order


def coo_to_graph(dst, src, n_dst, n_src=None, index_dtype=th.int32, dedup=False):
    """Build both CSR orientations from an edge list (dst <- src)."""
    n_src = n_dst if n_src is None else n_src
    dst = dst.to(th.int64)
    src = src.to(th.int64)
    key = dst * n_src + src
    key = th.unique(key) if dedup else th.sort(key).values
    dst = th.div(key, n_src, rounding_mode="floor")
    src = key - dst * n_src
    del key
    indptr = _indptr_from_sorted(dst, n_dst)
    indptr_t, indices_t, eid_t = transpose_csr(indptr, src, n_src)
    e = src.numel()
    cv = lambda t: t.to(index_dtype)
    return Graph(n_dst, n_src, cv(indptr), cv(src), cv(th.arange(e, device=src.device)),
                 cv(indptr_t), cv(indices_t), cv(eid_t))


def block_diagonal_graph(batch_size=512, l=30, index_dtype=th.int64, device="cpu"):
    """The reference's own test graph: `batch_size` fully-connected blocks of `l` nodes.

    Same arrays as the loops at wrapper.py:93-112 produce (row CSR with identity
    eid; column CSR with eid_c = b*l*l + (x%l)*l + (y%l)), built without loops.
    """
    n = batch_size * l
    b = th.arange(batch_size, device=device).view(-1, 1, 1)
    x = th.arange(l, device=device).view(1, -1, 1)
    y = th.arange(l, device=device).view(1, 1, -1)
    dst = (b * l + x).expand(batch_size, l, l).reshape(-1)
    src = (b * l + y).expand(batch_size, l, l).reshape(-1)
    return coo_to_graph(dst, src, n, index_dtype=index_dtype)


def er_graph(n=4096, k=15, seed=0, index_dtype=th.int32, device="cpu"):
    """Directed Erdos-Renyi-style graph: every node gets `k` distinct random
    in-neighbours other than itself, plus a self-loop (E = n*(k+1) exactly)."""
    g = th.Generator(device="cpu").manual_seed(seed)
    # k distinct values of 0..n-2 per row by ranking random keys, then skip over the diagonal
    pick = th.rand(n, n - 1, generator=g).topk(k, dim=1).indices
    rows = th.arange(n).view(-1, 1)
    pick = pick + (pick >= rows).to(pick.dtype)
    src = th.cat([pick, rows], 1).reshape(-1)
    dst = rows.expand(n, k + 1).reshape(-1)
    return coo_to_graph(dst.to(device), src.to(device), n, index_dtype=index_dtype)


def banded_graph(batch=4, length=8192, window=128, index_dtype=th.int32, device="cpu"):
    """Banded local attention as a graph: `batch` independent sequences, row i of a
    sequence attends to positions [max(0, i-window), min(length-1, i+window)]."""
    i = th.arange(length, device=device)
    lo = (i - window).clamp_(min=0)
    hi = (i + window).clamp_(max=length - 1)
    deg = hi - lo + 1
    dst1 = th.repeat_interleave(i, deg)
    start = th.cumsum(deg, 0) - deg
    src1 = th.arange(int(deg.sum()), device=device) - start[dst1] + lo[dst1]
    off = (th.arange(batch, device=device) * length).view(-1, 1)
    dst = (dst1.view(1, -1) + off).reshape(-1)
    src = (src1.view(1, -1) + off).reshape(-1)
    return coo_to_graph(dst, src, batch * length, index_dtype=index_dtype)


def rmat_graph(scale, edge_factor=16, a=0.57, b=0.19, c=0.19, d=0.05, seed=0,
               index_dtype=th.int32, device="cpu", chunk=1 << 25):
    """R-MAT graph: 2**scale nodes, edge_factor * 2**scale raw edges drawn with the
    quadrant probabilities (a, b, c, d); self-loops and duplicates removed, then one
    self-loop per node added.  Bit k of (dst, src) is drawn independently per level:
    quadrant a = (0,0), b = (0,1), c = (1,0), d = (1,1)."""
    n = 1 << scale
    m = edge_factor * n
    gen = th.Generator(device=device).manual_seed(seed)
    keys = []
    for s0 in range(0, m, chunk):
        cnt = min(chunk, m - s0)
        dst = th.zeros(cnt, dtype=th.int64, device=device)
        src = th.zeros(cnt, dtype=th.int64, device=device)
        for _ in range(scale):
            u = th.rand(cnt, generator=gen, device=device)
            dbit = (u >= a + b).to(th.int64)
            sbit = ((u >= a) & (u < a + b) | (u >= a + b + c)).to(th.int64)
            dst = (dst << 1) | dbit
            src = (src << 1) | sbit
        keep = dst != src
        keys.append(dst[keep] * n + src[keep])
    loops = th.arange(n, dtype=th.int64, device=device)
    keys.append(loops * n + loops)
    key = th.unique(th.cat(keys))
    del keys
    dst = th.div(key, n, rounding_mode="floor")
    src = key - dst * n
    return coo_to_graph(dst, src, n, index_dtype=index_dtype)


def zipf_degrees(n, total, s=1.1, cap=1_000_000):
    """Rank-size in-degree sequence deg_r = clip(floor(c * r**-s), 1, cap), r = 1..n,
    with c bisected so that the degrees sum as close to `total` as possible."""
    r = np.arange(1, n + 1, dtype=np.float64) ** (-s)

    def degs(cc):
        return np.clip(np.floor(cc * r), 1, cap).astype(np.int64)

    lo, hi = 1.0, float(total) * 4
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if degs(mid).sum() < total:
            lo = mid
        else:
            hi = mid
    return degs(hi)


def zipf_graph(n=1_000_000, total=50_000_000, s=1.1, cap=1_000_000, seed=0,
               index_dtype=th.int32, device="cpu"):
    """Skewed in-degrees: the rank-size degree sequence above is assigned to node ids
    by a seeded permutation; sources are uniform random, duplicates allowed."""
    deg = th.from_numpy(zipf_degrees(n, total, s, min(cap, total)))
    g = th.Generator(device="cpu").manual_seed(seed)
    perm = th.randperm(n, generator=g)
    deg_of_node = th.empty(n, dtype=th.int64)
    deg_of_node[perm] = deg
    deg_of_node = deg_of_node.to(device)
    e = int(deg_of_node.sum())
    dst = th.repeat_interleave(th.arange(n, dtype=th.int64, device=device), deg_of_node)
    gen = th.Generator(device=device).manual_seed(seed + 1)
    src = th.randint(0, n, (e,), generator=gen, device=device, dtype=th.int64)
    return coo_to_graph(dst, src, n, index_dtype=index_dtype)
