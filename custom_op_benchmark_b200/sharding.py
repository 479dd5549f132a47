"""Row-partitioned graphs for several GPUs (one process per GPU, torch.distributed).

The reference runs on one device only (wrapper.py:119, 142-145); nothing in it partitions a
graph across devices (part_csr.py cuts rows into chunks for load balance inside one GPU).  This
module adds the split the large configurations need:

* destination nodes are cut into P contiguous ranges with balanced edge counts; rank p owns rows
  ``[bounds[p], bounds[p+1])``, ``bounds[p] = searchsorted(indptr, floor(p * E / P), 'left')`` with
  ``bounds[0] = 0`` and ``bounds[P] = N``.  Integer arithmetic only, so every rank (and the host
  and the device) computes identical bounds;
* a rank's local CSR keeps *global* source ids, so the only exchange of a forward SpMM is one
  all-gather of the source-feature shards (features are sharded evenly by node id);
* the backward's dx uses the transposed CSR cut the same way by *source* node, with dy
  all-gathered, so every gradient row is owned by exactly one rank: no reduce-scatter and no
  atomics, results stay bit-reproducible.  dedata needs no exchange at all.

The compute is whatever ``ops`` namespace is passed (default: the CUDA ops of this package); the
CPU tests pass the oracle and run the same bookkeeping over gloo.
"""
from dataclasses import dataclass

import torch as th
import torch.distributed as dist

from .part_csr import partition_csr

__all__ = ["balanced_bounds", "even_bounds", "GraphShard", "shard_graph", "all_gather_rows",
           "sharded_spmm_forward", "sharded_spmm_backward"]


def balanced_bounds(indptr, parts):
    """Row boundaries of `parts` contiguous shards with balanced edge counts (int64 tensor, parts + 1)."""
    ip = indptr.to(th.int64)
    n, e = ip.numel() - 1, int(ip[-1]) - int(ip[0])
    targets = th.tensor([int(ip[0]) + (p * e) // parts for p in range(1, parts)], dtype=th.int64, device=ip.device)
    inner = th.searchsorted(ip, targets, right=False).clamp_(max=n)
    b = th.cat([th.zeros(1, dtype=th.int64, device=ip.device), inner, th.full((1,), n, dtype=th.int64, device=ip.device)])
    return th.cummax(b, 0).values  # monotone even when several targets fall into one long row


def even_bounds(n, parts):
    """Boundaries of `parts` equal row ranges (the feature sharding); needs parts | n."""
    if n % parts:
        raise ValueError("the node count must be divisible by the number of shards")
    return th.arange(parts + 1, dtype=th.int64) * (n // parts)


@dataclass
class GraphShard:
    """What one rank holds: its rows of the row CSR and its rows of the transposed CSR."""
    rank: int
    parts: int
    n_dst: int            # global number of destination nodes
    n_src: int            # global number of source nodes
    dst_bounds: th.Tensor  # (parts + 1,) destination-row ownership
    src_bounds: th.Tensor  # (parts + 1,) source-row ownership of the transposed CSR
    # row CSR of the owned destinations: chunk table, local edge ids 0..e_local-1, global source ids
    row: th.Tensor
    indptr: th.Tensor
    eid: th.Tensor
    indices: th.Tensor
    # transposed CSR of the owned sources: chunk table, *global* edge ids, global destination ids
    col: th.Tensor
    indptr_t: th.Tensor
    eid_t: th.Tensor
    indices_t: th.Tensor
    edge_lo: int          # global edge id of the rank's first row-CSR edge

    @property
    def rows(self):
        return int(self.dst_bounds[self.rank + 1] - self.dst_bounds[self.rank])

    @property
    def cols(self):
        return int(self.src_bounds[self.rank + 1] - self.src_bounds[self.rank])


def shard_graph(g, rank, parts, chunk_size=32, index_dtype=th.int32):
    """Cut a `graphs.Graph` for `rank` of `parts`.  Edge ids stay the global row-CSR positions."""
    db = balanced_bounds(g.indptr, parts)
    sb = balanced_bounds(g.indptr_t, parts)
    r0, r1 = int(db[rank]), int(db[rank + 1])
    ip = g.indptr.to(th.int64)
    lo, hi = int(ip[r0]), int(ip[r1])
    local_ip = ip[r0:r1 + 1] - lo
    row, ptr = partition_csr(local_ip, chunk_size)
    c0, c1 = int(sb[rank]), int(sb[rank + 1])
    ipt = g.indptr_t.to(th.int64)
    tlo, thi = int(ipt[c0]), int(ipt[c1])
    col, ptr_t = partition_csr(ipt[c0:c1 + 1] - tlo, chunk_size)
    cv = lambda t: t.to(index_dtype).contiguous()
    return GraphShard(rank, parts, g.n_dst, g.n_src, db, sb,
                      cv(row), cv(ptr), cv(th.arange(hi - lo, device=ip.device)), cv(g.indices[lo:hi]),
                      cv(col), cv(ptr_t), cv(g.eid_t[tlo:thi]), cv(g.indices_t[tlo:thi]), lo)


def all_gather_rows(local, bounds, group=None, async_op=False):
    """Concatenation over ranks of row blocks whose sizes are `bounds[p+1] - bounds[p]`.

    Equal blocks go through one all_gather_into_tensor.  Unequal blocks: on NCCL every rank's block is
    received straight into its slice of the result (all_gather over a list of views, which NCCL runs as
    one group of broadcasts), so the gathered rows are written once; other backends pad to the largest
    block for the collective and compact afterwards.

    async_op=True returns (result, work): the collective is only enqueued, and `work.wait()` (None when
    nothing is pending) must be called before the result is read, so that independent kernels can run
    on the compute stream meanwhile."""
    parts = bounds.numel() - 1
    counts = (bounds[1:] - bounds[:-1]).tolist()
    total = int(bounds[-1])
    done = (lambda out, work=None: (out, work) if async_op else out)
    if parts == 1:
        return done(local)
    out = th.empty((total,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    if len(set(counts)) == 1:
        work = dist.all_gather_into_tensor(out, local.contiguous(), group=group, async_op=async_op)
        return done(out, work)
    if local.is_cuda and min(counts) > 0 and dist.get_backend(group) == "nccl":
        views = [out[int(bounds[p]):int(bounds[p + 1])] for p in range(parts)]
        work = dist.all_gather(views, local.contiguous(), group=group, async_op=async_op)
        return done(out, work)
    width = max(counts)
    padded = th.zeros((width,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    buf = th.empty((parts * width,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    for p in range(parts):
        out[int(bounds[p]):int(bounds[p + 1])] = buf[p * width:p * width + counts[p]]
    return done(out)


def _default_ops():
    from . import graphop
    return graphop


def sharded_spmm_forward(sh, edata_local, x_shard, ops=None, group=None):
    """y rows of the owned destinations.  `edata_local`: weights of the owned edges (local edge
    order), `x_shard`: this rank's even share of the source features.  Returns (y_local, x_all)."""
    ops = ops or _default_ops()
    x_all = all_gather_rows(x_shard, even_bounds(sh.n_src, sh.parts), group)
    y = ops.vector_spmm_forward(sh.row, sh.indptr, sh.eid, sh.indices, edata_local, x_all, num_dst=sh.rows)
    return y, x_all


def sharded_spmm_backward(sh, edata_local, dy_local, x_all, edata_all, ops=None, group=None):
    """(dedata_local, dx_owned): gradients of the owned edges' weights, and of the source rows this
    rank owns in the transposed split.  `edata_all`: the weights of all edges by global edge id
    (gathered once per graph by the caller; the transposed CSR reads them through eid_t)."""
    ops = ops or _default_ops()
    # the gather of dy is only needed by dx: it is enqueued first and travels while dedata is computed
    dy_all, pending = all_gather_rows(dy_local, sh.dst_bounds, group, async_op=True)
    # dedata: sampled dot products of the owned rows of dy against gathered x; no exchange.
    # The op reads dy by destination id and the local chunk table names local rows 0..rows-1.
    dedata = ops.maskedmm_csr_forward(sh.row, sh.indptr, sh.eid, sh.indices, dy_local, x_all)
    if pending is not None:
        pending.wait()
    # dx: row-owned aggregation over the transposed shard, dy gathered, weights by global edge id
    dx = ops.vector_spmm_forward(sh.col, sh.indptr_t, sh.eid_t, sh.indices_t, edata_all, dy_all, num_dst=sh.cols)
    return dedata, dx
