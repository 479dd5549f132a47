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
  atomics, results stay bit-reproducible.  dedata needs no exchange at all;
* edge weights are sharded like the edges: a rank holds the weights of its own destination rows only.
  The transposed shard reads weights of edges that other ranks own, so they travel every step (they are the
  softmax output in training and change with every step): one more exchange, by edge id.

All-gathering a node tensor delivers (P-1)/P of it to every rank whatever P is.  The alternative,
built once per graph by ``plan_shard_exchange``, fetches from their owners only the rows a shard's
edges reference (one all-to-all by index lists) and renumbers the shard's indices into that compact
set; ``sharded_spmm_forward/backward(..., exchange=plan)`` use it.

The compute is whatever ``ops`` namespace is passed (default: the CUDA ops of this package); the
CPU tests pass the oracle and run the same bookkeeping over gloo.
"""
from dataclasses import dataclass

import torch as th
import torch.distributed as dist

from .part_csr import partition_csr

__all__ = ["balanced_bounds", "even_bounds", "GraphShard", "shard_graph", "all_gather_rows",
           "RowExchange", "ShardExchange", "PeerRows", "plan_row_exchange", "plan_shard_exchange", "exchange_rows",
           "gather_edge_weights", "sharded_spmm_forward", "sharded_spmm_backward"]


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
    edge_bounds: th.Tensor = None  # (parts + 1,) global edge id ranges of the ranks' row shards

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
                      cv(col), cv(ptr_t), cv(g.eid_t[tlo:thi]), cv(g.indices_t[tlo:thi]), lo,
                      ip[db.to(ip.device)].to("cpu"))


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


@dataclass
class RowExchange:
    """How one rank obtains the rows of a row-sharded tensor that its shard references.  The received
    buffer holds the rows of the other ranks in rank order, then the rows of this rank's own block
    (which never pass through the collective)."""
    needed: th.Tensor     # (M,) global row ids in buffer order
    send_idx: th.Tensor   # rows of this rank's own block to send, concatenated by receiving rank
    send_counts: list     # rows sent to each rank (0 for this rank)
    recv_counts: list     # rows received from each rank, in rank order (0 for this rank)
    own_idx: th.Tensor    # rows of this rank's own block that it references itself
    pull_idx: th.Tensor = None   # (sum(recv_counts),) int32: the other ranks' rows as ids local to their owner


@dataclass
class ShardExchange:
    """The exchanges of a sharded SpMM step and the shard's indices renumbered into the received rows."""
    x: RowExchange            # source features, owners by even_bounds(n_src)
    dy: RowExchange           # upstream gradient rows, owners by the shard's dst_bounds
    w: RowExchange            # weights of the transposed shard's edges, owners by the shard's edge_bounds
    indices: th.Tensor        # sh.indices as positions in x.needed
    indices_t: th.Tensor      # sh.indices_t as positions in dy.needed
    eid_t: th.Tensor          # sh.eid_t as positions in w.needed


def plan_row_exchange(indices, owner_bounds, rank, group=None):
    """(RowExchange, compact indices) for the rows named by `indices` of a tensor whose row block p lives on
    rank p (`owner_bounds`, P + 1 entries).  Collective: every rank of the group calls it once per graph."""
    parts = owner_bounds.numel() - 1
    dev = indices.device
    idx = indices.to(th.int64)
    uniq = th.unique(idx)                                     # sorted
    ob = owner_bounds.to(device=dev, dtype=th.int64)
    cuts = th.searchsorted(uniq, ob)                          # rows of owner p: uniq[cuts[p]:cuts[p+1]]
    counts = cuts[1:] - cuts[:-1]
    local_id = uniq - th.repeat_interleave(ob[:-1], counts)   # row ids local to their owner
    c0, c1 = int(cuts[rank]), int(cuts[rank + 1])
    own_n, m = c1 - c0, uniq.numel()
    # buffer order: the other ranks' rows (sorted), then the own rows
    pos = th.searchsorted(uniq, idx)
    compact = th.where(pos < c0, pos, th.where(pos < c1, pos - c0 + (m - own_n), pos - own_n)).to(indices.dtype)
    needed = th.cat([uniq[:c0], uniq[c1:], uniq[c0:c1]])
    request = th.cat([local_id[:c0], local_id[c1:]])
    recv_counts = counts.tolist()
    recv_counts[rank] = 0
    own_idx = local_id[c0:c1].contiguous()
    pull_idx = request.to(th.int32) if int(ob[-1]) < 2 ** 31 else None
    if parts == 1:
        return RowExchange(needed, request, [0], [0], own_idx, pull_idx), compact
    send_counts_t = th.empty(parts, dtype=th.int64, device=dev)
    dist.all_to_all_single(send_counts_t, th.tensor(recv_counts, dtype=th.int64, device=dev), group=group)
    send_counts = send_counts_t.tolist()
    send_idx = th.empty(sum(send_counts), dtype=th.int64, device=dev)
    dist.all_to_all_single(send_idx, request.contiguous(), output_split_sizes=send_counts,
                           input_split_sizes=recv_counts, group=group)
    if int(ob[-1]) < 2 ** 31:   # row ids of one block: the copy kernel takes them as int32
        send_idx, own_idx = send_idx.to(th.int32), own_idx.to(th.int32)
    return RowExchange(needed, send_idx, send_counts, recv_counts, own_idx, pull_idx), compact


def plan_shard_exchange(sh, group=None):
    """The three exchanges of `sh` (collective; once per graph)."""
    x_plan, ic = plan_row_exchange(sh.indices, even_bounds(sh.n_src, sh.parts), sh.rank, group)
    dy_plan, itc = plan_row_exchange(sh.indices_t, sh.dst_bounds, sh.rank, group)
    w_plan, etc = plan_row_exchange(sh.eid_t, sh.edge_bounds, sh.rank, group)
    return ShardExchange(x_plan, dy_plan, w_plan, ic.contiguous(), itc.contiguous(), etc.contiguous())


def _torch_gather_rows(table, idx, out=None):
    return th.index_select(table, 0, idx, out=out)


def exchange_rows(local, plan, group=None, async_op=False, gather=None):
    """The rows `plan.needed` of the row-sharded tensor whose block on this rank is `local`, in that order.
    async_op=True returns (rows, work) like all_gather_rows.  `gather(table, idx, out=None)` packs rows
    (default: torch.index_select; the CUDA ops bring their own copy kernel)."""
    gather = gather or _torch_gather_rows
    peers, own = sum(plan.recv_counts), plan.own_idx.numel()
    out = th.empty((peers + own,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    work = None
    if len(plan.recv_counts) > 1:
        send = gather(local, plan.send_idx)
        work = dist.all_to_all_single(out[:peers], send, output_split_sizes=plan.recv_counts,
                                      input_split_sizes=plan.send_counts, group=group, async_op=async_op)
    gather(local, plan.own_idx, out=out[peers:])   # own rows: a local copy, meanwhile
    return (out, work if async_op else None) if async_op else out


class PeerRows:
    """A row-sharded tensor whose block on every rank lives in symmetric memory, so that every rank can read every
    block with plain loads over NVLink.  Built once (collective): `local` is this rank's block to write into,
    `pull(plan)` fetches the rows `plan.needed` with one kernel on this GPU (graphop_pull_rows_i32) instead of
    pack + all-to-all + unpack, `barrier()` orders the ranks (all blocks written before anyone pulls; everyone done
    pulling before a block is written again).  NVLink multicast is not used and is switched off for the mapping."""

    def __init__(self, rows, row_shape, dtype, device, group=None):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        group = group or dist.group.WORLD
        world = dist.get_world_size(group)
        counts = [th.zeros(1, dtype=th.int64, device=device) for _ in range(world)]
        dist.all_gather(counts, th.tensor([rows], dtype=th.int64, device=device), group=group)
        most = max(int(c) for c in counts)                 # symmetric allocations have one size on all ranks
        self.buffer = symm.empty((max(most, 1),) + tuple(row_shape), dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.buffer, group)
        self.local = self.buffer[:rows]
        self.tables = [int(p) for p in self.handle.buffer_ptrs]
        self.rank, self.world = dist.get_rank(group), world
        self.row_bytes = self.buffer[0].numel() * self.buffer.element_size()   # also for a rank that owns no row

    def barrier(self):
        self.handle.barrier()

    def pull(self, plan, ops=None):
        ops = ops or _default_ops()
        peers, own = sum(plan.recv_counts), plan.own_idx.numel()
        out = th.empty((peers + own,) + tuple(self.local.shape[1:]), dtype=self.local.dtype, device=self.local.device)
        seg = [0]
        for c in plan.recv_counts:
            seg.append(seg[-1] + c)
        if peers:
            ops.pull_rows(self.tables, seg, plan.pull_idx, self.row_bytes, out[:peers])
        ops.gather_rows(self.local, plan.own_idx, out=out[peers:])
        return out


def _default_ops():
    from . import graphop
    return graphop


def sharded_spmm_forward(sh, edata_local, x_shard, ops=None, group=None, exchange=None):
    """y rows of the owned destinations.  `edata_local`: weights of the owned edges (local edge
    order), `x_shard`: this rank's even share of the source features.  Returns (y_local, x_rows):
    x_rows is the gathered node tensor, or with `exchange` only the rows the shard references."""
    ops = ops or _default_ops()
    if isinstance(x_shard, PeerRows):     # the block lives in symmetric memory: pull the referenced rows from the peers
        x_rows = x_shard.pull(exchange.x, ops)
        y = ops.vector_spmm_forward(sh.row, sh.indptr, sh.eid, exchange.indices, edata_local, x_rows, num_dst=sh.rows)
        return y, x_rows
    if exchange is not None:
        x_rows = exchange_rows(x_shard, exchange.x, group, gather=getattr(ops, "gather_rows", None))
        y = ops.vector_spmm_forward(sh.row, sh.indptr, sh.eid, exchange.indices, edata_local, x_rows, num_dst=sh.rows)
        return y, x_rows
    x_all = all_gather_rows(x_shard, even_bounds(sh.n_src, sh.parts), group)
    y = ops.vector_spmm_forward(sh.row, sh.indptr, sh.eid, sh.indices, edata_local, x_all, num_dst=sh.rows)
    return y, x_all


def gather_edge_weights(sh, edata_local, group=None, exchange=None):
    """Weights of the transposed shard's edges.  With `exchange`: (weights of exactly those edges, fetched from
    the ranks that own them, indexed by exchange.eid_t).  Without: (every rank's weights all-gathered, indexed by
    global edge id, i.e. by sh.eid_t).  Returns (weights, edge ids to read them with)."""
    if exchange is not None:
        rows = exchange_rows(edata_local.reshape(edata_local.shape[0], -1), exchange.w, group)
        return rows.reshape((rows.shape[0],) + tuple(edata_local.shape[1:])), exchange.eid_t
    return all_gather_rows(edata_local, sh.edge_bounds, group), sh.eid_t


def sharded_spmm_backward(sh, edata_local, dy_local, x_all, edata_all=None, ops=None, group=None, exchange=None):
    """(dedata_local, dx_owned): gradients of the owned edges' weights, and of the source rows this
    rank owns in the transposed split.  `x_all`: what the forward returned (with `exchange`: the referenced
    rows).  The transposed shard needs the weights of edges other ranks own: they are exchanged here, every
    call, unless the caller passes `edata_all` (all weights by global edge id, e.g. a graph whose weights never
    change)."""
    ops = ops or _default_ops()
    # the rows of dy are only needed by dx: their transfer is enqueued first and travels while dedata is computed
    if isinstance(dy_local, PeerRows):
        dy_rows, pending = dy_local.pull(exchange.dy, ops), None
        src_ids, dst_ids = exchange.indices, exchange.indices_t
        dy_local = dy_local.local
    elif exchange is not None:
        dy_rows, pending = exchange_rows(dy_local, exchange.dy, group, async_op=True,
                                         gather=getattr(ops, "gather_rows", None))
        src_ids, dst_ids = exchange.indices, exchange.indices_t
    else:
        dy_rows, pending = all_gather_rows(dy_local, sh.dst_bounds, group, async_op=True)
        src_ids, dst_ids = sh.indices, sh.indices_t
    if edata_all is not None:
        w_t, eid_t = edata_all, sh.eid_t
    else:
        w_t, eid_t = gather_edge_weights(sh, edata_local, group, exchange)
    # dedata: sampled dot products of the owned rows of dy against the source rows; no exchange.
    # The op reads dy by destination id and the local chunk table names local rows 0..rows-1.
    dedata = ops.maskedmm_csr_forward(sh.row, sh.indptr, sh.eid, src_ids, dy_local, x_all)
    if pending is not None:
        pending.wait()
    # dx: row-owned aggregation over the transposed shard
    dx = ops.vector_spmm_forward(sh.col, sh.indptr_t, eid_t, dst_ids, w_t, dy_rows, num_dst=sh.cols)
    return dedata, dx
