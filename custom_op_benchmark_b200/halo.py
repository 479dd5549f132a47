"""Banded (sliding-window) attention cut by rows over several GPUs, with a halo exchange of K and V.

The reference has one long-sequence case, batched block-diagonal attention written as a graph and run on one device
(wrapper.py:79-112).  For sequences that should be spread over GPUs the natural cut of such a graph is by contiguous
destination rows: rank p owns the queries (and the K / V rows) of ``[bounds[p], bounds[p+1])``, and because every
row's neighbours are a run of consecutive ids, the columns a shard references form one window
``[win_lo, win_hi)`` around its own rows.  What lies outside the own range is the halo: ``window`` rows of K and V
on each side for a band of half-width ``window``.

* forward: one all-to-all delivers the halo rows of K and V (both in one message per peer; only neighbours
  exchange anything), then the ordinary attention op runs on (own Q rows) x (window K / V rows) - on a dense
  band in bfloat16 that is the tensor-core kernel;
* backward: the same op gives dQ for the own rows and dK / dV for every window row; the halo parts travel back
  to their owners (the forward's all-to-all with the roles swapped) and are added there in rank order, so every
  gradient row is summed in a fixed order and the result is bit-reproducible.

All ranks cut the same global CSR, so every rank works out every window and message size from the graph alone:
setting a shard up needs no communication.  The compute is a pair of callables (default: the CUDA ops of this
package through graph plans); the CPU tests pass a float64 reference and run the same bookkeeping over gloo.
"""
from dataclasses import dataclass, field

import torch as th
import torch.distributed as dist

from .part_csr import partition_csr

__all__ = ["BandShard", "shard_band", "halo_gather", "halo_scatter_add", "band_attention_forward",
           "band_attention_backward"]


@dataclass
class BandShard:
    """One rank's rows of a banded graph and the window of columns they reference."""
    rank: int
    parts: int
    bounds: th.Tensor        # (parts + 1,) row split, the same on every rank
    windows: th.Tensor       # (parts, 2) [win_lo, win_hi) of every rank
    indptr: th.Tensor        # local row CSR: own rows ...
    indices: th.Tensor       # ... columns relative to win_lo
    indptr_t: th.Tensor      # local transposed CSR: one row per window column ...
    indices_t: th.Tensor     # ... own-row ids relative to bounds[rank]
    eid_t: th.Tensor         # position in the local row CSR of every transposed position
    send_counts: list = field(default_factory=list)   # own rows sent to each rank (forward direction)
    recv_counts: list = field(default_factory=list)   # halo rows received from each rank
    send_slices: list = field(default_factory=list)   # (start, stop) in own rows, per rank
    recv_slices: list = field(default_factory=list)   # (start, stop) in window rows, per rank
    cache: dict = field(default_factory=dict)         # what the compute callables keep per shard (chunk tables, plans)

    @property
    def lo(self):
        return int(self.bounds[self.rank])

    @property
    def hi(self):
        return int(self.bounds[self.rank + 1])

    @property
    def rows(self):
        return self.hi - self.lo

    @property
    def win_lo(self):
        return int(self.windows[self.rank, 0])

    @property
    def win_hi(self):
        return int(self.windows[self.rank, 1])

    @property
    def window_rows(self):
        return self.win_hi - self.win_lo

    @property
    def own_offset(self):
        """Where the own rows start inside the window."""
        return self.lo - self.win_lo


def _overlap(a0, a1, b0, b1):
    lo, hi = max(a0, b0), min(a1, b1)
    return (lo, hi) if hi > lo else (0, 0)


def shard_band(indptr, indices, rank, parts, bounds=None, index_dtype=th.int32):
    """Cuts the square graph (indptr, indices: CSR by destination over n nodes, K / V rows owned like the query
    rows) into `parts` contiguous row ranges and returns rank's BandShard.  `bounds` defaults to equal ranges rounded
    to multiples of 128 rows (the tensor-core kernel's tile).  No communication: every rank reads the same CSR."""
    ip = indptr.to(th.int64)
    n = ip.numel() - 1
    dev = ip.device
    if bounds is None:
        per = -(-n // parts)
        per = -(-per // 128) * 128
        bounds = th.tensor([min(n, p * per) for p in range(parts + 1)], dtype=th.int64)
    bounds = bounds.to("cpu", th.int64)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    e0, e1 = int(ip[lo]), int(ip[hi])
    cols = indices[e0:e1].to(th.int64)
    # every rank holds the whole CSR: each computes every rank's window itself, no collective
    windows = th.empty(parts, 2, dtype=th.int64)
    for p in range(parts):
        plo, phi = int(bounds[p]), int(bounds[p + 1])
        pc = indices[int(ip[plo]):int(ip[phi])]
        windows[p, 0] = min(int(pc.min()), plo) if pc.numel() else plo
        windows[p, 1] = max(int(pc.max()) + 1, phi) if pc.numel() else phi
    win = [int(windows[rank, 0]), int(windows[rank, 1])]
    local_ptr = (ip[lo:hi + 1] - e0)
    local_idx = cols - win[0]
    # transposed local CSR over the window columns
    w = win[1] - win[0]
    order = th.argsort(local_idx, stable=True)
    counts = th.bincount(local_idx, minlength=w) if local_idx.numel() else th.zeros(w, dtype=th.int64, device=dev)
    ptr_t = th.cat([th.zeros(1, dtype=th.int64, device=dev), th.cumsum(counts, 0)])
    dst_local = th.repeat_interleave(th.arange(hi - lo, device=dev), local_ptr[1:] - local_ptr[:-1])
    sh = BandShard(rank, parts, bounds, windows, local_ptr.to(index_dtype), local_idx.to(index_dtype),
                   ptr_t.to(index_dtype), dst_local[order].to(index_dtype), order.to(index_dtype))
    for p in range(parts):
        plo, phi = int(bounds[p]), int(bounds[p + 1])
        if p == rank:
            sh.send_slices.append((0, 0))
            sh.recv_slices.append((0, 0))
        else:
            a, b = _overlap(int(windows[p, 0]), int(windows[p, 1]), lo, hi)      # own rows rank p wants
            sh.send_slices.append((a - lo, b - lo) if b > a else (0, 0))
            c, d = _overlap(win[0], win[1], plo, phi)                            # rows of rank p in my window
            sh.recv_slices.append((c - win[0], d - win[0]) if d > c else (0, 0))
        sh.send_counts.append(sh.send_slices[-1][1] - sh.send_slices[-1][0])
        sh.recv_counts.append(sh.recv_slices[-1][1] - sh.recv_slices[-1][0])
    return sh


def halo_gather(sh, local, group=None):
    """The window rows of a row-sharded node tensor: the own block in place, the halo rows from their owners."""
    out = th.zeros((sh.window_rows,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    out[sh.own_offset:sh.own_offset + sh.rows] = local
    if sh.parts == 1:
        return out
    send = th.cat([local[a:b] for a, b in sh.send_slices]) if sum(sh.send_counts) else local[:0]
    recv = th.empty((sum(sh.recv_counts),) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_to_all_single(recv, send.contiguous(), output_split_sizes=sh.recv_counts,
                           input_split_sizes=sh.send_counts, group=group)
    at = 0
    for (a, b), c in zip(sh.recv_slices, sh.recv_counts):
        if c:
            out[a:b] = recv[at:at + c]
            at += c
    return out


def halo_scatter_add(sh, window, group=None):
    """The reverse of halo_gather for gradients: every window row goes to its owner, and an owner adds what it
    receives to its own part in rank order (a fixed order: reproducible sums).  Returns the own rows."""
    own = window[sh.own_offset:sh.own_offset + sh.rows].clone()
    if sh.parts == 1:
        return own
    send = th.cat([window[a:b] for a, b in sh.recv_slices]) if sum(sh.recv_counts) else window[:0]
    recv = th.empty((sum(sh.send_counts),) + tuple(window.shape[1:]), dtype=window.dtype, device=window.device)
    dist.all_to_all_single(recv, send.contiguous(), output_split_sizes=sh.send_counts,
                           input_split_sizes=sh.recv_counts, group=group)
    at = 0
    for (a, b), c in zip(sh.send_slices, sh.send_counts):
        if c:
            own[a:b] += recv[at:at + c]
            at += c
    return own


def _plans(sh):
    """Graph plans of the shard's two local CSR orientations (built once, kept in the shard)."""
    if "plans" not in sh.cache:
        from . import graphop
        row, ptr = partition_csr(sh.indptr, 32)
        col, ptr_t = partition_csr(sh.indptr_t, 32)
        dt = sh.indices.dtype
        eid = th.arange(sh.indices.numel(), dtype=dt, device=sh.indices.device)
        plan_r = graphop.GraphPlan(row.to(dt), ptr.to(dt), eid, sh.indices, sh.rows)
        plan_t = graphop.GraphPlan(col.to(dt), ptr_t.to(dt), sh.eid_t, sh.indices_t, sh.window_rows)
        sh.cache["plans"] = (plan_r, plan_t)
    return sh.cache["plans"]


def _cuda_forward(sh, q, k_win, v_win, scale):
    from . import graphop
    return graphop.attention_forward_planned(_plans(sh)[0], q, k_win, v_win, scale)


def _cuda_backward(sh, q, k_win, v_win, o, lse, d_o, scale):
    from . import graphop
    plan_r, plan_t = _plans(sh)
    return graphop.attention_backward_planned(plan_r, plan_t, q, k_win, v_win, o, lse, d_o, scale)


def band_attention_forward(sh, q_local, k_local, v_local, scale, group=None, compute=None):
    """(o_local, lse_local, saved): attention of the own query rows over their window.  `compute(sh, q, k_win,
    v_win, scale) -> (o, lse)` defaults to the CUDA op on the shard's plan.  `saved` = (k_win, v_win) for the
    backward."""
    if sh.parts == 1:
        k_win, v_win = k_local, v_local                                      # the window is the whole tensor
    else:
        kv = halo_gather(sh, th.cat([k_local, v_local], dim=-1), group)      # one message per neighbour
        d = k_local.shape[-1]
        k_win, v_win = kv[..., :d].contiguous(), kv[..., d:].contiguous()
    o, lse = (compute or _cuda_forward)(sh, q_local, k_win, v_win, scale)
    return o, lse, (k_win, v_win)


def band_attention_backward(sh, q_local, saved, o, lse, d_o, scale, group=None, compute=None):
    """(dq_local, dk_local, dv_local).  `compute(sh, q, k_win, v_win, o, lse, d_o, scale) -> (dq, dk_win, dv_win)`
    defaults to the CUDA op on the shard's plans; the window gradients are summed at their owners."""
    k_win, v_win = saved
    dq, dk_win, dv_win = (compute or _cuda_backward)(sh, q_local, k_win, v_win, o, lse, d_o, scale)
    if sh.parts == 1:
        return dq, dk_win, dv_win
    d = k_win.shape[-1]
    back = halo_scatter_add(sh, th.cat([dk_win, dv_win], dim=-1), group)
    return dq, back[..., :d].contiguous(), back[..., d:].contiguous()
