"""Banded attention cut by rows over ranks with a halo exchange of K / V (custom_op_benchmark_b200/halo.py): gloo
runs of 2, 3 and 4 ranks, with the float64 edge-list reference as the local compute, reproduce the unsharded layer;
the halo is exactly the band's half-width; the transposed local CSR is a permutation of the local edges."""
import os
import socket

import pytest
import torch as th
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import assert_close
from custom_op_benchmark_b200 import graphs, halo
from oracle import edge_list_f64 as ref

H, D, SCALE = 2, 8, 0.3


def _graph(kind):
    if kind == "band":                       # two sequences of 192 positions, half-width 20
        return graphs.banded_graph(2, 192, 20)
    if kind == "wide":                       # half-width larger than a shard of 4: rows travel two ranks far
        return graphs.banded_graph(1, 256, 100)
    return graphs.block_diagonal_graph(9, 30)  # the reference's own test shape: blocks of 30, no halo inside a block


def _inputs(n):
    gen = th.Generator().manual_seed(7)
    return [th.randn(n, H, D, generator=gen, dtype=th.float64) for _ in range(4)]


def _ref_forward(sh, q, k_win, v_win, scale):
    return ref.attention_f64(sh.indptr, sh.indices, q, k_win, v_win, scale)


def _ref_backward(sh, q, k_win, v_win, o, lse, d_o, scale):
    return ref.attention_f64(sh.indptr, sh.indices, q, k_win, v_win, scale, d_o)[2:]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir, kind, per):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = _graph(kind)
    n = g.n_dst
    Q, K, V, dO = _inputs(n)
    bounds = th.tensor([min(n, p * per) for p in range(world)] + [n])
    sh = halo.shard_band(g.indptr, g.indices, rank, world, bounds=bounds, index_dtype=th.int64)
    lo, hi = sh.lo, sh.hi
    # the window is the own rows plus what the band reaches on either side
    cols = g.indices[int(g.indptr[lo]):int(g.indptr[hi])]
    if cols.numel():
        assert sh.win_lo == min(int(cols.min()), lo) and sh.win_hi == max(int(cols.max()) + 1, hi)
    else:
        assert (sh.win_lo, sh.win_hi, sh.rows) == (lo, hi, 0)     # a rank without rows: an empty window
    assert sh.send_counts[rank] == 0 and sh.recv_counts[rank] == 0
    assert sum(sh.recv_counts) == sh.window_rows - sh.rows           # every halo row comes from exactly one owner
    # the transposed local CSR lists every local edge once, under its window column
    e = sh.indices.numel()
    assert th.equal(th.sort(sh.eid_t).values, th.arange(e)) and int(sh.indptr_t[-1]) == e
    col_of = th.repeat_interleave(th.arange(sh.window_rows), sh.indptr_t[1:] - sh.indptr_t[:-1])
    assert th.equal(sh.indices[sh.eid_t], col_of)
    kw = halo.halo_gather(sh, K[lo:hi].contiguous())
    assert th.equal(kw, K[sh.win_lo:sh.win_hi])
    o, lse, saved = halo.band_attention_forward(sh, Q[lo:hi].contiguous(), K[lo:hi].contiguous(), V[lo:hi].contiguous(),
                                                SCALE, compute=_ref_forward)
    dq, dk, dv = halo.band_attention_backward(sh, Q[lo:hi].contiguous(), saved, o, lse, dO[lo:hi].contiguous(), SCALE,
                                              compute=_ref_backward)
    th.save({"rows": (lo, hi), "o": o, "lse": lse, "dq": dq, "dk": dk, "dv": dv, "halo": sum(sh.recv_counts)},
            os.path.join(out_dir, "r%d.pt" % rank))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,kind,per", [(2, "band", 192), (3, "band", 128), (4, "wide", 64), (2, "blocks", 135),
                                            (3, "wide", 128)])    # the last rank of three owns no row at all
def test_halo_sharded_attention_matches_unsharded(tmp_path, world, kind, per):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path), kind, per), nprocs=world, join=True)
    g = _graph(kind)
    Q, K, V, dO = _inputs(g.n_dst)
    want = ref.attention_f64(g.indptr, g.indices, Q, K, V, SCALE, dO)
    got = [th.zeros_like(w) for w in want]
    halos = []
    for rank in range(world):
        o = th.load(os.path.join(str(tmp_path), "r%d.pt" % rank))
        for t, name in zip(got, ("o", "lse", "dq", "dk", "dv")):
            t[o["rows"][0]:o["rows"][1]] = o[name]
        halos.append(o["halo"])
    for a, b, name in zip(got, want, ("o", "lse", "dq", "dk", "dv")):
        assert_close(a, b, 1e-12, 1e-12, name)
    if kind == "band" and world == 2:
        assert halos == [0, 0]          # the cut falls between the two sequences: nothing to exchange
    if kind == "band" and world == 3:
        assert halos == [20, 40, 20]     # half-width 20 on every open side
    if kind == "wide" and world == 4:
        assert halos == [100, 164, 164, 100]   # half-width 100 over shards of 64: rows travel two ranks far
    if kind == "wide" and world == 3:
        assert halos == [100, 100, 0]           # two shards of 128 rows and a rank that owns nothing


def test_single_rank_needs_no_process_group():
    g = _graph("band")
    Q, K, V, dO = _inputs(g.n_dst)
    sh = halo.shard_band(g.indptr, g.indices, 0, 1, index_dtype=th.int64)
    assert (sh.win_lo, sh.win_hi, sh.rows) == (0, g.n_dst, g.n_dst)
    o, lse, saved = halo.band_attention_forward(sh, Q, K, V, SCALE, compute=_ref_forward)
    dq, dk, dv = halo.band_attention_backward(sh, Q, saved, o, lse, dO, SCALE, compute=_ref_backward)
    want = ref.attention_f64(g.indptr, g.indices, Q, K, V, SCALE, dO)
    for a, b, name in zip((o, lse, dq, dk, dv), want, ("o", "lse", "dq", "dk", "dv")):
        assert_close(a, b, 1e-12, 1e-12, name)
