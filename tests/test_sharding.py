"""Row partition across ranks: the balanced-nnz bounds are bit-exact against a pure-Python
rule, and a 2-rank gloo run of the sharded SpMM forward + backward (oracle as the local compute)
reproduces the unsharded result."""
import bisect
import os
import socket

import pytest
import torch as th
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import assert_close, chunked, random_graph
from custom_op_benchmark_b200 import graphs, sharding
from oracle import graphop_oracle as orc


def _bounds_python(indptr, parts):
    ip = [int(v) for v in indptr]
    n, e = len(ip) - 1, ip[-1] - ip[0]
    b = [0] + [min(n, bisect.bisect_left(ip, ip[0] + (p * e) // parts)) for p in range(1, parts)] + [n]
    for i in range(1, len(b)):
        b[i] = max(b[i], b[i - 1])
    return b


@pytest.mark.parametrize("parts", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_balanced_bounds_match_python_rule(parts, seed):
    g = th.Generator().manual_seed(seed)
    deg = th.randint(0, 30, (257,), generator=g)
    deg[th.rand(257, generator=g) < 0.3] = 0
    deg[5] = 2000  # a row longer than a whole shard
    ip = th.cat([th.zeros(1, dtype=th.long), th.cumsum(deg, 0)])
    b = sharding.balanced_bounds(ip, parts)
    assert b.tolist() == _bounds_python(ip.tolist(), parts)
    assert b[0] == 0 and b[-1] == 257 and bool((b[1:] >= b[:-1]).all())
    # every shard's edge count is within one row of the ideal share
    e = int(ip[-1])
    for p in range(parts):
        cnt = int(ip[b[p + 1]] - ip[b[p]])
        assert cnt <= e / parts + int(deg.max())
    assert sharding.balanced_bounds(ip.to(th.int32), parts).tolist() == b.tolist()


def test_shards_cover_the_graph_exactly():
    g = graphs.rmat_graph(9, 8, seed=3)
    seen_rows, seen_edges, seen_t = 0, [], []
    for r in range(4):
        sh = sharding.shard_graph(g, r, 4, chunk_size=32)
        seen_rows += sh.rows
        seen_edges.append(sh.indices)
        seen_t.append(sh.eid_t.long())
        assert int(sh.indptr[-1]) == sh.indices.numel() and int(sh.indptr_t[-1]) == sh.eid_t.numel()
        assert sh.edge_lo == int(g.indptr[int(sh.dst_bounds[r])])
    assert seen_rows == g.n_dst
    assert th.equal(th.cat(seen_edges), g.indices)
    assert th.equal(th.cat(seen_t), g.eid_t.long())  # every edge id exactly once on the transposed side


def _test_graph(world):
    """R-MAT 256 nodes for 2 ranks; for 3 ranks a graph whose node count 3 divides, with empty rows and one
    row longer than a shard."""
    if world == 2:
        return graphs.rmat_graph(8, 8, seed=5, index_dtype=th.int64)
    gen = th.Generator().manual_seed(11)
    degs = th.randint(0, 12, (150,), generator=gen)
    degs[th.rand(150, generator=gen) < 0.3] = 0
    degs[17] = 900
    return random_graph(150, 150, degs, 12)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = _test_graph(world)
    h, d = 2, 4
    gen = th.Generator().manual_seed(6)
    x = th.randn(g.n_src, h, d, generator=gen, dtype=th.float64)
    w = th.rand(g.n_edges, h, generator=gen, dtype=th.float64)
    dy = th.randn(g.n_dst, h, d, generator=gen, dtype=th.float64)
    sh = sharding.shard_graph(g, rank, world, chunk_size=8, index_dtype=th.int64)
    xb = sharding.even_bounds(g.n_src, world)
    lo, hi = sh.edge_lo, sh.edge_lo + sh.indices.numel()
    r0, r1 = int(sh.dst_bounds[rank]), int(sh.dst_bounds[rank + 1])
    y, x_all = sharding.sharded_spmm_forward(sh, w[lo:hi].contiguous(), x[int(xb[rank]):int(xb[rank + 1])].contiguous(),
                                             ops=orc)
    # weights sharded like the edges: the transposed shard's weights are all-gathered inside the call
    dw, dx = sharding.sharded_spmm_backward(sh, w[lo:hi].contiguous(), dy[r0:r1].contiguous(), x_all, ops=orc)
    # ... or handed over by a caller that keeps every weight on every rank
    dw0, dx0 = sharding.sharded_spmm_backward(sh, w[lo:hi].contiguous(), dy[r0:r1].contiguous(), x_all, w, ops=orc)
    assert th.equal(dw0, dw) and th.equal(dx0, dx)
    # the same step fetching only the referenced rows
    ex = sharding.plan_shard_exchange(sh)
    assert th.equal(ex.x.needed[ex.indices.long()], sh.indices.long())
    assert th.equal(ex.dy.needed[ex.indices_t.long()], sh.indices_t.long())
    assert sum(ex.x.recv_counts) + ex.x.own_idx.numel() == ex.x.needed.numel() <= g.n_src
    assert ex.x.recv_counts[rank] == 0 and ex.x.send_counts[rank] == 0   # own rows stay out of the collective
    y2, x_rows = sharding.sharded_spmm_forward(sh, w[lo:hi].contiguous(),
                                               x[int(xb[rank]):int(xb[rank + 1])].contiguous(), ops=orc, exchange=ex)
    assert th.equal(x_rows, x[ex.x.needed])
    # the weights of the transposed shard's edges travel by edge id, from the ranks that own them
    assert th.equal(ex.w.needed[ex.eid_t.long()], sh.eid_t.long())
    w_t, ids = sharding.gather_edge_weights(sh, w[lo:hi].contiguous(), exchange=ex)
    assert th.equal(w_t[ids.long()], w[sh.eid_t.long()])
    dw2, dx2 = sharding.sharded_spmm_backward(sh, w[lo:hi].contiguous(), dy[r0:r1].contiguous(), x_rows, ops=orc,
                                              exchange=ex)
    th.save({"y": y, "dw": dw, "dx": dx, "y2": y2, "dw2": dw2, "dx2": dx2, "rows": (r0, r1), "edges": (lo, hi),
             "cols": (int(sh.src_bounds[rank]), int(sh.src_bounds[rank + 1]))}, os.path.join(out_dir, "r%d.pt" % rank))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_spmm_matches_unsharded(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g = _test_graph(world)
    h, d = 2, 4
    gen = th.Generator().manual_seed(6)
    x = th.randn(g.n_src, h, d, generator=gen, dtype=th.float64)
    w = th.rand(g.n_edges, h, generator=gen, dtype=th.float64)
    dy = th.randn(g.n_dst, h, d, generator=gen, dtype=th.float64)
    r, c = chunked(g, 8), chunked(g, 8, transposed=True)
    want_y = orc.vector_spmm_forward(*r, w, x)
    want_dw, want_dx = orc.vector_spmm_backward(*r, *c, w, dy, x)
    for suffix in ("", "2"):   # all-gathered rows, then only the referenced rows
        y, dw, dx = th.zeros_like(want_y), th.zeros_like(want_dw), th.zeros_like(want_dx)
        for rank in range(world):
            o = th.load(os.path.join(str(tmp_path), "r%d.pt" % rank))
            y[o["rows"][0]:o["rows"][1]] = o["y" + suffix]
            dw[o["edges"][0]:o["edges"][1]] = o["dw" + suffix]
            dx[o["cols"][0]:o["cols"][1]] = o["dx" + suffix]
        assert_close(y, want_y, 1e-12, 1e-13, "y" + suffix)
        assert_close(dw, want_dw, 1e-12, 1e-13, "dedata" + suffix)
        assert_close(dx, want_dx, 1e-12, 1e-13, "dx" + suffix)
