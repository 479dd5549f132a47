"""Sharded SpMM on real GPUs: 2 ranks over NCCL against the unsharded CUDA ops (needs 2 devices)."""
import os
import socket

import pytest
import torch as th
import torch.distributed as dist
import torch.multiprocessing as mp

from helpers import chunked
from custom_op_benchmark_b200 import graphs, sharding

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _inputs():
    g = graphs.rmat_graph(12, 16, seed=5)
    gen = th.Generator().manual_seed(6)
    x = th.randn(g.n_src, 128, generator=gen)
    w = th.rand(g.n_edges, generator=gen)
    dy = th.randn(g.n_dst, 128, generator=gen)
    return g, x, w, dy


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    th.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=th.device("cuda", rank))
    dev = "cuda:%d" % rank
    g, x, w, dy = _inputs()
    sh = sharding.shard_graph(g.to(dev), rank, world, chunk_size=32)
    xb = sharding.even_bounds(g.n_src, world)
    lo, hi = sh.edge_lo, sh.edge_lo + sh.indices.numel()
    r0, r1 = int(sh.dst_bounds[rank]), int(sh.dst_bounds[rank + 1])
    y, x_all = sharding.sharded_spmm_forward(sh, w[lo:hi].to(dev), x[int(xb[rank]):int(xb[rank + 1])].to(dev))
    dw, dx = sharding.sharded_spmm_backward(sh, w[lo:hi].to(dev), dy[r0:r1].to(dev), x_all)
    # the same step fetching only the rows the shard references
    ex = sharding.plan_shard_exchange(sh)
    y2, x_rows = sharding.sharded_spmm_forward(sh, w[lo:hi].to(dev), x[int(xb[rank]):int(xb[rank + 1])].to(dev),
                                               exchange=ex)
    assert th.equal(x_rows.cpu(), x[ex.x.needed.cpu()])
    dw2, dx2 = sharding.sharded_spmm_backward(sh, w[lo:hi].to(dev), dy[r0:r1].to(dev), x_rows, exchange=ex)
    assert th.equal(y2, y) and th.equal(dw2, dw) and th.equal(dx2, dx)   # same rows, same order of summation
    # the same rows pulled straight out of the peers' memory by one kernel per rank (no collective in the data path)
    px = sharding.PeerRows(int(xb[rank + 1] - xb[rank]), (128,), th.float32, dev)
    pdy = sharding.PeerRows(r1 - r0, (128,), th.float32, dev)
    px.local.copy_(x[int(xb[rank]):int(xb[rank + 1])])
    pdy.local.copy_(dy[r0:r1])
    px.barrier()
    pdy.barrier()
    y3, x_rows3 = sharding.sharded_spmm_forward(sh, w[lo:hi].to(dev), px, exchange=ex)
    dw3, dx3 = sharding.sharded_spmm_backward(sh, w[lo:hi].to(dev), pdy, x_rows3, exchange=ex)
    th.cuda.synchronize()
    dist.barrier()      # every rank is done reading its peers' blocks; only then may a rank fail and leave
    assert th.equal(x_rows3, x_rows) and th.equal(y3, y) and th.equal(dw3, dw) and th.equal(dx3, dx)
    th.save({"y": y.cpu(), "dw": dw.cpu(), "dx": dx.cpu(), "rows": (r0, r1), "edges": (lo, hi),
             "cols": (int(sh.src_bounds[rank]), int(sh.src_bounds[rank + 1]))}, os.path.join(out_dir, "r%d.pt" % rank))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(th.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_sharded_spmm_matches_single_gpu(tmp_path):
    from custom_op_benchmark_b200 import graphop
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    g, x, w, dy = _inputs()
    dev = "cuda:0"
    R = [t.to(dev) for t in chunked(g, 32)]
    C = [t.to(dev) for t in chunked(g, 32, transposed=True)]
    want_y = graphop.vector_spmm_forward(*R, w.to(dev), x.to(dev)).cpu()
    want_dw, want_dx = (t.cpu() for t in graphop.vector_spmm_backward(*R, *C, w.to(dev), dy.to(dev), x.to(dev)))
    y, dw, dx = th.zeros_like(want_y), th.zeros_like(want_dw), th.zeros_like(want_dx)
    for rank in range(world):
        o = th.load(os.path.join(str(tmp_path), "r%d.pt" % rank))
        y[o["rows"][0]:o["rows"][1]] = o["y"]
        dw[o["edges"][0]:o["edges"][1]] = o["dw"]
        dx[o["cols"][0]:o["cols"][1]] = o["dx"]
    # per-edge results are identical; per-row sums may differ in the last bits where a shard boundary
    # moves a tile boundary
    assert th.equal(dw, want_dw)
    assert th.allclose(y, want_y, rtol=1e-5, atol=1e-5) and th.allclose(dx, want_dx, rtol=1e-5, atol=1e-5)
