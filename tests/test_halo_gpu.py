"""The halo-sharded banded attention on the GPU: every shard's (own rows) x (window rows) problem runs through the
shard's graph plans - in bfloat16 with 64 features per head that is the tensor-core kernel on a rectangular problem
with the window's offset - and the shards together reproduce the unsharded layer.  The exchange itself is host
bookkeeping tested over gloo (test_halo.py); here one process plays every rank in turn and slices the halo rows
out of the full tensors."""
import pytest
import torch as th

from helpers import assert_close
from custom_op_benchmark_b200 import graphs, halo
from oracle import edge_list_f64 as ref

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("parts,dt,h,d", [(1, th.bfloat16, 8, 64), (2, th.bfloat16, 8, 64), (3, th.bfloat16, 4, 64),
                                          (3, th.float32, 4, 32)])
def test_shards_reproduce_the_unsharded_layer(parts, dt, h, d):
    g = graphs.banded_graph(2, 768, 128).to(device=DEV)
    n, scale = g.n_dst, d ** -0.5
    gen = th.Generator(device=DEV).manual_seed(51)
    Q, K, V, dO = (th.randn(n, h, d, generator=gen, device=DEV).to(dt) for _ in range(4))
    o, lse = th.empty_like(Q), th.empty(n, h, device=DEV)
    dq = th.empty_like(Q)
    dk, dv = th.zeros(n, h, d, device=DEV), th.zeros(n, h, d, device=DEV)
    for rank in range(parts):
        sh = halo.shard_band(g.indptr, g.indices, rank, parts)
        plan_r, plan_t = halo._plans(sh)
        assert plan_r.dense_band and plan_t.dense_band
        q, g_o = Q[sh.lo:sh.hi].contiguous(), dO[sh.lo:sh.hi].contiguous()
        k_win, v_win = K[sh.win_lo:sh.win_hi].contiguous(), V[sh.win_lo:sh.win_hi].contiguous()
        o_l, lse_l = halo._cuda_forward(sh, q, k_win, v_win, scale)
        dq_l, dk_w, dv_w = halo._cuda_backward(sh, q, k_win, v_win, o_l, lse_l, g_o, scale)
        o[sh.lo:sh.hi], lse[sh.lo:sh.hi], dq[sh.lo:sh.hi] = o_l, lse_l, dq_l
        dk[sh.win_lo:sh.win_hi] += dk_w.float()      # what halo_scatter_add does across ranks
        dv[sh.win_lo:sh.win_hi] += dv_w.float()
    want = ref.attention_f64(g.indptr, g.indices, Q, K, V, scale, dO)
    rt, at = (2e-2, 2e-2) if dt == th.bfloat16 else (2e-5, 2e-5)
    for got, w, name in zip((o, lse, dq, dk, dv), want, ("o", "lse", "dq", "dk", "dv")):
        assert_close(got, w, rt, at * max(1.0, float(w.abs().max())), name)
