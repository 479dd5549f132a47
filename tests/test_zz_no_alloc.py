"""The scratch-free SpMM entry point (graphop_vector_spmm_forward_f32_i32_static) against the
ordinary one.

The static variant exists for hosts that cannot give the library a workspace because they cannot
allocate device memory themselves; it keeps its scratch in a fixed array inside the library.  The
test calls it through the C ABI twice in a row, on different inputs, so that the second call runs
on whatever the first left in the shared array, and requires bit-identical output to the
workspace-taking entry point both times.  It also checks that an oversized problem is refused
before anything is launched.  This file sorts last on purpose: a failure here must not hide the
results of the other GPU tests in a run that stops at the first failure."""
import pytest
import torch as th

from helpers import chunked, random_graph
from custom_op_benchmark_b200 import _capi, graphop

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, n, h, d):
    g = th.Generator().manual_seed(seed)
    degs = th.randint(0, 40, (n,), generator=g)
    degs[th.rand(n, generator=g) < 0.2] = 0
    degs[n // 3] = 900            # after the zeroing: a node that spans several tiles, so the carry scratch is used
    gr = random_graph(n, n, degs, seed)
    r = [t.to(DEV) for t in chunked(gr, 32, dtype=th.int32)]
    w = th.rand(gr.n_edges, h, generator=g).to(DEV)
    x = th.randn(n, h, d, generator=g).to(DEV)
    return gr, r, w, x


def _static(gr, r, w, x, h, d):
    lib = _capi.lib()
    y = th.full_like(x, float("nan"))
    rc = lib.graphop_vector_spmm_forward_f32_i32_static(
        r[0].data_ptr(), r[1].data_ptr(), r[2].data_ptr(), r[3].data_ptr(), w.data_ptr(), x.data_ptr(), y.data_ptr(),
        r[0].numel(), gr.n_edges, gr.n_dst, gr.n_src, h, d, th.cuda.current_stream().cuda_stream)
    return rc, y


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    lib = _capi.lib()
    assert lib.graphop_static_scratch_bytes() == 32 << 20
    for seed, n, h, d in ((1, 700, 4, 32), (2, 1500, 2, 64)):
        gr, r, w, x = _case(seed, n, h, d)
        assert int((gr.indptr[1:] - gr.indptr[:-1]).max()) >= 900
        want = graphop.vector_spmm_forward(*r, w, x)
        rc, got = _static(gr, r, w, x, h, d)
        th.cuda.synchronize()
        assert rc == _capi.OK, _capi.error_message(rc)
        assert th.equal(got, want)   # same kernels, same tiling: not merely close, identical


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib = _capi.lib()
    # 40 M edges need far more than the 32 MiB the library carries: refused, nothing launched
    rc = lib.graphop_vector_spmm_forward_f32_i32_static(None, None, None, None, None, None, None, 10, 40_000_000,
                                                        1000, 1000, 4, 32, None)
    assert rc == _capi.ERR_UNSUPPORTED
    th.cuda.synchronize()
