"""Golden vectors produced by the reference's own CUDA extension (compiled unmodified, run on a
B200 by oracle/make_reference_golden.py): the CPU oracle must reproduce them (this is what pins
the oracle), and so must the CUDA kernels of this package.  float32 outputs of the reference carry
its atomic-order rounding noise, hence rel 1e-5 / abs 1e-6 there and 1e-12 for float64."""
import glob
import os

import numpy as np
import pytest
import torch as th

from helpers import ROOT, assert_close
from custom_op_benchmark_b200 import graphs
from custom_op_benchmark_b200.part_csr import partition_csr
from oracle import graphop_oracle as orc

FILES = sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "reference_cuda_*.npz")))


def _load(path):
    z = np.load(path)
    t = {k: th.from_numpy(z[k]) for k in z.files if z[k].ndim > 0}
    n = t["indptr"].numel() - 1
    tr = graphs.transpose_csr(t["indptr"], t["indices"], n)
    cs = int(z["chunk_size"])
    row, ptr = partition_csr(t["indptr"], cs)
    col, ptr_t = partition_csr(tr[0], cs)
    eid = th.arange(t["indices"].numel())
    R = [row, ptr, eid, t["indices"]]
    C = [col, ptr_t, tr[2], tr[1]]
    assert [row.numel(), col.numel()] == z["chunks"].tolist()
    f64 = z["A"].dtype == np.float64
    return t, R, C, ((1e-12, 1e-13) if f64 else (1e-5, 1e-6)), bool(z["dx_complete"])


def _check_all(t, tol, dx_complete, run):
    """`run(name, *args)` computes one op; compare everything with the stored reference outputs."""
    rt, at = tol
    got = {}
    got["mm_y"] = run("maskedmm_csr_forward", "R", t["A"], t["B"])
    got["mm_dA"], got["mm_dB"] = run("maskedmm_csr_backward", "RC", t["A"], t["B"], t["dy_e"])
    got["nme_y"] = run("node_mul_edge_forward", "R3", t["A"], t["Be"])
    got["nme_dA"], got["nme_dB"] = run("node_mul_edge_backward", "R3", t["A"], t["Be"], t["dy_e"])
    got["sm_y"] = run("sparse_softmax_forward", "R3", t["x_e"])
    got["sm_dx"] = run("sparse_softmax_backward", "R3", t["sm_y"], t["dy_e"])
    got["sm_y_t"] = run("sparse_softmax_forward", "C3", t["x_e"])
    got["spmm_y"] = run("vector_spmm_forward", "R", t["w"], t["X"])
    got["spmm_dw"], got["spmm_dx"] = run("vector_spmm_backward", "RC", t["w"], t["dY"], t["X"])
    for name, val in got.items():
        if name == "spmm_dx" and not dx_complete:
            continue
        scale = max(1.0, float(t[name].abs().max()))
        assert_close(val, t[name], rt, at * scale, name)


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(p)[15:-4] for p in FILES])
def test_oracle_reproduces_reference_outputs(path):
    t, R, C, tol, dx_complete = _load(path)
    sel = {"R": R, "RC": R + C, "R3": R[:3], "C3": C[:3]}
    _check_all(t, tol, dx_complete, lambda name, g, *a: getattr(orc, name)(*sel[g], *a))


@pytest.mark.gpu
@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(p)[15:-4] for p in FILES])
@pytest.mark.parametrize("idt", [th.int64, th.int32])
def test_cuda_kernels_reproduce_reference_outputs(path, idt):
    from custom_op_benchmark_b200 import graphop
    t, R, C, tol, dx_complete = _load(path)
    dev = "cuda:0"
    Rc, Cc = [x.to(dev, idt) for x in R], [x.to(dev, idt) for x in C]
    sel = {"R": Rc, "RC": Rc + Cc, "R3": Rc[:3], "C3": Cc[:3]}
    _check_all(t, tol, dx_complete, lambda name, g, *a: getattr(graphop, name)(*sel[g], *[x.to(dev) for x in a]))


def test_golden_files_exist():
    assert len(FILES) == 3
