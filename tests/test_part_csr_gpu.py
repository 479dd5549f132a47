"""partition_csr on the device (the library's count / fill kernels): bit-exact against the reference's outputs
(golden JSON), against the reference's host loop restated in the oracle, and against the tensor-op path, for both
index types, every chunk size of interest, empty rows, an empty graph and a graph without rows."""
import json
import os

import pytest
import torch as th

from helpers import ROOT
from custom_op_benchmark_b200 import graphop, graphs
from custom_op_benchmark_b200.part_csr import partition_csr, partition_csr_tensor_ops
from oracle.graphop_oracle import partition_csr_loop

pytestmark = pytest.mark.gpu
GOLDEN = json.load(open(os.path.join(ROOT, "tests", "golden", "partition_csr.json")))
DEV = "cuda:0"


def _same(got, want):
    row, ptr = got
    assert row.dtype == th.int64 and ptr.dtype == th.int64 and row.is_cuda and ptr.is_cuda
    assert row.cpu().tolist() == [int(x) for x in want[0]]
    assert ptr.cpu().tolist() == [int(x) for x in want[1]]


@pytest.mark.parametrize("dt", [th.int32, th.int64])
@pytest.mark.parametrize("case", GOLDEN, ids=lambda c: "cs%d_n%d" % (c["chunk_size"], len(c["indptr"]) - 1))
def test_golden(case, dt):
    got = partition_csr(th.tensor(case["indptr"], dtype=dt, device=DEV), case["chunk_size"])
    if len(case["row"]) == 0:
        assert got[0].numel() == 0 and got[1].cpu().tolist() == case["indptr_"]
    else:
        _same(got, (case["row"], case["indptr_"]))


@pytest.mark.parametrize("dt", [th.int32, th.int64])
@pytest.mark.parametrize("chunk_size", [1, 2, 7, 32, 33, 1000, 2 ** 40])
def test_against_the_host_loop(chunk_size, dt):
    gen = th.Generator().manual_seed(chunk_size % 1000)
    deg = th.randint(0, 90, (257,), generator=gen)
    deg[th.randint(0, 257, (60,), generator=gen)] = 0          # empty rows, also runs of them and at both ends
    deg[:3] = 0
    deg[-2:] = 0
    ip = th.cat([th.zeros(1, dtype=th.int64), th.cumsum(deg, 0)])
    want = partition_csr_loop(ip.tolist(), chunk_size)
    _same(graphop.partition_csr(ip.to(dt).to(DEV), chunk_size), want)


@pytest.mark.parametrize("dt", [th.int32, th.int64])
def test_degenerate_graphs(dt):
    row, ptr = partition_csr(th.tensor([5], dtype=dt, device=DEV), 32)           # no rows: the sentinel alone
    assert row.numel() == 0 and ptr.cpu().tolist() == [5]
    row, ptr = partition_csr(th.zeros(11, dtype=dt, device=DEV), 32)             # rows, no edges
    assert row.numel() == 0 and ptr.cpu().tolist() == [0]
    row, ptr = partition_csr(th.tensor([0, 64], dtype=dt, device=DEV), 32)       # exact multiples: no empty chunk
    assert row.cpu().tolist() == [0, 0] and ptr.cpu().tolist() == [0, 32, 64]
    with pytest.raises(ValueError):
        partition_csr(th.tensor([0, 3], dtype=dt, device=DEV), 0)


def test_large_graph_matches_tensor_ops():
    g = graphs.rmat_graph(17, 16, seed=5)
    for ip in (g.indptr, g.indptr_t):
        for cs in (32, 5):
            want = partition_csr_tensor_ops(ip.to(DEV), cs)
            got = graphop.partition_csr(ip.to(DEV), cs)
            assert th.equal(got[0], want[0]) and th.equal(got[1], want[1])
    # a view with an offset and a non-default stream
    ip = g.indptr.to(DEV)
    s = th.cuda.Stream()
    s.wait_stream(th.cuda.current_stream())
    with th.cuda.stream(s):
        got = partition_csr(ip[1000:5001], 32)
    s.synchronize()
    want = partition_csr_tensor_ops(ip[1000:5001], 32)
    assert th.equal(got[0], want[0]) and th.equal(got[1], want[1])


def test_bad_arguments():
    with pytest.raises(RuntimeError):
        graphop.partition_csr(th.tensor([0, 3]), 32)                             # host tensor at the kernel entry
    with pytest.raises(RuntimeError):
        graphop.partition_csr(th.zeros(2, 2, dtype=th.int32, device=DEV), 32)
    row, ptr = partition_csr(th.tensor([0, 3], dtype=th.int16, device=DEV), 2)   # other integer types: tensor ops
    assert row.tolist() == [0, 0] and ptr.tolist() == [0, 2, 3]


# ---- transpose_csr on the device -------------------------------------------------------------------------------
from custom_op_benchmark_b200.graphs import transpose_csr, transpose_csr_tensor_ops  # noqa: E402


def _transpose_loop(indptr, indices, n_src):
    """Counting sort in plain Python: the definition (sources ascending, ties in row-CSR order)."""
    buckets = [[] for _ in range(n_src)]
    for r in range(len(indptr) - 1):
        for e in range(indptr[r], indptr[r + 1]):
            buckets[indices[e]].append((r, e))
    ptr, idx, eid = [0], [], []
    for b in buckets:
        idx += [r for r, _ in b]
        eid += [e for _, e in b]
        ptr.append(len(idx))
    return ptr, idx, eid


@pytest.mark.parametrize("dt", [th.int32, th.int64])
def test_transpose_small_against_the_definition(dt):
    gen = th.Generator().manual_seed(11)
    n_dst, n_src = 37, 53                                           # rectangular, sources without edges
    deg = th.randint(0, 9, (n_dst,), generator=gen)
    deg[[0, 5, 6, 36]] = 0
    ip = th.cat([th.zeros(1, dtype=th.int64), th.cumsum(deg, 0)])
    idx = th.randint(3, n_src - 4, (int(ip[-1]),), generator=gen)    # repeated sources inside a row too
    want = _transpose_loop(ip.tolist(), idx.tolist(), n_src)
    got = graphop.transpose_csr(ip.to(dt).to(DEV), idx.to(dt).to(DEV), n_src)
    for g, w in zip(got, want):
        assert g.dtype == dt and g.cpu().tolist() == w


@pytest.mark.parametrize("name", ["rmat", "zipf", "band"])
def test_transpose_large_matches_tensor_ops(name):
    g = {"rmat": lambda: graphs.rmat_graph(17, 16, seed=3), "zipf": lambda: graphs.zipf_graph(50000, 600000, seed=3),
         "band": lambda: graphs.banded_graph(2, 4096, 128)}[name]()
    for dt in (th.int32, th.int64):
        ip, idx = g.indptr.to(DEV, dt), g.indices.to(DEV, dt)
        got = transpose_csr(ip, idx, g.n_src)                        # int64 out, as the host path
        want = transpose_csr_tensor_ops(ip, idx, g.n_src)
        for a, b in zip(got, want):
            assert a.dtype == th.int64 and th.equal(a, b)
        assert th.equal(got[0].cpu(), g.indptr_t.long()) and th.equal(got[2].cpu(), g.eid_t.long())
    again = graphop.transpose_csr(ip, idx, g.n_src)                  # the same on every run
    assert th.equal(again[2], got[2])


@pytest.mark.parametrize("dt", [th.int32, th.int64])
def test_transpose_degenerate(dt):
    e = th.empty(0, dtype=dt, device=DEV)
    ptr_t, idx_t, eid_t = graphop.transpose_csr(th.zeros(6, dtype=dt, device=DEV), e, 4)   # rows, no edges
    assert ptr_t.tolist() == [0] * 5 and idx_t.numel() == 0 and eid_t.numel() == 0
    ptr_t, _, _ = graphop.transpose_csr(th.zeros(1, dtype=dt, device=DEV), e, 0)            # nothing at all
    assert ptr_t.tolist() == [0]
    ptr_t, idx_t, eid_t = graphop.transpose_csr(th.tensor([0, 3], dtype=dt, device=DEV),
                                                th.tensor([2, 0, 2], dtype=dt, device=DEV), 3)
    assert ptr_t.tolist() == [0, 1, 1, 3] and idx_t.tolist() == [0, 0, 0] and eid_t.tolist() == [1, 0, 2]
    with pytest.raises(RuntimeError):
        graphop.transpose_csr(th.tensor([0, 1], dtype=th.int32, device=DEV), th.tensor([0], device=DEV), 1)
