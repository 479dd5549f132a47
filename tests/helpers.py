"""Shared test plumbing: graph zoo, chunk tables, tolerance checks."""
import os
import sys

import torch as th

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from custom_op_benchmark_b200 import graphs  # noqa: E402
from custom_op_benchmark_b200.part_csr import partition_csr, unchunked_rows  # noqa: E402


def random_graph(n_dst, n_src, degs, seed, index_dtype=th.int64, dedup=False):
    """Graph with the given in-degree list (len n_dst), sources uniform random."""
    g = th.Generator().manual_seed(seed)
    deg = th.as_tensor(degs, dtype=th.int64)
    dst = th.repeat_interleave(th.arange(n_dst), deg)
    src = th.randint(0, n_src, (int(deg.sum()),), generator=g)
    return graphs.coo_to_graph(dst, src, n_dst, n_src, index_dtype=index_dtype, dedup=dedup)


def graph_zoo():
    """(name, Graph) pairs covering: empty rows, one-edge rows, rows spanning many chunks and
    tiles, a single huge row, rectangular shapes, no edges in the first / last nodes, node ids
    larger than the number of edges."""
    g = th.Generator().manual_seed(123)
    zoo = []
    zoo.append(("er64", graphs.er_graph(64, 5, seed=1, index_dtype=th.int64)))
    zoo.append(("blockdiag", graphs.block_diagonal_graph(4, 30)))
    degs = th.randint(0, 6, (200,), generator=g)
    degs[th.rand(200, generator=g) < 0.4] = 0
    degs[0] = 0
    degs[-3:] = 0
    zoo.append(("sparse_empty_rows", random_graph(200, 150, degs, 2)))
    degs = th.randint(0, 40, (97,), generator=g)
    degs[5] = 700
    degs[50] = 2500
    degs[51] = 1
    degs[96] = 300
    zoo.append(("long_rows", random_graph(97, 120, degs, 3)))
    zoo.append(("one_huge_row", random_graph(3, 50, [0, 5000, 0], 4)))
    zoo.append(("all_single", random_graph(300, 300, [1] * 300, 5)))
    zoo.append(("rect_wide", random_graph(20, 500, th.randint(0, 90, (20,), generator=g), 6)))
    # more nodes than edges, and the one long row (several chunks) sits at a node id above the edge count
    degs = th.zeros(1000, dtype=th.int64)
    degs[3], degs[400], degs[900], degs[999] = 7, 20, 300, 2
    zoo.append(("ids_above_edge_count", random_graph(1000, 1000, degs, 7)))
    return zoo


def chunked(g, chunk_size, transposed=False, dtype=None):
    """(row, indptr_, eid, indices) of one CSR orientation in the ops' argument order."""
    ip, idx, eid = (g.indptr_t, g.indices_t, g.eid_t) if transposed else (g.indptr, g.indices, g.eid)
    if chunk_size is None:
        row, ptr = unchunked_rows(ip)
    else:
        row, ptr = partition_csr(ip, chunk_size)
    dtype = dtype or idx.dtype
    return row.to(dtype), ptr.to(dtype), eid.to(dtype), idx.to(dtype)


def assert_close(actual, expected, rtol, atol, what=""):
    a = actual.detach().to("cpu", th.float64)
    b = expected.detach().to("cpu", th.float64)
    assert a.shape == b.shape, "%s: shape %s vs %s" % (what, tuple(a.shape), tuple(b.shape))
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = err > tol
    if bad.any():
        i = int(th.argmax(err - tol))
        raise AssertionError("%s: %d of %d elements out of tolerance (rtol %g atol %g); worst |%g - %g| = %g"
                             % (what, int(bad.sum()), a.numel(), rtol, atol, a.view(-1)[i], b.view(-1)[i],
                                err.view(-1)[i]))


def assert_rows_close(actual, expected, degree, rtol, atol, what=""):
    """Row r of `actual` against `expected`: |diff| <= rtol |expected| + atol * max(1, degree[r] / 256).

    Rows of at most 256 edges are held to (rtol, atol) as given; longer rows get an absolute allowance that grows
    with their edge count: an fp32 sum of n signed terms of size s picks up a rounding error of the order
    eps * n * s whatever order it is formed in (the reference's atomicAdd order included)."""
    a = actual.detach().to("cpu", th.float64)
    b = expected.detach().to("cpu", th.float64)
    assert a.shape == b.shape, "%s: shape %s vs %s" % (what, tuple(a.shape), tuple(b.shape))
    deg = th.as_tensor(degree).to("cpu", th.float64).clamp(min=256.0) / 256.0
    tol = rtol * b.abs() + atol * deg.view(-1, *([1] * (b.dim() - 1)))
    err = (a - b).abs()
    bad = err > tol
    if bad.any():
        i = int(th.argmax((err - tol).reshape(-1)))
        r = i // max(1, b[0].numel())
        raise AssertionError("%s: %d of %d elements out of tolerance (rtol %g atol %g); worst at row %d (degree %d): "
                             "|%g - %g| = %g" % (what, int(bad.sum()), a.numel(), rtol, atol, r, int(degree[r]),
                                                 a.reshape(-1)[i], b.reshape(-1)[i], err.reshape(-1)[i]))
