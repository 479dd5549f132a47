"""Generators and CSR plumbing: shapes, sortedness, both orientations describe one edge set."""
import torch as th

from custom_op_benchmark_b200 import graphs


def _check(g):
    e = g.n_edges
    assert g.indptr.numel() == g.n_dst + 1 and g.indptr_t.numel() == g.n_src + 1
    assert int(g.indptr[-1]) == e and int(g.indptr_t[-1]) == e
    assert th.equal(g.eid.long(), th.arange(e))
    assert th.equal(th.sort(g.eid_t.long()).values, th.arange(e))  # a true permutation
    dst = g.dst_of_edge()
    src = g.indices.long()
    # transposed position p holds edge eid_t[p]: its source is the transposed row, its destination indices_t[p]
    src_t = th.repeat_interleave(th.arange(g.n_src), (g.indptr_t[1:] - g.indptr_t[:-1]).long())
    assert th.equal(src[g.eid_t.long()], src_t)
    assert th.equal(dst[g.eid_t.long()], g.indices_t.long())
    key = dst * g.n_src + src
    assert bool((key[1:] >= key[:-1]).all())


def test_er_graph():
    g = graphs.er_graph(256, 15, seed=0)
    _check(g)
    assert g.n_edges == 256 * 16
    deg = g.indptr[1:] - g.indptr[:-1]
    assert bool((deg == 16).all())
    dst, src = g.dst_of_edge(), g.indices.long()
    assert int((dst == src).sum()) == 256                       # exactly one self-loop per node
    assert th.unique(dst * 256 + src).numel() == g.n_edges      # no duplicate edge


def test_banded_graph_counts():
    g = graphs.banded_graph(batch=2, length=512, window=16)
    _check(g)
    per = sum(min(511, i + 16) - max(0, i - 16) + 1 for i in range(512))
    assert g.n_edges == 2 * per
    # the full-size configuration: 4 x 8192 rows, window 128 -> 2,088,832 edges per sequence
    assert sum(min(8191, i + 128) - max(0, i - 128) + 1 for i in range(8192)) == 2_088_832


def test_block_diagonal_matches_reference_formulas():
    b, l = 3, 5
    g = graphs.block_diagonal_graph(b, l)
    _check(g)
    # wrapper.py:104-112: column CSR position cnt -> eid_c = b*l*l + (x % l)*l + (y % l)
    cnt, want_idx, want_eid = 0, [], []
    for bb in range(b):
        for y in range(bb * l, (bb + 1) * l):
            for x in range(bb * l, (bb + 1) * l):
                want_idx.append(x)
                want_eid.append(bb * l * l + (x % l) * l + (y % l))
    assert g.indices_t.tolist() == want_idx and g.eid_t.tolist() == want_eid


def test_rmat_small():
    g = graphs.rmat_graph(10, 8, seed=0)
    _check(g)
    n = 1024
    dst, src = g.dst_of_edge(), g.indices.long()
    assert int((dst == src).sum()) == n
    assert th.unique(dst * n + src).numel() == g.n_edges
    deg = (g.indptr[1:] - g.indptr[:-1]).long()
    assert int(deg.max()) > 20 * int(deg.median())  # skewed
    g2 = graphs.rmat_graph(10, 8, seed=0)
    assert th.equal(g.indices, g2.indices) and th.equal(g.indptr, g2.indptr)


def test_zipf_degrees_and_graph():
    deg = graphs.zipf_degrees(2000, 100_000, 1.1, cap=20_000)
    assert abs(int(deg.sum()) - 100_000) <= 2000 and deg.min() >= 1 and deg.max() <= 20_000
    g = graphs.zipf_graph(2000, 100_000, 1.1, cap=20_000, seed=0)
    _check(g)
    assert g.n_edges == int(deg.sum())
