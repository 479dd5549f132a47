"""partition_csr: bit-exact against the reference's outputs (golden JSON made by running
part_csr.py:13-27 itself) and against the oracle's loop restatement on random inputs."""
import json
import os

import pytest
import torch as th
from hypothesis import given, settings, strategies as st

from helpers import ROOT
from custom_op_benchmark_b200.part_csr import partition_csr, unchunked_rows
from oracle.graphop_oracle import partition_csr_loop

GOLDEN = json.load(open(os.path.join(ROOT, "tests", "golden", "partition_csr.json")))


@pytest.mark.parametrize("case", GOLDEN, ids=lambda c: "cs%d_n%d" % (c["chunk_size"], len(c["indptr"]) - 1))
def test_matches_reference_golden(case):
    dt = th.int32 if case.get("input_dtype") == "torch.int32" else th.int64
    row, ptr = partition_csr(th.tensor(case["indptr"], dtype=dt), case["chunk_size"])
    assert row.dtype == th.int64 and ptr.dtype == th.int64  # int64 out whatever comes in
    assert row.tolist() == case["row"]
    assert ptr.tolist() == case["indptr_"]
    assert case["indptr_dtype"] == "torch.int64"
    if case["row"]:
        assert case["row_dtype"] == "torch.int64"
    else:
        # the reference returns an empty float32 `row` here (th.tensor([])); int64 is the
        # deliberate deviation
        assert case["row_dtype"] == "torch.float32"


@pytest.mark.parametrize("case", GOLDEN[:6], ids=lambda c: "cs%d" % c["chunk_size"])
def test_oracle_loop_matches_reference_golden(case):
    row, ptr = partition_csr_loop(case["indptr"], case["chunk_size"])
    assert row == case["row"] and ptr == case["indptr_"]


@settings(max_examples=150, deadline=None)
@given(st.lists(st.integers(0, 90), min_size=0, max_size=60), st.integers(1, 40), st.integers(0, 7))
def test_matches_loop_on_random_rows(degs, chunk_size, base):
    ip = [base]
    for d in degs:
        ip.append(ip[-1] + d)
    row, ptr = partition_csr(th.tensor(ip), chunk_size)
    erow, eptr = partition_csr_loop(ip, chunk_size)
    assert row.tolist() == erow and ptr.tolist() == eptr
    # structural properties: chunks tile [ip[0], ip[-1]) in order, none longer than chunk_size
    ln = ptr[1:] - ptr[:-1]
    assert bool((ln > 0).all()) and bool((ln <= chunk_size).all())
    assert int(ptr[-1]) == ip[-1]
    assert bool((row[1:] >= row[:-1]).all())


def test_rejects_bad_chunk_size():
    with pytest.raises(ValueError):
        partition_csr(th.tensor([0, 3]), 0)


def test_large_graph_is_fast_and_consistent():
    g = th.Generator().manual_seed(0)
    deg = th.randint(0, 70, (200_000,), generator=g)
    ip = th.cat([th.zeros(1, dtype=th.long), th.cumsum(deg, 0)])
    row, ptr = partition_csr(ip, 32)
    nch = (deg + 31) // 32
    assert row.numel() == int(nch.sum())
    assert th.equal(th.bincount(row, minlength=deg.numel()), nch)
    assert th.equal(ptr[:-1][th.cumsum(nch, 0)[:-1][nch[1:] > 0]], ip[1:-1][nch[1:] > 0])


def test_unchunked_rows():
    row, ptr = unchunked_rows(th.tensor([0, 2, 2, 5], dtype=th.int32))
    assert row.tolist() == [0, 1, 2] and ptr.tolist() == [0, 2, 2, 5] and ptr.dtype == th.int64
