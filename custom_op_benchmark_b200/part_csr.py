"""CSR row chunker: the `(row, indptr_)` format every graphop op consumes.

Mirrors ``partition_csr(indptr, chunk_size=32)`` of the reference
(part_csr.py:13-27): each CSR row ``[indptr[r], indptr[r+1])`` is cut into
consecutive chunks of at most ``chunk_size`` positions; ``row[c]`` is the row
that owns chunk ``c``, ``indptr_[c]`` its first position, and a final sentinel
equal to ``indptr[-1]`` closes the last chunk.  Rows with no edges emit no
chunk.  Both outputs are int64 on the input's device, whatever the input
integer dtype.

The reference walks the rows in a Python double loop after copying the array
to the host (part_csr.py:15-21), which is O(N + C) interpreter steps.  Here an
int32 / int64 indptr on a CUDA device goes through the library's own kernels
(csrc/graphop_capi_prep.cu: chunk counts, a prefix sum, one thread per chunk);
anything else (host tensors, other integer types) through a handful of tensor
ops.  Both are bit-exact with the loop.  One deliberate deviation: for a graph with no edges at all the
reference returns ``row`` as an empty *float32* tensor (an artefact of
``th.tensor([])``, part_csr.py:24); here ``row`` is an empty int64 tensor.
"""
import torch as th

__all__ = ["partition_csr", "partition_csr_tensor_ops", "unchunked_rows"]


def partition_csr(indptr, chunk_size=32):
    if chunk_size <= 0:
        # range(a, b, 0) raises ValueError in the reference loop (part_csr.py:19)
        raise ValueError("chunk_size must be positive")
    if indptr.is_cuda and indptr.dtype in (th.int32, th.int64) and indptr.dim() == 1 and indptr.numel() >= 1:
        from . import graphop   # the CUDA library; raises if it has not been built
        return graphop.partition_csr(indptr, chunk_size)
    return partition_csr_tensor_ops(indptr, chunk_size)


def partition_csr_tensor_ops(indptr, chunk_size=32):
    """The same table by tensor ops on the input's device (the host path, and the checker of the kernels)."""
    if chunk_size <= 0:
        raise ValueError("chunk_size must be positive")
    device = indptr.device
    ip = indptr.to(th.int64)
    n = ip.numel() - 1
    if n < 0:
        raise IndexError("indptr must hold at least one element")
    last = ip[-1:].clone()
    if n == 0:
        return th.empty(0, dtype=th.int64, device=device), last
    start = ip[:-1]
    deg = (ip[1:] - start).clamp_(min=0)  # range(a, b, cs) is empty when b <= a
    nch = (deg + (chunk_size - 1)) // chunk_size
    row = th.repeat_interleave(th.arange(n, dtype=th.int64, device=device), nch)
    first = th.cumsum(nch, 0) - nch  # index of each row's first chunk
    k = th.arange(row.numel(), dtype=th.int64, device=device) - first[row]
    indptr_ = th.cat([start[row] + k * chunk_size, last])
    return row, indptr_


def unchunked_rows(indptr):
    """The un-chunked form the ops also accept: one chunk per row, empty rows included.

    Returns ``(arange(N), indptr)`` as int64, so a plain CSR can be passed to any op
    without calling ``partition_csr`` first.
    """
    ip = indptr.to(th.int64)
    return th.arange(ip.numel() - 1, dtype=th.int64, device=ip.device), ip
