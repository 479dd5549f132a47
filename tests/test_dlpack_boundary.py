"""The DLPack boundary without a GPU: host tensors are refused from their descriptors alone, before any CUDA
call is made."""
import pytest
import torch as th

from helpers import chunked, graph_zoo
from custom_op_benchmark_b200 import _capi, dlpack_ops as dl


def test_host_tensors_are_refused():
    g = graph_zoo()[0][1]
    r = chunked(g, 32, dtype=th.int32)
    A, B = th.randn(g.n_dst, 2, 8), th.randn(g.n_src, 2, 8)
    y, ws = th.empty(g.n_edges, 2), th.empty(4096, dtype=th.uint8)
    with pytest.raises(RuntimeError, match="invalid argument"):
        dl.maskedmm_csr_forward(*r, A, B, y, ws)
    with pytest.raises(RuntimeError, match="invalid argument"):
        dl.sparse_softmax_forward(*r[:3], y, y.clone(), g.n_dst, ws)


def test_descriptor_layout_matches_dlpack():
    """The ctypes mirror of DLTensor reads a torch capsule correctly: pointer, dtype, shape."""
    import ctypes
    x = th.arange(24, dtype=th.float32).reshape(2, 3, 4)
    cap = x.__dlpack__()
    t = ctypes.cast(dl._get_pointer(cap, b"dltensor"), dl._T).contents
    assert t.data == x.data_ptr() and t.ndim == 3 and [t.shape[i] for i in range(3)] == [2, 3, 4]
    assert (t.dtype.code, t.dtype.bits, t.dtype.lanes) == (2, 32, 1) and t.device.device_type == 1
    b = th.zeros(3, dtype=th.bfloat16).__dlpack__()
    tb = ctypes.cast(dl._get_pointer(b, b"dltensor"), dl._T).contents
    assert (tb.dtype.code, tb.dtype.bits) == (4, 16)


def test_every_dlpack_entry_point_is_bound_with_its_arity():
    text = open(__import__("os").path.join(__import__("helpers").ROOT, "include", "graphop_dlpack.h")).read()
    import re
    for name, kinds in dl.DL_SIGNATURES.items():
        decl = re.search(r"int %s\((.*?)\);" % name, text, re.S).group(1)
        assert len(decl.split(",")) == len(kinds) + 1, name       # + the stream
    assert sorted(dl.DL_SIGNATURES) == sorted(_capi.DLPACK_ENTRY_POINTS)
