"""ctypes binding of libgraphop_b200.so, the C ABI declared in include/graphop_b200.h.

The library is loaded from this package's directory and nowhere else.  There is no
fallback: if the shared object is missing or a symbol cannot be resolved, importing the
ops fails with an error that says how to build it.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgraphop_b200.so")

OK, ERR_INVALID_ARGUMENT, ERR_WORKSPACE, ERR_UNSUPPORTED, ERR_CUDA = range(5)

OP_MASKEDMM_FWD, OP_MASKEDMM_BWD, OP_NODE_MUL_EDGE_FWD, OP_NODE_MUL_EDGE_BWD, OP_SOFTMAX_FWD, \
    OP_SOFTMAX_BWD, OP_SPMM_FWD, OP_SPMM_BWD, OP_ATTENTION_FWD, OP_ATTENTION_BWD, OP_ATTENTION_BWD_PAIRS = range(11)

ELEM_SUFFIXES = ("f32", "f64", "bf16")
INDEX_SUFFIXES = ("i32", "i64")

_P, _I64, _INT, _SZ, _DBL = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t, ctypes.c_double
_TAIL = [_P, _SZ, _P]  # workspace, workspace_bytes, stream

# argument lists of the typed entry points, in the order of include/graphop_b200.h
SIGNATURES = {
    "maskedmm_csr_forward": [_P] * 7 + [_I64] * 4 + [_INT] * 2 + _TAIL,
    "maskedmm_csr_backward": [_P] * 4 + [_I64] + [_P] * 4 + [_I64] + [_P] * 5 + [_I64] * 3 + [_INT] * 2 + _TAIL,
    "node_mul_edge_forward": [_P] * 6 + [_I64] * 3 + [_INT] * 2 + _TAIL,
    "node_mul_edge_backward": [_P] * 8 + [_I64] * 3 + [_INT] * 2 + _TAIL,
    "sparse_softmax_forward": [_P] * 5 + [_I64] * 3 + [_INT] + _TAIL,
    "sparse_softmax_backward": [_P] * 6 + [_I64] * 3 + [_INT] + _TAIL,
    "vector_spmm_forward": [_P] * 7 + [_I64] * 4 + [_INT] * 2 + _TAIL,
    "vector_spmm_backward": [_P] * 4 + [_I64] + [_P] * 4 + [_I64] + [_P] * 5 + [_I64] * 3 + [_INT] * 2 + _TAIL,
    "attention_forward": [_P] * 3 + [_I64] + [_P] * 3 + [_DBL] + [_P] * 2 + [_I64] * 3 + [_INT] * 2 + _TAIL,
    "attention_backward": [_P] * 3 + [_I64] + [_P] * 4 + [_I64] + [_P] * 6 + [_DBL] + [_P] * 3 + [_I64] * 3
                          + [_INT] * 2 + _TAIL,
    "attention_bias_forward": [_P] * 3 + [_I64] + [_P] * 4 + [_DBL] + [_P] * 2 + [_I64] * 3 + [_INT] * 2 + _TAIL,
    "attention_bias_backward": [_P] * 3 + [_I64] + [_P] * 4 + [_I64] + [_P] * 7 + [_DBL] + [_P] * 4 + [_I64] * 3
                               + [_INT] * 2 + _TAIL,
}

class Plan(ctypes.Structure):
    """graphop_plan_t of include/graphop_b200.h."""
    _fields_ = [("n_chunks", ctypes.c_int64), ("n_edges", ctypes.c_int64), ("n_nodes", ctypes.c_int64),
                ("header", ctypes.c_void_p), ("erow", ctypes.c_void_p), ("other", ctypes.c_void_p),
                ("eid", ctypes.c_void_p), ("node_lo", ctypes.c_void_p), ("node_deg", ctypes.c_void_p),
                ("flags", ctypes.c_int32), ("band_span", ctypes.c_int32), ("tile_start", ctypes.c_void_p),
                ("tile", ctypes.c_int32), ("reserved", ctypes.c_int32)]


PLAN_DENSE_BAND, PLAN_ROW_TILES, PLAN_NO_CARRY = 1, 2, 4
_PP = ctypes.POINTER(Plan)

# argument lists of the plan forms (one per element type), in the order of include/graphop_b200.h
PLANNED_SIGNATURES = {
    "maskedmm_csr_forward_planned": [_PP] + [_P] * 3 + [_I64] * 2 + [_INT] * 2 + _TAIL,
    "maskedmm_csr_backward_planned": [_PP] * 2 + [_P] * 5 + [_I64] * 2 + [_INT] * 2 + _TAIL,
    "node_mul_edge_forward_planned": [_PP] + [_P] * 3 + [_I64] + [_INT] * 2 + _TAIL,
    "node_mul_edge_backward_planned": [_PP] + [_P] * 5 + [_I64] + [_INT] * 2 + _TAIL,
    "sparse_softmax_forward_planned": [_PP] + [_P] * 2 + [_INT] + _TAIL,
    "sparse_softmax_backward_planned": [_PP] + [_P] * 3 + [_INT] + _TAIL,
    "vector_spmm_forward_planned": [_PP] + [_P] * 3 + [_I64] * 2 + [_INT] * 2 + _TAIL,
    "vector_spmm_backward_planned": [_PP] * 2 + [_P] * 5 + [_I64] * 2 + [_INT] * 2 + _TAIL,
    "attention_forward_planned": [_PP] + [_P] * 3 + [_DBL] + [_P] * 2 + [_I64] * 2 + [_INT] * 2 + _TAIL,
    "attention_backward_planned": [_PP] * 2 + [_P] * 6 + [_DBL] + [_P] * 3 + [_I64] * 2 + [_INT] * 2 + _TAIL,
}

UNTYPED = {
    "graphop_plan_bytes": ([_I64, _I64, _I64, _INT], _SZ),
    "graphop_plan_build_i32": ([_P] * 4 + [_I64] * 3 + [_P, _SZ, _PP, _P], _INT),
    "graphop_plan_build_i64": ([_P] * 4 + [_I64] * 3 + [_P, _SZ, _PP, _P], _INT),
    "graphop_version": ([], _INT),
    "graphop_error_string": ([_INT], ctypes.c_char_p),
    "graphop_last_cuda_error": ([], _INT),
    "graphop_workspace_bytes": ([_INT, _I64, _I64, _INT, _INT, _INT, _INT], _SZ),
    "graphop_static_scratch_bytes": ([], _SZ),
    "graphop_vector_spmm_forward_f32_i32_static": ([_P] * 7 + [_I64] * 4 + [_INT] * 2 + [_P], _INT),
    "graphop_gather_rows_i32": ([_P, _I64, _P, _I64, _P, _P], _INT),
    "graphop_pull_rows_i32": ([_P, _P, _INT, _P, _I64, _P, _P], _INT),
    "graphop_partition_csr_workspace_bytes": ([_I64], _SZ),
    "graphop_partition_csr_count_i32": ([_P, _I64, _I64, _P, _SZ, _P, _P], _INT),
    "graphop_partition_csr_count_i64": ([_P, _I64, _I64, _P, _SZ, _P, _P], _INT),
    "graphop_partition_csr_fill_i32": ([_P, _I64, _I64, _P, _I64, _P, _P, _P], _INT),
    "graphop_partition_csr_fill_i64": ([_P, _I64, _I64, _P, _I64, _P, _P, _P], _INT),
    "graphop_transpose_csr_workspace_bytes": ([_I64, _INT], _SZ),
    "graphop_transpose_csr_i32": ([_P, _P, _I64, _I64, _I64, _P, _P, _P, _P, _SZ, _P], _INT),
    "graphop_transpose_csr_i64": ([_P, _P, _I64, _I64, _I64, _P, _P, _P, _P, _SZ, _P], _INT),
    "graphop_check_graph_i32": ([_P] * 4 + [_I64] * 4 + [_P, _P], _INT),
    "graphop_check_graph_i64": ([_P] * 4 + [_I64] * 4 + [_P, _P], _INT),
}


DLPACK_ENTRY_POINTS = ["graphop_dl_" + op for op in (
    "maskedmm_csr_forward", "maskedmm_csr_backward", "node_mul_edge_forward", "node_mul_edge_backward",
    "sparse_softmax_forward", "sparse_softmax_backward", "vector_spmm_forward", "vector_spmm_backward",
    "attention_forward", "attention_backward")]   # include/graphop_dlpack.h; bound in dlpack_ops.py


def exported_symbols():
    """Every symbol include/graphop_b200.h and include/graphop_dlpack.h declare."""
    names = list(UNTYPED) + list(DLPACK_ENTRY_POINTS)
    for op in SIGNATURES:
        for e in ELEM_SUFFIXES:
            for i in INDEX_SUFFIXES:
                names.append("graphop_%s_%s_%s" % (op, e, i))
    for op in PLANNED_SIGNATURES:
        for e in ELEM_SUFFIXES:
            names.append("graphop_%s_%s" % (op, e))
    return names


_lib = None


def bind(handle, strict=True):
    """Sets argtypes / restype of every entry point of include/graphop_b200.h on a loaded library.
    strict=False skips symbols the library does not export (a build with fewer element types)."""
    for name, (args, res) in UNTYPED.items():
        fn = getattr(handle, name, None) if not strict else getattr(handle, name)
        if fn is not None:
            fn.argtypes, fn.restype = args, res
    for op, args in SIGNATURES.items():
        for e in ELEM_SUFFIXES:
            for i in INDEX_SUFFIXES:
                name = "graphop_%s_%s_%s" % (op, e, i)
                fn = getattr(handle, name, None) if not strict else getattr(handle, name)
                if fn is not None:
                    fn.argtypes, fn.restype = args, _INT
    for op, args in PLANNED_SIGNATURES.items():
        for e in ELEM_SUFFIXES:
            name = "graphop_%s_%s" % (op, e)
            fn = getattr(handle, name, None) if not strict else getattr(handle, name)
            if fn is not None:
                fn.argtypes, fn.restype = args, _INT
    return handle


def lib():
    """The loaded library with argtypes set; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "graphop_b200: %s is missing; build it with `python -m custom_op_benchmark_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback." % LIB_PATH)
    _lib = bind(ctypes.CDLL(LIB_PATH))
    return _lib


def error_message(code):
    handle = lib()
    msg = handle.graphop_error_string(code).decode()
    if code == ERR_CUDA:
        msg += " (cudaError %d)" % handle.graphop_last_cuda_error()
    return msg
