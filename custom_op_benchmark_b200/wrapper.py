"""Autograd wiring of the graphop ops: the four `torch.autograd.Function` classes of the
reference (wrapper.py:8-55) with the same names, the same positional `apply` signatures and
the same `None` gradients for every index argument, plus `GraphAttention`, the fused chain.
"""
import torch as th
from torch.autograd import Function

from . import graphop as _g
from .part_csr import partition_csr  # noqa: F401  (the reference wrapper re-exports it, wrapper.py:4)

__all__ = ["SparseSoftmax", "MaskedMMCSR", "NodeMulEdge", "VectorSPMM", "GraphAttention", "GraphAttentionBias", "GraphAttentionPlanned",
           "graph_attention", "partition_csr", "chunk_size"]

chunk_size = 32  # wrapper.py:6


class SparseSoftmax(Function):
    """wrapper.py:8-18"""

    @staticmethod
    def forward(ctx, row, indptr, eid, x):
        y = _g.sparse_softmax_forward(row, indptr, eid, x)
        ctx.save_for_backward(row, indptr, eid, y)
        return y

    @staticmethod
    def backward(ctx, dy):
        row, indptr, eid, y = ctx.saved_tensors
        return None, None, None, _g.sparse_softmax_backward(row, indptr, eid, y, dy.contiguous())


class MaskedMMCSR(Function):
    """wrapper.py:20-30"""

    @staticmethod
    def forward(ctx, row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B):
        ctx.save_for_backward(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B)
        return _g.maskedmm_csr_forward(row, indptr_r, eid_r, indices_r, A, B)

    @staticmethod
    def backward(ctx, grad):
        row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B = ctx.saved_tensors
        dA, dB = _g.maskedmm_csr_backward(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B,
                                          grad)
        return None, None, None, None, None, None, None, None, dA, dB


class NodeMulEdge(Function):
    """wrapper.py:32-42"""

    @staticmethod
    def forward(ctx, row, indptr, eid, A, B):
        ctx.save_for_backward(row, indptr, eid, A, B)
        return _g.node_mul_edge_forward(row, indptr, eid, A, B)

    @staticmethod
    def backward(ctx, grad):
        row, indptr, eid, A, B = ctx.saved_tensors
        dA, dB = _g.node_mul_edge_backward(row, indptr, eid, A, B, grad)
        return None, None, None, dA, dB


class VectorSPMM(Function):
    """wrapper.py:44-55"""

    @staticmethod
    def forward(ctx, row, indptr, eid, indices, col, ptr_t, eid_t, indices_t, edata, x):
        y = _g.vector_spmm_forward(row, indptr, eid, indices, edata, x)
        ctx.save_for_backward(row, indptr, eid, indices, col, ptr_t, eid_t, indices_t, edata, x)
        return y

    @staticmethod
    def backward(ctx, dy):
        row, indptr, eid, indices, col, ptr_t, eid_t, indices_t, edata, x = ctx.saved_tensors
        dedata, dx = _g.vector_spmm_backward(row, indptr, eid, indices, col, ptr_t, eid_t, indices_t, edata,
                                             dy.contiguous(), x)
        return None, None, None, None, None, None, None, None, dedata, dx


class GraphAttention(Function):
    """O = VectorSPMM(SparseSoftmax(scale * MaskedMMCSR(Q, K)), V) in one kernel per direction.

    ``apply(row, indptr, indices, col, indptr_t, indices_t, Q, K, V, scale, eid_t=None)``; no edge tensor is
    materialised and only the (n, h) log-sum-exp is saved.  ``eid_t`` (the transposed CSR's edge ids, valid
    when the row CSR's edge ids are its positions) lets the backward pass each edge's probability from its
    destination-side kernel to its source-side kernel instead of recomputing it."""

    @staticmethod
    def forward(ctx, row, indptr, indices, col, indptr_t, indices_t, Q, K, V, scale, eid_t=None):
        cached = getattr(_g, "cached_plan", None)
        if cached is not None and getattr(_g, "plan_cache_size", 0) > 0 and indices.numel() > 0:
            # the same graph tensors come back every step: their plans are built once and looked up here, so this
            # per-call signature runs the planned kernels (and, on a dense band in bfloat16, the tensor-core ones)
            ctx.plans = (cached(row, indptr, None, indices, Q.size(0)), cached(col, indptr_t, eid_t, indices_t, K.size(0)))
            o, lse = _g.attention_forward_planned(ctx.plans[0], Q, K, V, scale)
        else:
            ctx.plans = None
            o, lse = _g.attention_forward(row, indptr, indices, Q, K, V, scale)
        ctx.save_for_backward(row, indptr, indices, col, indptr_t, indices_t, Q, K, V, o, lse)
        ctx.scale = scale
        ctx.eid_t = eid_t
        return o

    @staticmethod
    def backward(ctx, d_o):
        row, indptr, indices, col, indptr_t, indices_t, Q, K, V, o, lse = ctx.saved_tensors
        if ctx.plans is not None:
            dq, dk, dv = _g.attention_backward_planned(ctx.plans[0], ctx.plans[1], Q, K, V, o, lse, d_o, ctx.scale)
        else:
            dq, dk, dv = _g.attention_backward(row, indptr, indices, col, indptr_t, indices_t, Q, K, V, o, lse, d_o,
                                               ctx.scale, eid_t=ctx.eid_t)
        return None, None, None, None, None, None, dq, dk, dv, None, None


class GraphAttentionBias(Function):
    """The attention layer with a relative-position term, fused:
    O = VectorSPMM(SparseSoftmax(scale * (MaskedMMCSR(Q, K) + NodeMulEdge(Q, rel))), V), the chain the reference's
    ops compose (wrapper.py:20-55) without the (e, h) score tensors.

    ``apply(row, indptr, indices, col, indptr_t, eid_t, indices_t, Q, K, V, rel, scale)``; ``rel`` is (e, d), one row
    per edge in row-CSR order, shared by the heads; ``eid_t`` gives for every position of the transposed CSR the
    row-CSR position of the same edge."""

    @staticmethod
    def forward(ctx, row, indptr, indices, col, indptr_t, eid_t, indices_t, Q, K, V, rel, scale):
        o, lse = _g.attention_bias_forward(row, indptr, indices, Q, K, V, rel, scale)
        ctx.save_for_backward(row, indptr, indices, col, indptr_t, eid_t, indices_t, Q, K, V, rel, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        row, indptr, indices, col, indptr_t, eid_t, indices_t, Q, K, V, rel, o, lse = ctx.saved_tensors
        dq, dk, dv, d_rel = _g.attention_bias_backward(row, indptr, indices, col, indptr_t, eid_t, indices_t, Q, K, V,
                                                       rel, o, lse, d_o, ctx.scale)
        return None, None, None, None, None, None, None, dq, dk, dv, d_rel, None


class GraphAttentionPlanned(Function):
    """GraphAttention on graph plans: ``apply(plan_r, plan_t, Q, K, V, scale)`` with ``graphop.GraphPlan`` objects of
    the row CSR and of the transposed CSR (the latter built with its edge ids).  Nothing that depends on the graph
    alone is recomputed per call."""

    @staticmethod
    def forward(ctx, plan_r, plan_t, Q, K, V, scale):
        o, lse = _g.attention_forward_planned(plan_r, Q, K, V, scale)
        ctx.save_for_backward(Q, K, V, o, lse)
        ctx.plans, ctx.scale = (plan_r, plan_t), scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        Q, K, V, o, lse = ctx.saved_tensors
        dq, dk, dv = _g.attention_backward_planned(ctx.plans[0], ctx.plans[1], Q, K, V, o, lse, d_o, ctx.scale)
        return None, None, dq, dk, dv, None


def graph_attention(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, Q, K, V, scale):
    """The attention chain with the argument list of the unfused ops: the fused kernels when the
    shape allows, otherwise MaskedMMCSR -> scale -> SparseSoftmax -> VectorSPMM."""
    if _g.attention_supported(Q):
        return GraphAttention.apply(row, indptr, indices, col, indptr_t, indices_t, Q, K, V, scale)
    s = MaskedMMCSR.apply(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, Q, K) * scale
    p = SparseSoftmax.apply(row, indptr, eid, s)
    return VectorSPMM.apply(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, p, V)
