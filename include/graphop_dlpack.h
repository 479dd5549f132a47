/*
 * graphop_b200, DLPack boundary: the operator set of graphop_b200.h taking DLPack tensor descriptors.
 *
 * The reference extension is bound to one framework (graphop/graphop.cpp takes at::Tensor) and names
 * "switch backend to dlpack" as its open item (README.md:5-7).  These entry points are that boundary: every
 * tensor argument is a DLTensor (dmlc/dlpack, dlpack.h: the struct every DLPack capsule carries), so any
 * producer of DLPack capsules - PyTorch, CuPy, JAX, TVM, a C program filling the struct by hand - can call the
 * kernels without a binding of its own.  Element type (float32, float64, bfloat16), index type (int32, int64)
 * and all sizes are read from the descriptors and dispatched to the typed entry points of graphop_b200.h; the
 * arithmetic and the results are theirs.
 *
 * Nothing is allocated and nothing is retained: outputs and the workspace are the caller's tensors, and the
 * descriptors are only read during the call.  Checked before anything is launched (GRAPHOP_ERR_INVALID_ARGUMENT):
 * every tensor on a CUDA device (kDLCUDA or kDLCUDAManaged) and all on the same one, compact row-major
 * (strides NULL or those of a contiguous tensor), lanes == 1, the index tensors of one integer type, the value
 * tensors of one float type, shapes consistent with each other.  The caller makes that device current and
 * orders `stream` after the producers of the inputs.
 *
 * Shapes follow the reference (graphop_b200.h): node tensors (n, H, D) or (n, D) for H = 1; edge tensors
 * (n_edges, H) or (n_edges) for H = 1; `row` (n_chunks), `indptr` (n_chunks + 1), `eid` / `indices` (n_edges).
 * `eid` may be NULL (the identity) wherever graphop_b200.h allows it.  The workspace is a tensor of any 1-byte
 * type with at least graphop_workspace_bytes(...) elements.
 */
#ifndef GRAPHOP_DLPACK_H_
#define GRAPHOP_DLPACK_H_

#include "graphop_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifdef DLPACK_VERSION
typedef DLTensor graphop_dltensor_t; /* dlpack.h was included first: use its type */
#else
/* Layout of DLTensor and its members as dlpack.h (0.2 - 1.x) defines them. */
typedef struct {
  int32_t device_type; /* 2 = kDLCUDA, 13 = kDLCUDAManaged are accepted */
  int32_t device_id;
} graphop_dldevice_t;
typedef struct {
  uint8_t code; /* 0 = kDLInt, 1 = kDLUInt, 2 = kDLFloat, 4 = kDLBfloat */
  uint8_t bits;
  uint16_t lanes;
} graphop_dldatatype_t;
typedef struct {
  void* data;
  graphop_dldevice_t device;
  int32_t ndim;
  graphop_dldatatype_t dtype;
  int64_t* shape;
  int64_t* strides; /* in elements; NULL = compact row-major */
  uint64_t byte_offset;
} graphop_dltensor_t;
#endif

/* graphop_maskedmm_csr_forward_*: A (n_dst, H, D), B (n_src, H, D), y (n_edges, H). */
int graphop_dl_maskedmm_csr_forward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                    const graphop_dltensor_t* eid, const graphop_dltensor_t* indices,
                                    const graphop_dltensor_t* A, const graphop_dltensor_t* B, graphop_dltensor_t* y,
                                    graphop_dltensor_t* workspace, graphop_stream_t stream);
/* graphop_maskedmm_csr_backward_*: dy (n_edges, H); dA like A, dB like B. */
int graphop_dl_maskedmm_csr_backward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr_r,
                                     const graphop_dltensor_t* eid_r, const graphop_dltensor_t* indices_r,
                                     const graphop_dltensor_t* col, const graphop_dltensor_t* indptr_c,
                                     const graphop_dltensor_t* eid_c, const graphop_dltensor_t* indices_c,
                                     const graphop_dltensor_t* A, const graphop_dltensor_t* B,
                                     const graphop_dltensor_t* dy, graphop_dltensor_t* dA, graphop_dltensor_t* dB,
                                     graphop_dltensor_t* workspace, graphop_stream_t stream);
/* graphop_node_mul_edge_forward_*: A (n_dst, H, D), B (n_edges, D), y (n_edges, H). */
int graphop_dl_node_mul_edge_forward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                     const graphop_dltensor_t* eid, const graphop_dltensor_t* A,
                                     const graphop_dltensor_t* B, graphop_dltensor_t* y,
                                     graphop_dltensor_t* workspace, graphop_stream_t stream);
int graphop_dl_node_mul_edge_backward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                      const graphop_dltensor_t* eid, const graphop_dltensor_t* A,
                                      const graphop_dltensor_t* B, const graphop_dltensor_t* dy,
                                      graphop_dltensor_t* dA, graphop_dltensor_t* dB, graphop_dltensor_t* workspace,
                                      graphop_stream_t stream);
/* graphop_sparse_softmax_*: x, y, dy, dx (n_edges, H); n_nodes bounds node id + 1. */
int graphop_dl_sparse_softmax_forward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                      const graphop_dltensor_t* eid, const graphop_dltensor_t* x,
                                      graphop_dltensor_t* y, int64_t n_nodes, graphop_dltensor_t* workspace,
                                      graphop_stream_t stream);
int graphop_dl_sparse_softmax_backward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                       const graphop_dltensor_t* eid, const graphop_dltensor_t* y,
                                       const graphop_dltensor_t* dy, graphop_dltensor_t* dx, int64_t n_nodes,
                                       graphop_dltensor_t* workspace, graphop_stream_t stream);
/* graphop_vector_spmm_*: edata (n_edges, H), x (n_src, H, D), y / dy (n_dst, H, D). */
int graphop_dl_vector_spmm_forward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                   const graphop_dltensor_t* eid, const graphop_dltensor_t* indices,
                                   const graphop_dltensor_t* edata, const graphop_dltensor_t* x,
                                   graphop_dltensor_t* y, graphop_dltensor_t* workspace, graphop_stream_t stream);
int graphop_dl_vector_spmm_backward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                    const graphop_dltensor_t* eid, const graphop_dltensor_t* indices,
                                    const graphop_dltensor_t* col, const graphop_dltensor_t* indptr_t,
                                    const graphop_dltensor_t* eid_t, const graphop_dltensor_t* indices_t,
                                    const graphop_dltensor_t* edata, const graphop_dltensor_t* dy,
                                    const graphop_dltensor_t* x, graphop_dltensor_t* dedata, graphop_dltensor_t* dx,
                                    graphop_dltensor_t* workspace, graphop_stream_t stream);
/* graphop_attention_forward_*: q, o (n_dst, H, D), k, v (n_src, H, D), lse (n_dst, H) float32 (float64 for
 * float64 values). */
int graphop_dl_attention_forward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                 const graphop_dltensor_t* indices, const graphop_dltensor_t* q,
                                 const graphop_dltensor_t* k, const graphop_dltensor_t* v, double scale,
                                 graphop_dltensor_t* o, graphop_dltensor_t* lse, graphop_dltensor_t* workspace,
                                 graphop_stream_t stream);
/* graphop_attention_backward_*; eid_t may be NULL. */
int graphop_dl_attention_backward(const graphop_dltensor_t* row, const graphop_dltensor_t* indptr,
                                  const graphop_dltensor_t* indices, const graphop_dltensor_t* col,
                                  const graphop_dltensor_t* indptr_t, const graphop_dltensor_t* eid_t,
                                  const graphop_dltensor_t* indices_t, const graphop_dltensor_t* q,
                                  const graphop_dltensor_t* k, const graphop_dltensor_t* v,
                                  const graphop_dltensor_t* o, const graphop_dltensor_t* lse,
                                  const graphop_dltensor_t* d_o, double scale, graphop_dltensor_t* dq,
                                  graphop_dltensor_t* dk, graphop_dltensor_t* dv, graphop_dltensor_t* workspace,
                                  graphop_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GRAPHOP_DLPACK_H_ */
