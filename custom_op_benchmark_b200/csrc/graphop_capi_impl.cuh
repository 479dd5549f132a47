// Expands to the extern "C" entry points of one element type (see include/graphop_b200.h).
#pragma once
#include "gk_host.cuh"

#define GRAPHOP_DEFINE_OPS(SUF, CT, T, I)                                                                               \
  extern "C" int graphop_maskedmm_csr_forward_##SUF(                                                                 \
      const I* row, const I* indptr, const I* eid, const I* indices, const CT* A, const CT* B, CT* y,                \
      int64_t n_chunks, int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D, void* ws, size_t wsb,           \
      graphop_stream_t stream) {                                                                                     \
    return gk::maskedmm_forward<T, I>(row, indptr, eid, indices, (const T*)A, (const T*)B, (T*)y, n_chunks, n_edges, \
                                      n_dst, n_src, H, D, ws, wsb, (cudaStream_t)stream);                            \
  }                                                                                                                  \
  extern "C" int graphop_maskedmm_csr_backward_##SUF(                                                                \
      const I* row, const I* indptr_r, const I* eid_r, const I* indices_r, int64_t n_chunks_r, const I* col,         \
      const I* indptr_c, const I* eid_c, const I* indices_c, int64_t n_chunks_c, const CT* A, const CT* B,           \
      const CT* dy, CT* dA, CT* dB, int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D, void* ws,           \
      size_t wsb, graphop_stream_t stream) {                                                                         \
    return gk::maskedmm_backward<T, I>(row, indptr_r, eid_r, indices_r, n_chunks_r, col, indptr_c, eid_c, indices_c, \
                                       n_chunks_c, (const T*)A, (const T*)B, (const T*)dy, (T*)dA, (T*)dB, n_edges,  \
                                       n_dst, n_src, H, D, ws, wsb, (cudaStream_t)stream);                           \
  }                                                                                                                  \
  extern "C" int graphop_node_mul_edge_forward_##SUF(const I* row, const I* indptr, const I* eid, const CT* A,       \
                                                     const CT* B, CT* y, int64_t n_chunks, int64_t n_edges,          \
                                                     int64_t n_dst, int H, int D, void* ws, size_t wsb,              \
                                                     graphop_stream_t stream) {                                      \
    return gk::node_mul_edge_forward<T, I>(row, indptr, eid, (const T*)A, (const T*)B, (T*)y, n_chunks, n_edges,     \
                                           n_dst, H, D, ws, wsb, (cudaStream_t)stream);                              \
  }                                                                                                                  \
  extern "C" int graphop_node_mul_edge_backward_##SUF(const I* row, const I* indptr, const I* eid, const CT* A,      \
                                                      const CT* B, const CT* dy, CT* dA, CT* dB, int64_t n_chunks,   \
                                                      int64_t n_edges, int64_t n_dst, int H, int D, void* ws,        \
                                                      size_t wsb, graphop_stream_t stream) {                         \
    return gk::node_mul_edge_backward<T, I>(row, indptr, eid, (const T*)A, (const T*)B, (const T*)dy, (T*)dA,        \
                                            (T*)dB, n_chunks, n_edges, n_dst, H, D, ws, wsb, (cudaStream_t)stream);  \
  }                                                                                                                  \
  extern "C" int graphop_sparse_softmax_forward_##SUF(const I* row, const I* indptr, const I* eid, const CT* x,      \
                                                      CT* y, int64_t n_chunks, int64_t n_edges, int64_t n_nodes,     \
                                                      int H, void* ws, size_t wsb, graphop_stream_t stream) {        \
    return gk::sparse_softmax<T, I, false>(row, indptr, eid, (const T*)x, (const T*)nullptr, (T*)y, n_chunks,        \
                                           n_edges, n_nodes, H, ws, wsb, (cudaStream_t)stream);                      \
  }                                                                                                                  \
  extern "C" int graphop_sparse_softmax_backward_##SUF(const I* row, const I* indptr, const I* eid, const CT* y,     \
                                                       const CT* dy, CT* dx, int64_t n_chunks, int64_t n_edges,      \
                                                       int64_t n_nodes, int H, void* ws, size_t wsb,                 \
                                                       graphop_stream_t stream) {                                    \
    return gk::sparse_softmax<T, I, true>(row, indptr, eid, (const T*)y, (const T*)dy, (T*)dx, n_chunks, n_edges,    \
                                          n_nodes, H, ws, wsb, (cudaStream_t)stream);                                \
  }                                                                                                                  \
  extern "C" int graphop_vector_spmm_forward_##SUF(const I* row, const I* indptr, const I* eid, const I* indices,    \
                                                   const CT* edata, const CT* x, CT* y, int64_t n_chunks,            \
                                                   int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D,      \
                                                   void* ws, size_t wsb, graphop_stream_t stream) {                  \
    return gk::spmm_forward<T, I>(row, indptr, eid, indices, (const T*)edata, (const T*)x, (T*)y, n_chunks, n_edges, \
                                  n_dst, n_src, H, D, ws, wsb, (cudaStream_t)stream);                                \
  }                                                                                                                  \
  extern "C" int graphop_vector_spmm_backward_##SUF(                                                                 \
      const I* row, const I* indptr, const I* eid, const I* indices, int64_t n_chunks, const I* col,                 \
      const I* indptr_t, const I* eid_t, const I* indices_t, int64_t n_chunks_t, const CT* edata, const CT* dy,      \
      const CT* x, CT* dedata, CT* dx, int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D, void* ws,        \
      size_t wsb, graphop_stream_t stream) {                                                                         \
    return gk::spmm_backward<T, I>(row, indptr, eid, indices, n_chunks, col, indptr_t, eid_t, indices_t, n_chunks_t, \
                                   (const T*)edata, (const T*)dy, (const T*)x, (T*)dedata, (T*)dx, n_edges, n_dst,   \
                                   n_src, H, D, ws, wsb, (cudaStream_t)stream);                                      \
  }

#define GRAPHOP_DEFINE_ATTENTION(SUF, CT, T, I)                                                                      \
  extern "C" int graphop_attention_forward_##SUF(const I* row, const I* indptr, const I* indices, int64_t n_chunks,  \
                                                 const CT* q, const CT* k, const CT* v, double scale, CT* o,         \
                                                 void* lse, int64_t n_edges, int64_t n_dst, int64_t n_src, int H,    \
                                                 int D, void* ws, size_t wsb, graphop_stream_t stream) {             \
    return gk::attention_forward<T, I>(row, indptr, indices, n_chunks, (const T*)q, (const T*)k, (const T*)v, scale, \
                                       (T*)o, lse, n_edges, n_dst, n_src, H, D, ws, wsb, (cudaStream_t)stream);      \
  }                                                                                                                  \
  extern "C" int graphop_attention_backward_##SUF(                                                                   \
      const I* row, const I* indptr, const I* indices, int64_t n_chunks, const I* col, const I* indptr_t,            \
      const I* eid_t, const I* indices_t, int64_t n_chunks_t, const CT* q, const CT* k, const CT* v, const CT* o,    \
      const void* lse, const CT* d_o, double scale, CT* dq, CT* dk, CT* dv, int64_t n_edges, int64_t n_dst,          \
      int64_t n_src, int H, int D, void* ws, size_t wsb, graphop_stream_t stream) {                                  \
    return gk::attention_backward<T, I>(row, indptr, indices, n_chunks, col, indptr_t, eid_t, indices_t, n_chunks_t, \
                                        (const T*)q, (const T*)k, (const T*)v, (const T*)o, lse, (const T*)d_o,      \
                                        scale, (T*)dq, (T*)dk, (T*)dv, n_edges, n_dst, n_src, H, D, ws, wsb,         \
                                        (cudaStream_t)stream);                                                       \
  }
