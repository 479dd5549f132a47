// Expands to the extern "C" entry points of one element type (see include/graphop_b200.h): the chunk-table
// forms GRAPHOP_DEFINE_OPS / GRAPHOP_DEFINE_ATTENTION / GRAPHOP_DEFINE_ATTENTION_BIAS per index type, and the plan forms
// GRAPHOP_DEFINE_PLANNED_OPS / GRAPHOP_DEFINE_PLANNED_ATTENTION once per element type.
#pragma once
#include "gk_host.cuh"

#define GK_CH(I, row, indptr, eid, indices, C, E) gk::FromChunks<I>{row, indptr, eid, indices, (long long)(C), (long long)(E)}
#define GK_ST (cudaStream_t)stream

#define GRAPHOP_DEFINE_OPS(SUF, CT, T, I)                                                                               \
  extern "C" int graphop_maskedmm_csr_forward_##SUF(                                                                 \
      const I* row, const I* indptr, const I* eid, const I* indices, const CT* A, const CT* B, CT* y,                \
      int64_t n_chunks, int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D, void* ws, size_t wsb,           \
      graphop_stream_t stream) {                                                                                     \
    return gk::maskedmm_forward<T>(GK_CH(I, row, indptr, eid, indices, n_chunks, n_edges), (const T*)A, (const T*)B, \
                                   (T*)y, n_chunks, n_edges, n_dst, n_src, H, D, ws, wsb, GK_ST);                    \
  }                                                                                                                  \
  extern "C" int graphop_maskedmm_csr_backward_##SUF(                                                                \
      const I* row, const I* indptr_r, const I* eid_r, const I* indices_r, int64_t n_chunks_r, const I* col,         \
      const I* indptr_c, const I* eid_c, const I* indices_c, int64_t n_chunks_c, const CT* A, const CT* B,           \
      const CT* dy, CT* dA, CT* dB, int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D, void* ws,           \
      size_t wsb, graphop_stream_t stream) {                                                                         \
    return gk::maskedmm_backward<T>(GK_CH(I, row, indptr_r, eid_r, indices_r, n_chunks_r, n_edges),                  \
                                    GK_CH(I, col, indptr_c, eid_c, indices_c, n_chunks_c, n_edges), n_chunks_r,      \
                                    n_chunks_c, (const T*)A, (const T*)B, (const T*)dy, (T*)dA, (T*)dB, n_edges,     \
                                    n_dst, n_src, H, D, ws, wsb, GK_ST);                                             \
  }                                                                                                                  \
  extern "C" int graphop_node_mul_edge_forward_##SUF(const I* row, const I* indptr, const I* eid, const CT* A,       \
                                                     const CT* B, CT* y, int64_t n_chunks, int64_t n_edges,          \
                                                     int64_t n_dst, int H, int D, void* ws, size_t wsb,              \
                                                     graphop_stream_t stream) {                                      \
    return gk::node_mul_edge_forward<T>(GK_CH(I, row, indptr, eid, (const I*)nullptr, n_chunks, n_edges),            \
                                        (const T*)A, (const T*)B, (T*)y, n_chunks, n_edges, n_dst, H, D, ws, wsb,    \
                                        GK_ST);                                                                      \
  }                                                                                                                  \
  extern "C" int graphop_node_mul_edge_backward_##SUF(const I* row, const I* indptr, const I* eid, const CT* A,      \
                                                      const CT* B, const CT* dy, CT* dA, CT* dB, int64_t n_chunks,   \
                                                      int64_t n_edges, int64_t n_dst, int H, int D, void* ws,        \
                                                      size_t wsb, graphop_stream_t stream) {                         \
    return gk::node_mul_edge_backward<T>(GK_CH(I, row, indptr, eid, (const I*)nullptr, n_chunks, n_edges),           \
                                         (const T*)A, (const T*)B, (const T*)dy, (T*)dA, (T*)dB, n_chunks, n_edges,  \
                                         n_dst, H, D, ws, wsb, GK_ST);                                               \
  }                                                                                                                  \
  extern "C" int graphop_sparse_softmax_forward_##SUF(const I* row, const I* indptr, const I* eid, const CT* x,      \
                                                      CT* y, int64_t n_chunks, int64_t n_edges, int64_t n_nodes,     \
                                                      int H, void* ws, size_t wsb, graphop_stream_t stream) {        \
    return gk::sparse_softmax<T, false>(GK_CH(I, row, indptr, eid, (const I*)nullptr, n_chunks, n_edges),            \
                                        (const T*)x, (const T*)nullptr, (T*)y, n_chunks, n_edges, n_nodes, H, ws,    \
                                        wsb, GK_ST);                                                                 \
  }                                                                                                                  \
  extern "C" int graphop_sparse_softmax_backward_##SUF(const I* row, const I* indptr, const I* eid, const CT* y,     \
                                                       const CT* dy, CT* dx, int64_t n_chunks, int64_t n_edges,      \
                                                       int64_t n_nodes, int H, void* ws, size_t wsb,                 \
                                                       graphop_stream_t stream) {                                    \
    return gk::sparse_softmax<T, true>(GK_CH(I, row, indptr, eid, (const I*)nullptr, n_chunks, n_edges),             \
                                       (const T*)y, (const T*)dy, (T*)dx, n_chunks, n_edges, n_nodes, H, ws, wsb,    \
                                       GK_ST);                                                                       \
  }                                                                                                                  \
  extern "C" int graphop_vector_spmm_forward_##SUF(const I* row, const I* indptr, const I* eid, const I* indices,    \
                                                   const CT* edata, const CT* x, CT* y, int64_t n_chunks,            \
                                                   int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D,      \
                                                   void* ws, size_t wsb, graphop_stream_t stream) {                  \
    return gk::spmm_forward<T>(GK_CH(I, row, indptr, eid, indices, n_chunks, n_edges), (const T*)edata,              \
                               (const T*)x, (T*)y, n_chunks, n_edges, n_dst, n_src, H, D, ws, wsb, GK_ST);           \
  }                                                                                                                  \
  extern "C" int graphop_vector_spmm_backward_##SUF(                                                                 \
      const I* row, const I* indptr, const I* eid, const I* indices, int64_t n_chunks, const I* col,                 \
      const I* indptr_t, const I* eid_t, const I* indices_t, int64_t n_chunks_t, const CT* edata, const CT* dy,      \
      const CT* x, CT* dedata, CT* dx, int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D, void* ws,        \
      size_t wsb, graphop_stream_t stream) {                                                                         \
    return gk::spmm_backward<T>(GK_CH(I, row, indptr, eid, indices, n_chunks, n_edges),                              \
                                GK_CH(I, col, indptr_t, eid_t, indices_t, n_chunks_t, n_edges), n_chunks,            \
                                n_chunks_t, (const T*)edata, (const T*)dy, (const T*)x, (T*)dedata, (T*)dx, n_edges, \
                                n_dst, n_src, H, D, ws, wsb, GK_ST);                                                 \
  }

#define GRAPHOP_DEFINE_ATTENTION(SUF, CT, T, I)                                                                      \
  extern "C" int graphop_attention_forward_##SUF(const I* row, const I* indptr, const I* indices, int64_t n_chunks,  \
                                                 const CT* q, const CT* k, const CT* v, double scale, CT* o,         \
                                                 void* lse, int64_t n_edges, int64_t n_dst, int64_t n_src, int H,    \
                                                 int D, void* ws, size_t wsb, graphop_stream_t stream) {             \
    return gk::attention_forward<T>(GK_CH(I, row, indptr, (const I*)nullptr, indices, n_chunks, n_edges), n_chunks,  \
                                    (const T*)q, (const T*)k, (const T*)v, scale, (T*)o, lse, n_edges, n_dst,        \
                                    n_src, H, D, ws, wsb, GK_ST);                                                    \
  }                                                                                                                  \
  extern "C" int graphop_attention_backward_##SUF(                                                                   \
      const I* row, const I* indptr, const I* indices, int64_t n_chunks, const I* col, const I* indptr_t,            \
      const I* eid_t, const I* indices_t, int64_t n_chunks_t, const CT* q, const CT* k, const CT* v, const CT* o,    \
      const void* lse, const CT* d_o, double scale, CT* dq, CT* dk, CT* dv, int64_t n_edges, int64_t n_dst,          \
      int64_t n_src, int H, int D, void* ws, size_t wsb, graphop_stream_t stream) {                                  \
    return gk::attention_backward<T>(GK_CH(I, row, indptr, (const I*)nullptr, indices, n_chunks, n_edges),           \
                                     GK_CH(I, col, indptr_t, eid_t, indices_t, n_chunks_t, n_edges),                 \
                                     eid_t != nullptr, n_chunks, n_chunks_t, (const T*)q, (const T*)k, (const T*)v,  \
                                     (const T*)o, lse, (const T*)d_o, scale, (T*)dq, (T*)dk, (T*)dv, n_edges, n_dst, \
                                     n_src, H, D, ws, wsb, GK_ST);                                                   \
  }

#define GRAPHOP_DEFINE_ATTENTION_BIAS(SUF, CT, T, I)                                                                 \
  extern "C" int graphop_attention_bias_forward_##SUF(                                                               \
      const I* row, const I* indptr, const I* indices, int64_t n_chunks, const CT* q, const CT* k, const CT* v,      \
      const CT* rel, double scale, CT* o, void* lse, int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D,    \
      void* ws, size_t wsb, graphop_stream_t stream) {                                                               \
    return gk::attention_bias_forward<T>(GK_CH(I, row, indptr, (const I*)nullptr, indices, n_chunks, n_edges),       \
                                         n_chunks, (const T*)q, (const T*)k, (const T*)v, (const T*)rel, scale,      \
                                         (T*)o, lse, n_edges, n_dst, n_src, H, D, ws, wsb, GK_ST);                   \
  }                                                                                                                  \
  extern "C" int graphop_attention_bias_backward_##SUF(                                                              \
      const I* row, const I* indptr, const I* indices, int64_t n_chunks, const I* col, const I* indptr_t,            \
      const I* eid_t, const I* indices_t, int64_t n_chunks_t, const CT* q, const CT* k, const CT* v, const CT* rel,  \
      const CT* o, const void* lse, const CT* d_o, double scale, CT* dq, CT* dk, CT* dv, CT* d_rel,                  \
      int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D, void* ws, size_t wsb, graphop_stream_t stream) {  \
    return gk::attention_bias_backward<T>(GK_CH(I, row, indptr, (const I*)nullptr, indices, n_chunks, n_edges),      \
                                          GK_CH(I, col, indptr_t, eid_t, indices_t, n_chunks_t, n_edges),            \
                                          eid_t != nullptr, n_chunks, n_chunks_t, (const T*)q, (const T*)k,          \
                                          (const T*)v, (const T*)rel, (const T*)o, lse, (const T*)d_o, scale,        \
                                          (T*)dq, (T*)dk, (T*)dv, (T*)d_rel, n_edges, n_dst, n_src, H, D, ws, wsb,   \
                                          GK_ST);                                                                    \
  }

// The same operations on plans (graphop_plan_build_*): the owner table and the 32-bit index copies come from the
// plan instead of being rebuilt in the workspace by every call.
#define GK_PL(plan) gk::FromPlan{plan}
#define GK_PE(plan) ((plan) ? (plan)->n_edges : -1)
#define GK_PC(plan) ((plan) ? (plan)->n_chunks : -1)

#define GRAPHOP_DEFINE_PLANNED_OPS(SUF, CT, T)                                                                       \
  extern "C" int graphop_maskedmm_csr_forward_planned_##SUF(const graphop_plan_t* plan, const CT* A, const CT* B,    \
                                                            CT* y, int64_t n_dst, int64_t n_src, int H, int D,       \
                                                            void* ws, size_t wsb, graphop_stream_t stream) {         \
    return gk::maskedmm_forward<T>(GK_PL(plan), (const T*)A, (const T*)B, (T*)y, GK_PC(plan), GK_PE(plan), n_dst,    \
                                   n_src, H, D, ws, wsb, GK_ST);                                                     \
  }                                                                                                                  \
  extern "C" int graphop_maskedmm_csr_backward_planned_##SUF(const graphop_plan_t* plan_r,                           \
                                                             const graphop_plan_t* plan_c, const CT* A, const CT* B, \
                                                             const CT* dy, CT* dA, CT* dB, int64_t n_dst,            \
                                                             int64_t n_src, int H, int D, void* ws, size_t wsb,      \
                                                             graphop_stream_t stream) {                              \
    return gk::maskedmm_backward<T>(GK_PL(plan_r), GK_PL(plan_c), GK_PC(plan_r), GK_PC(plan_c), (const T*)A,         \
                                    (const T*)B, (const T*)dy, (T*)dA, (T*)dB, GK_PE(plan_r), n_dst, n_src, H, D,    \
                                    ws, wsb, GK_ST);                                                                 \
  }                                                                                                                  \
  extern "C" int graphop_node_mul_edge_forward_planned_##SUF(const graphop_plan_t* plan, const CT* A, const CT* B,   \
                                                             CT* y, int64_t n_dst, int H, int D, void* ws,           \
                                                             size_t wsb, graphop_stream_t stream) {                  \
    return gk::node_mul_edge_forward<T>(GK_PL(plan), (const T*)A, (const T*)B, (T*)y, GK_PC(plan), GK_PE(plan),      \
                                        n_dst, H, D, ws, wsb, GK_ST);                                                \
  }                                                                                                                  \
  extern "C" int graphop_node_mul_edge_backward_planned_##SUF(const graphop_plan_t* plan, const CT* A, const CT* B,  \
                                                              const CT* dy, CT* dA, CT* dB, int64_t n_dst, int H,    \
                                                              int D, void* ws, size_t wsb,                           \
                                                              graphop_stream_t stream) {                             \
    return gk::node_mul_edge_backward<T>(GK_PL(plan), (const T*)A, (const T*)B, (const T*)dy, (T*)dA, (T*)dB,        \
                                         GK_PC(plan), GK_PE(plan), n_dst, H, D, ws, wsb, GK_ST);                     \
  }                                                                                                                  \
  extern "C" int graphop_sparse_softmax_forward_planned_##SUF(const graphop_plan_t* plan, const CT* x, CT* y, int H, \
                                                              void* ws, size_t wsb, graphop_stream_t stream) {       \
    return gk::sparse_softmax<T, false>(GK_PL(plan), (const T*)x, (const T*)nullptr, (T*)y, GK_PC(plan),             \
                                        GK_PE(plan), plan ? plan->n_nodes : 0, H, ws, wsb, GK_ST);                   \
  }                                                                                                                  \
  extern "C" int graphop_sparse_softmax_backward_planned_##SUF(const graphop_plan_t* plan, const CT* y,              \
                                                               const CT* dy, CT* dx, int H, void* ws, size_t wsb,    \
                                                               graphop_stream_t stream) {                            \
    return gk::sparse_softmax<T, true>(GK_PL(plan), (const T*)y, (const T*)dy, (T*)dx, GK_PC(plan), GK_PE(plan),     \
                                       plan ? plan->n_nodes : 0, H, ws, wsb, GK_ST);                                 \
  }                                                                                                                  \
  extern "C" int graphop_vector_spmm_forward_planned_##SUF(const graphop_plan_t* plan, const CT* edata, const CT* x, \
                                                           CT* y, int64_t n_dst, int64_t n_src, int H, int D,        \
                                                           void* ws, size_t wsb, graphop_stream_t stream) {          \
    return gk::spmm_forward<T>(GK_PL(plan), (const T*)edata, (const T*)x, (T*)y, GK_PC(plan), GK_PE(plan), n_dst,    \
                               n_src, H, D, ws, wsb, GK_ST);                                                         \
  }                                                                                                                  \
  extern "C" int graphop_vector_spmm_backward_planned_##SUF(const graphop_plan_t* plan_r,                            \
                                                            const graphop_plan_t* plan_t, const CT* edata,           \
                                                            const CT* dy, const CT* x, CT* dedata, CT* dx,           \
                                                            int64_t n_dst, int64_t n_src, int H, int D, void* ws,    \
                                                            size_t wsb, graphop_stream_t stream) {                   \
    return gk::spmm_backward<T>(GK_PL(plan_r), GK_PL(plan_t), GK_PC(plan_r), GK_PC(plan_t), (const T*)edata,         \
                                (const T*)dy, (const T*)x, (T*)dedata, (T*)dx, GK_PE(plan_r), n_dst, n_src, H, D,    \
                                ws, wsb, GK_ST);                                                                     \
  }

#define GRAPHOP_DEFINE_PLANNED_ATTENTION(SUF, CT, T)                                                                 \
  extern "C" int graphop_attention_forward_planned_##SUF(const graphop_plan_t* plan, const CT* q, const CT* k,       \
                                                         const CT* v, double scale, CT* o, void* lse, int64_t n_dst, \
                                                         int64_t n_src, int H, int D, void* ws, size_t wsb,          \
                                                         graphop_stream_t stream) {                                  \
    return gk::attention_forward_planned<T>(plan, (const T*)q, (const T*)k, (const T*)v, scale, (T*)o, lse, n_dst,   \
                                            n_src, H, D, ws, wsb, GK_ST);                                            \
  }                                                                                                                  \
  extern "C" int graphop_attention_backward_planned_##SUF(                                                           \
      const graphop_plan_t* plan_r, const graphop_plan_t* plan_t, const CT* q, const CT* k, const CT* v,             \
      const CT* o, const void* lse, const CT* d_o, double scale, CT* dq, CT* dk, CT* dv, int64_t n_dst,              \
      int64_t n_src, int H, int D, void* ws, size_t wsb, graphop_stream_t stream) {                                  \
    return gk::attention_backward_planned<T>(plan_r, plan_t, (const T*)q, (const T*)k, (const T*)v, (const T*)o,     \
                                             lse, (const T*)d_o, scale, (T*)dq, (T*)dk, (T*)dv, n_dst, n_src, H, D,  \
                                             ws, wsb, GK_ST);                                                        \
  }
