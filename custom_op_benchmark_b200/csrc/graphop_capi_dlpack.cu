// The DLPack boundary (include/graphop_dlpack.h): reads element type, index type and sizes from the tensor
// descriptors, checks them, and calls the typed entry point.  Host code only; no kernel lives here.
#include "../../include/graphop_dlpack.h"

namespace {

using DL = graphop_dltensor_t;
constexpr int kDLCUDA = 2, kDLCUDAManaged = 13;
constexpr int kDLInt = 0, kDLUInt = 1, kDLFloat = 2, kDLBfloat = 4;

// 0 f32, 1 f64, 2 bf16; 0 i32, 1 i64; -1: none of them
int elem_kind(const DL* t) {
  if (t->dtype.lanes != 1) return -1;
  if (t->dtype.code == kDLFloat && t->dtype.bits == 32) return 0;
  if (t->dtype.code == kDLFloat && t->dtype.bits == 64) return 1;
  if (t->dtype.code == kDLBfloat && t->dtype.bits == 16) return 2;
  return -1;
}
int index_kind(const DL* t) {
  if (t->dtype.lanes != 1 || t->dtype.code != kDLInt) return -1;
  return t->dtype.bits == 32 ? 0 : (t->dtype.bits == 64 ? 1 : -1);
}

// What one call has seen so far: every tensor must agree with it.
struct Call {
  int device = -1;
  int elem = -1;
  int index = -1;
  bool bad = false;

  // a tensor on the call's device, compact row-major, 1 to 3 dimensions; returns its data pointer
  void* base(const DL* t) {
    if (!t || t->ndim < 1 || t->ndim > 3 || !t->shape) { bad = true; return nullptr; }
    if (t->device.device_type != kDLCUDA && t->device.device_type != kDLCUDAManaged) { bad = true; return nullptr; }
    if (device < 0) device = t->device.device_id;
    if (t->device.device_id != device) { bad = true; return nullptr; }
    int64_t count = 1;
    for (int i = t->ndim - 1; i >= 0; --i) {
      if (t->shape[i] < 0) { bad = true; return nullptr; }
      if (t->strides && t->shape[i] > 1 && t->strides[i] != count) { bad = true; return nullptr; }
      count *= t->shape[i];
    }
    if (!t->data && count > 0) { bad = true; return nullptr; }
    return (char*)t->data + t->byte_offset;
  }
  // an index vector of `want` entries (want < 0: any length)
  const void* index_vec(const DL* t, int64_t want, int64_t* len = nullptr) {
    void* p = base(t);
    if (bad) return nullptr;
    const int k = index_kind(t);
    if (k < 0 || t->ndim != 1 || (index >= 0 && k != index) || (want >= 0 && t->shape[0] != want)) {
      bad = true;
      return nullptr;
    }
    index = k;
    if (len) *len = t->shape[0];
    return p;
  }
  void* value(const DL* t) {
    void* p = base(t);
    if (bad) return nullptr;
    const int k = elem_kind(t);
    if (k < 0 || (elem >= 0 && k != elem)) { bad = true; return nullptr; }
    elem = k;
    return p;
  }
  // node tensor (n, H, D) or (n, D): fills n and checks or sets H, D
  void* node(const DL* t, int64_t* n, int* H, int* D) {
    void* p = value(t);
    if (bad) return nullptr;
    if (t->ndim < 2) { bad = true; return nullptr; }
    const int64_t h = t->ndim == 3 ? t->shape[1] : 1, d = t->shape[t->ndim - 1];
    if (h < 1 || d < 1 || h > INT32_MAX || d > INT32_MAX || (*H > 0 && h != *H) || (*D > 0 && d != *D)) {
      bad = true;
      return nullptr;
    }
    *H = (int)h;
    *D = (int)d;
    if (*n >= 0 && t->shape[0] != *n) { bad = true; return nullptr; }
    *n = t->shape[0];
    return p;
  }
  // edge tensor (n_edges, H) or (n_edges) for H = 1
  void* edge(const DL* t, int64_t* e, int* H) {
    void* p = value(t);
    if (bad) return nullptr;
    if (t->ndim > 2) { bad = true; return nullptr; }
    const int64_t h = t->ndim == 2 ? t->shape[1] : 1;
    if (h < 1 || h > INT32_MAX || (*H > 0 && h != *H)) { bad = true; return nullptr; }
    *H = (int)h;
    if (*e >= 0 && t->shape[0] != *e) { bad = true; return nullptr; }
    *e = t->shape[0];
    return p;
  }
  // the workspace: any tensor of 1-byte elements
  void* bytes(const DL* t, size_t* n) {
    *n = 0;
    if (!t) return nullptr;
    void* p = base(t);
    if (bad) return nullptr;
    if (t->dtype.bits != 8 || t->dtype.lanes != 1 || (t->dtype.code != kDLInt && t->dtype.code != kDLUInt)) {
      bad = true;
      return nullptr;
    }
    size_t count = 1;
    for (int i = 0; i < t->ndim; ++i) count *= (size_t)t->shape[i];
    *n = count;
    return p;
  }
  // one orientation of the graph: chunk owners, chunk boundaries, optional edge ids, optional other endpoints
  struct Graph {
    const void *row, *indptr, *eid, *indices;
    int64_t n_chunks;
  };
  Graph graph(const DL* row, const DL* indptr, const DL* eid, const DL* indices, bool want_indices, int64_t* n_edges) {
    Graph g{};
    g.row = index_vec(row, -1, &g.n_chunks);
    if (bad) return g;
    g.indptr = index_vec(indptr, g.n_chunks + 1);
    if (eid) g.eid = index_vec(eid, *n_edges, n_edges);
    if (want_indices) g.indices = index_vec(indices, *n_edges, n_edges);
    return g;
  }
  int key() const { return elem * 2 + index; }
};

}  // namespace

// One case per (element, index) pair; ARGS uses the local type names T and I.
#define GK_DL_CASE(OP, SUF, TT, II, ARGS) \
  {                                       \
    using T = TT;                         \
    using I = II;                         \
    return graphop_##OP##_##SUF ARGS;     \
  }
#define GK_DL_DISPATCH(OP, ARGS)                                  \
  switch (c.key()) {                                              \
    case 0: GK_DL_CASE(OP, f32_i32, float, int32_t, ARGS)         \
    case 1: GK_DL_CASE(OP, f32_i64, float, int64_t, ARGS)         \
    case 2: GK_DL_CASE(OP, f64_i32, double, int32_t, ARGS)        \
    case 3: GK_DL_CASE(OP, f64_i64, double, int64_t, ARGS)        \
    case 4: GK_DL_CASE(OP, bf16_i32, uint16_t, int32_t, ARGS)     \
    case 5: GK_DL_CASE(OP, bf16_i64, uint16_t, int64_t, ARGS)     \
    default: return GRAPHOP_ERR_INVALID_ARGUMENT;                 \
  }

extern "C" int graphop_dl_maskedmm_csr_forward(const DL* row, const DL* indptr, const DL* eid, const DL* indices,
                                               const DL* A, const DL* B, DL* y, DL* workspace,
                                               graphop_stream_t stream) {
  Call c;
  int64_t E = -1, n_dst = -1, n_src = -1;
  int H = 0, D = 0;
  size_t ws_bytes;
  void* yp = c.edge(y, &E, &H);
  const auto g = c.graph(row, indptr, eid, indices, true, &E);
  const void* a = c.node(A, &n_dst, &H, &D);
  const void* b = c.node(B, &n_src, &H, &D);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(maskedmm_csr_forward,
                 ((const I*)g.row, (const I*)g.indptr, (const I*)g.eid, (const I*)g.indices, (const T*)a, (const T*)b,
                  (T*)yp, g.n_chunks, E, n_dst, n_src, H, D, ws, ws_bytes, stream))
}

extern "C" int graphop_dl_maskedmm_csr_backward(const DL* row, const DL* indptr_r, const DL* eid_r,
                                                const DL* indices_r, const DL* col, const DL* indptr_c,
                                                const DL* eid_c, const DL* indices_c, const DL* A, const DL* B,
                                                const DL* dy, DL* dA, DL* dB, DL* workspace,
                                                graphop_stream_t stream) {
  Call c;
  int64_t E = -1, n_dst = -1, n_src = -1;
  int H = 0, D = 0;
  size_t ws_bytes;
  const void* g_y = c.edge(dy, &E, &H);
  const auto gr = c.graph(row, indptr_r, eid_r, indices_r, true, &E);
  const auto gc = c.graph(col, indptr_c, eid_c, indices_c, true, &E);
  const void* a = c.node(A, &n_dst, &H, &D);
  const void* b = c.node(B, &n_src, &H, &D);
  void* da = c.node(dA, &n_dst, &H, &D);
  void* db = c.node(dB, &n_src, &H, &D);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(maskedmm_csr_backward,
                 ((const I*)gr.row, (const I*)gr.indptr, (const I*)gr.eid, (const I*)gr.indices, gr.n_chunks,
                  (const I*)gc.row, (const I*)gc.indptr, (const I*)gc.eid, (const I*)gc.indices, gc.n_chunks,
                  (const T*)a, (const T*)b, (const T*)g_y, (T*)da, (T*)db, E, n_dst, n_src, H, D, ws, ws_bytes, stream))
}

extern "C" int graphop_dl_node_mul_edge_forward(const DL* row, const DL* indptr, const DL* eid, const DL* A,
                                                const DL* B, DL* y, DL* workspace, graphop_stream_t stream) {
  Call c;
  int64_t E = -1, n_dst = -1;
  int H = 0, D = 0, one = 1;
  size_t ws_bytes;
  void* yp = c.edge(y, &E, &H);
  const auto g = c.graph(row, indptr, eid, nullptr, false, &E);
  const void* a = c.node(A, &n_dst, &H, &D);
  const void* b = c.node(B, &E, &one, &D);   // (n_edges, D): one row per edge, shared by the heads
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad || B->ndim != 2) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(node_mul_edge_forward, ((const I*)g.row, (const I*)g.indptr, (const I*)g.eid, (const T*)a, (const T*)b,
                                         (T*)yp, g.n_chunks, E, n_dst, H, D, ws, ws_bytes, stream))
}

extern "C" int graphop_dl_node_mul_edge_backward(const DL* row, const DL* indptr, const DL* eid, const DL* A,
                                                 const DL* B, const DL* dy, DL* dA, DL* dB, DL* workspace,
                                                 graphop_stream_t stream) {
  Call c;
  int64_t E = -1, n_dst = -1;
  int H = 0, D = 0, one = 1;
  size_t ws_bytes;
  const void* g_y = c.edge(dy, &E, &H);
  const auto g = c.graph(row, indptr, eid, nullptr, false, &E);
  const void* a = c.node(A, &n_dst, &H, &D);
  const void* b = c.node(B, &E, &one, &D);
  void* da = c.node(dA, &n_dst, &H, &D);
  void* db = c.node(dB, &E, &one, &D);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad || B->ndim != 2 || dB->ndim != 2) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(node_mul_edge_backward,
                 ((const I*)g.row, (const I*)g.indptr, (const I*)g.eid, (const T*)a, (const T*)b, (const T*)g_y, (T*)da,
                  (T*)db, g.n_chunks, E, n_dst, H, D, ws, ws_bytes, stream))
}

extern "C" int graphop_dl_sparse_softmax_forward(const DL* row, const DL* indptr, const DL* eid, const DL* x, DL* y,
                                                 int64_t n_nodes, DL* workspace, graphop_stream_t stream) {
  Call c;
  int64_t E = -1;
  int H = 0;
  size_t ws_bytes;
  const void* xp = c.edge(x, &E, &H);
  void* yp = c.edge(y, &E, &H);
  const auto g = c.graph(row, indptr, eid, nullptr, false, &E);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(sparse_softmax_forward, ((const I*)g.row, (const I*)g.indptr, (const I*)g.eid, (const T*)xp, (T*)yp,
                                          g.n_chunks, E, n_nodes, H, ws, ws_bytes, stream))
}

extern "C" int graphop_dl_sparse_softmax_backward(const DL* row, const DL* indptr, const DL* eid, const DL* y,
                                                  const DL* dy, DL* dx, int64_t n_nodes, DL* workspace,
                                                  graphop_stream_t stream) {
  Call c;
  int64_t E = -1;
  int H = 0;
  size_t ws_bytes;
  const void* yp = c.edge(y, &E, &H);
  const void* g_y = c.edge(dy, &E, &H);
  void* g_x = c.edge(dx, &E, &H);
  const auto g = c.graph(row, indptr, eid, nullptr, false, &E);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(sparse_softmax_backward, ((const I*)g.row, (const I*)g.indptr, (const I*)g.eid, (const T*)yp,
                                           (const T*)g_y, (T*)g_x, g.n_chunks, E, n_nodes, H, ws, ws_bytes, stream))
}

extern "C" int graphop_dl_vector_spmm_forward(const DL* row, const DL* indptr, const DL* eid, const DL* indices,
                                              const DL* edata, const DL* x, DL* y, DL* workspace,
                                              graphop_stream_t stream) {
  Call c;
  int64_t E = -1, n_dst = -1, n_src = -1;
  int H = 0, D = 0;
  size_t ws_bytes;
  const void* w = c.edge(edata, &E, &H);
  const auto g = c.graph(row, indptr, eid, indices, true, &E);
  const void* xp = c.node(x, &n_src, &H, &D);
  void* yp = c.node(y, &n_dst, &H, &D);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(vector_spmm_forward,
                 ((const I*)g.row, (const I*)g.indptr, (const I*)g.eid, (const I*)g.indices, (const T*)w, (const T*)xp,
                  (T*)yp, g.n_chunks, E, n_dst, n_src, H, D, ws, ws_bytes, stream))
}

extern "C" int graphop_dl_vector_spmm_backward(const DL* row, const DL* indptr, const DL* eid, const DL* indices,
                                               const DL* col, const DL* indptr_t, const DL* eid_t,
                                               const DL* indices_t, const DL* edata, const DL* dy, const DL* x,
                                               DL* dedata, DL* dx, DL* workspace, graphop_stream_t stream) {
  Call c;
  int64_t E = -1, n_dst = -1, n_src = -1;
  int H = 0, D = 0;
  size_t ws_bytes;
  const void* w = c.edge(edata, &E, &H);
  void* dw = c.edge(dedata, &E, &H);
  const auto gr = c.graph(row, indptr, eid, indices, true, &E);
  const auto gt = c.graph(col, indptr_t, eid_t, indices_t, true, &E);
  const void* g_y = c.node(dy, &n_dst, &H, &D);
  const void* xp = c.node(x, &n_src, &H, &D);
  void* g_x = c.node(dx, &n_src, &H, &D);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(vector_spmm_backward,
                 ((const I*)gr.row, (const I*)gr.indptr, (const I*)gr.eid, (const I*)gr.indices, gr.n_chunks,
                  (const I*)gt.row, (const I*)gt.indptr, (const I*)gt.eid, (const I*)gt.indices, gt.n_chunks,
                  (const T*)w, (const T*)g_y, (const T*)xp, (T*)dw, (T*)g_x, E, n_dst, n_src, H, D, ws, ws_bytes,
                  stream))
}

namespace {
// lse: (n_dst, H) or (n_dst) for H = 1, float32 beside float32 / bfloat16 values, float64 beside float64
void* lse_tensor(Call& c, const DL* lse, int64_t n_dst, int H) {
  void* p = c.base(lse);
  if (c.bad) return nullptr;
  const bool wide = c.elem == 1;
  if (lse->dtype.code != kDLFloat || lse->dtype.lanes != 1 || lse->dtype.bits != (wide ? 64 : 32) || lse->ndim > 2 ||
      lse->shape[0] != n_dst || (lse->ndim == 2 ? lse->shape[1] : 1) != H) {
    c.bad = true;
    return nullptr;
  }
  return p;
}
}  // namespace

extern "C" int graphop_dl_attention_forward(const DL* row, const DL* indptr, const DL* indices, const DL* q,
                                            const DL* k, const DL* v, double scale, DL* o, DL* lse, DL* workspace,
                                            graphop_stream_t stream) {
  Call c;
  int64_t E = -1, n_dst = -1, n_src = -1;
  int H = 0, D = 0;
  size_t ws_bytes;
  const auto g = c.graph(row, indptr, nullptr, indices, true, &E);
  const void* qp = c.node(q, &n_dst, &H, &D);
  const void* kp = c.node(k, &n_src, &H, &D);
  const void* vp = c.node(v, &n_src, &H, &D);
  void* op = c.node(o, &n_dst, &H, &D);
  void* lp = c.bad ? nullptr : lse_tensor(c, lse, n_dst, H);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(attention_forward,
                 ((const I*)g.row, (const I*)g.indptr, (const I*)g.indices, g.n_chunks, (const T*)qp, (const T*)kp,
                  (const T*)vp, scale, (T*)op, lp, E, n_dst, n_src, H, D, ws, ws_bytes, stream))
}

extern "C" int graphop_dl_attention_backward(const DL* row, const DL* indptr, const DL* indices, const DL* col,
                                             const DL* indptr_t, const DL* eid_t, const DL* indices_t, const DL* q,
                                             const DL* k, const DL* v, const DL* o, const DL* lse, const DL* d_o,
                                             double scale, DL* dq, DL* dk, DL* dv, DL* workspace,
                                             graphop_stream_t stream) {
  Call c;
  int64_t E = -1, n_dst = -1, n_src = -1;
  int H = 0, D = 0;
  size_t ws_bytes;
  const auto gr = c.graph(row, indptr, nullptr, indices, true, &E);
  const auto gt = c.graph(col, indptr_t, eid_t, indices_t, true, &E);
  const void* qp = c.node(q, &n_dst, &H, &D);
  const void* kp = c.node(k, &n_src, &H, &D);
  const void* vp = c.node(v, &n_src, &H, &D);
  const void* op = c.node(o, &n_dst, &H, &D);
  const void* gp = c.node(d_o, &n_dst, &H, &D);
  void* dqp = c.node(dq, &n_dst, &H, &D);
  void* dkp = c.node(dk, &n_src, &H, &D);
  void* dvp = c.node(dv, &n_src, &H, &D);
  const void* lp = c.bad ? nullptr : lse_tensor(c, lse, n_dst, H);
  void* ws = c.bytes(workspace, &ws_bytes);
  if (c.bad) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_DL_DISPATCH(attention_backward,
                 ((const I*)gr.row, (const I*)gr.indptr, (const I*)gr.indices, gr.n_chunks, (const I*)gt.row,
                  (const I*)gt.indptr, (const I*)gt.eid, (const I*)gt.indices, gt.n_chunks, (const T*)qp, (const T*)kp,
                  (const T*)vp, (const T*)op, lp, (const T*)gp, scale, (T*)dqp, (T*)dkp, (T*)dvp, E, n_dst, n_src, H, D,
                  ws, ws_bytes, stream))
}
