// The Python module `graphop`: the eight functions the reference extension exports (graphop/graphop.cpp:216-225),
// with the same names, positional arguments and return values, on top of the C ABI.
//
// This file is the whole binding: it checks the tensors the way the reference does (CUDA, contiguous;
// graphop.cpp:4-6), allocates the outputs and a workspace with torch, describes every tensor as a DLPack tensor
// and calls the graphop_dl_* entry point (include/graphop_dlpack.h) on the current stream of the tensors' device.
// Element and index types are dispatched on the C side: float32, float64 and bfloat16 values, int32 and int64
// indices (the reference takes float32 / float64 with int64 only).  A non-zero status becomes a RuntimeError,
// which is what the reference's TORCH checks raise.
//
// Two more functions, attention_forward and attention_backward, expose the fused chain.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <algorithm>
#include <string>
#include <vector>

#include "../../../include/graphop_dlpack.h"

namespace {

using at::Tensor;

// A DLPack descriptor of a torch tensor, alive as long as this object is.
struct View {
  graphop_dltensor_t t{};
  std::vector<int64_t> shape;
  View() = default;
  View(const Tensor& x, const char* name) { set(x, name); }
  void set(const Tensor& x, const char* name) {
    TORCH_CHECK(x.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(x.is_contiguous(), name, " must be contiguous");
    shape.assign(x.sizes().begin(), x.sizes().end());
    t.data = x.data_ptr();
    t.device.device_type = 2;  // kDLCUDA
    t.device.device_id = x.get_device();
    t.ndim = (int32_t)shape.size();
    t.shape = shape.data();
    t.strides = nullptr;
    t.byte_offset = 0;
    t.dtype.lanes = 1;
    switch (x.scalar_type()) {
      case at::kFloat: t.dtype.code = 2; t.dtype.bits = 32; break;
      case at::kDouble: t.dtype.code = 2; t.dtype.bits = 64; break;
      case at::kBFloat16: t.dtype.code = 4; t.dtype.bits = 16; break;
      case at::kInt: t.dtype.code = 0; t.dtype.bits = 32; break;
      case at::kLong: t.dtype.code = 0; t.dtype.bits = 64; break;
      case at::kByte: t.dtype.code = 1; t.dtype.bits = 8; break;
      default: TORCH_CHECK(false, "\"graphop\" not implemented for '", x.scalar_type(), "' (", name, ")");
    }
  }
  View(const View&) = delete;
  View& operator=(const View&) = delete;
  graphop_dltensor_t* p() { return &t; }
};

int heads_of_node(const Tensor& x) { return x.dim() == 3 ? (int)x.size(1) : 1; }

const Tensor& on_cuda(const Tensor& x) {
  TORCH_CHECK(x.is_cuda(), "graphop: the tensors must be CUDA tensors");
  return x;
}

// One call: device guard, stream, workspace.
struct Call {
  c10::cuda::CUDAGuard guard;
  cudaStream_t stream;
  Tensor ws_tensor;
  explicit Call(const Tensor& on) : guard(on_cuda(on).device()), stream(at::cuda::getCurrentCUDAStream(on.get_device())) {}
  // workspace for `op`; the returned view stays valid while this Call lives
  graphop_dltensor_t* workspace(View& v, int op, int64_t n_edges, int64_t n_nodes, int H, int D, const Tensor& value,
                                const Tensor& index) {
    const size_t bytes = graphop_workspace_bytes(op, n_edges, n_nodes, H, D, (int)value.element_size(),
                                                 (int)index.element_size());
    ws_tensor = at::empty({(int64_t)std::max<size_t>(bytes, 256)}, value.options().dtype(at::kByte));
    v.set(ws_tensor, "workspace");
    return v.p();
  }
  void check(int rc, const char* what) {
    if (rc == GRAPHOP_OK) return;
    std::string msg = std::string("graphop.") + what + ": " + graphop_error_string(rc);
    if (rc == GRAPHOP_ERR_CUDA) msg += " (cudaError " + std::to_string(graphop_last_cuda_error()) + ")";
    TORCH_CHECK(false, msg);
  }
};

// (n_edges, H) like the reference: (n_edges) when the node tensors are 2-D
Tensor edge_like(const Tensor& node, int64_t n_edges) {
  return node.dim() == 3 ? at::empty({n_edges, node.size(1)}, node.options()) : at::empty({n_edges}, node.options());
}

// an upper bound on node id + 1 from the chunk table: its owners are non-decreasing (one small device read)
int64_t node_bound(const Tensor& row) { return row.numel() ? row[-1].item<int64_t>() + 1 : 0; }

// graphop.cpp:16-30
Tensor maskedmm_csr_forward(const Tensor& row, const Tensor& indptr, const Tensor& eid, const Tensor& indices,
                            const Tensor& A, const Tensor& B) {
  Call c(A);
  const int64_t E = eid.numel();
  Tensor y = edge_like(A, E);
  View vr(row, "row"), vp(indptr, "indptr"), ve(eid, "eid"), vi(indices, "indices"), va(A, "A"), vb(B, "B"),
      vy(y, "y"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_MASKEDMM_FWD, E, std::max(A.size(0), B.size(0)), heads_of_node(A),
                         (int)A.size(-1), A, row);
  c.check(graphop_dl_maskedmm_csr_forward(vr.p(), vp.p(), ve.p(), vi.p(), va.p(), vb.p(), vy.p(), ws, c.stream),
          "maskedmm_csr_forward");
  return y;
}

// graphop.cpp:108-131
std::vector<Tensor> maskedmm_csr_backward(const Tensor& row, const Tensor& indptr_r, const Tensor& eid_r,
                                          const Tensor& indices_r, const Tensor& col, const Tensor& indptr_c,
                                          const Tensor& eid_c, const Tensor& indices_c, const Tensor& A,
                                          const Tensor& B, const Tensor& dy) {
  Call c(A);
  Tensor dA = at::empty_like(A), dB = at::empty_like(B);
  View v0(row, "row"), v1(indptr_r, "indptr_r"), v2(eid_r, "eid_r"), v3(indices_r, "indices_r"), v4(col, "col"),
      v5(indptr_c, "indptr_c"), v6(eid_c, "eid_c"), v7(indices_c, "indices_c"), va(A, "A"), vb(B, "B"), vg(dy, "dy"),
      vda(dA, "dA"), vdb(dB, "dB"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_MASKEDMM_BWD, eid_r.numel(), std::max(A.size(0), B.size(0)), heads_of_node(A),
                         (int)A.size(-1), A, row);
  c.check(graphop_dl_maskedmm_csr_backward(v0.p(), v1.p(), v2.p(), v3.p(), v4.p(), v5.p(), v6.p(), v7.p(), va.p(),
                                           vb.p(), vg.p(), vda.p(), vdb.p(), ws, c.stream),
          "maskedmm_csr_backward");
  return {dA, dB};
}

// graphop.cpp:39-51
Tensor node_mul_edge_forward(const Tensor& row, const Tensor& indptr, const Tensor& eid, const Tensor& A,
                             const Tensor& B) {
  Call c(A);
  const int64_t E = eid.numel();
  Tensor y = edge_like(A, E);
  View vr(row, "row"), vp(indptr, "indptr"), ve(eid, "eid"), va(A, "A"), vb(B, "B"), vy(y, "y"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_NODE_MUL_EDGE_FWD, E, A.size(0), heads_of_node(A), (int)A.size(-1), A, row);
  c.check(graphop_dl_node_mul_edge_forward(vr.p(), vp.p(), ve.p(), va.p(), vb.p(), vy.p(), ws, c.stream),
          "node_mul_edge_forward");
  return y;
}

// graphop.cpp:141-154
std::vector<Tensor> node_mul_edge_backward(const Tensor& row, const Tensor& indptr, const Tensor& eid, const Tensor& A,
                                           const Tensor& B, const Tensor& dy) {
  Call c(A);
  Tensor dA = at::empty_like(A), dB = at::empty_like(B);
  View vr(row, "row"), vp(indptr, "indptr"), ve(eid, "eid"), va(A, "A"), vb(B, "B"), vg(dy, "dy"), vda(dA, "dA"),
      vdb(dB, "dB"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_NODE_MUL_EDGE_BWD, eid.numel(), A.size(0), heads_of_node(A), (int)A.size(-1),
                         A, row);
  c.check(graphop_dl_node_mul_edge_backward(vr.p(), vp.p(), ve.p(), va.p(), vb.p(), vg.p(), vda.p(), vdb.p(), ws,
                                            c.stream),
          "node_mul_edge_backward");
  return {dA, dB};
}

// graphop.cpp:59-69
Tensor sparse_softmax_forward(const Tensor& row, const Tensor& indptr, const Tensor& eid, const Tensor& x) {
  Call c(x);
  Tensor y = at::empty_like(x);
  const int64_t n = node_bound(row);
  View vr(row, "row"), vp(indptr, "indptr"), ve(eid, "eid"), vx(x, "x"), vy(y, "y"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_SOFTMAX_FWD, x.size(0), n, x.dim() == 2 ? (int)x.size(1) : 1, 1, x, row);
  c.check(graphop_dl_sparse_softmax_forward(vr.p(), vp.p(), ve.p(), vx.p(), vy.p(), n, ws, c.stream),
          "sparse_softmax_forward");
  return y;
}

// graphop.cpp:163-175
Tensor sparse_softmax_backward(const Tensor& row, const Tensor& indptr, const Tensor& eid, const Tensor& y,
                               const Tensor& dy) {
  Call c(y);
  Tensor dx = at::empty_like(y);
  const int64_t n = node_bound(row);
  View vr(row, "row"), vp(indptr, "indptr"), ve(eid, "eid"), vy(y, "y"), vg(dy, "dy"), vdx(dx, "dx"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_SOFTMAX_BWD, y.size(0), n, y.dim() == 2 ? (int)y.size(1) : 1, 1, y, row);
  c.check(graphop_dl_sparse_softmax_backward(vr.p(), vp.p(), ve.p(), vy.p(), vg.p(), vdx.p(), n, ws, c.stream),
          "sparse_softmax_backward");
  return dx;
}

// graphop.cpp:79-93; like the reference, y takes x's shape (graphop_kernel.cu:527)
Tensor vector_spmm_forward(const Tensor& row, const Tensor& indptr, const Tensor& eid, const Tensor& indices,
                           const Tensor& edata, const Tensor& x) {
  Call c(x);
  Tensor y = at::empty_like(x);
  View vr(row, "row"), vp(indptr, "indptr"), ve(eid, "eid"), vi(indices, "indices"), vd(edata, "edata"), vx(x, "x"),
      vy(y, "y"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_SPMM_FWD, eid.numel(), x.size(0), heads_of_node(x), (int)x.size(-1), x, row);
  c.check(graphop_dl_vector_spmm_forward(vr.p(), vp.p(), ve.p(), vi.p(), vd.p(), vx.p(), vy.p(), ws, c.stream),
          "vector_spmm_forward");
  return y;
}

// graphop.cpp:190-214
std::vector<Tensor> vector_spmm_backward(const Tensor& row, const Tensor& indptr, const Tensor& eid,
                                         const Tensor& indices, const Tensor& col, const Tensor& indptr_t,
                                         const Tensor& eid_t, const Tensor& indices_t, const Tensor& edata,
                                         const Tensor& dy, const Tensor& x) {
  Call c(x);
  Tensor dedata = at::empty_like(edata), dx = at::empty_like(x);
  View v0(row, "row"), v1(indptr, "indptr"), v2(eid, "eid"), v3(indices, "indices"), v4(col, "col"),
      v5(indptr_t, "indptr_t"), v6(eid_t, "eid_t"), v7(indices_t, "indices_t"), vd(edata, "edata"), vg(dy, "dy"),
      vx(x, "x"), vde(dedata, "dedata"), vdx(dx, "dx"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_SPMM_BWD, eid.numel(), std::max(x.size(0), dy.size(0)), heads_of_node(x),
                         (int)x.size(-1), x, row);
  c.check(graphop_dl_vector_spmm_backward(v0.p(), v1.p(), v2.p(), v3.p(), v4.p(), v5.p(), v6.p(), v7.p(), vd.p(),
                                          vg.p(), vx.p(), vde.p(), vdx.p(), ws, c.stream),
          "vector_spmm_backward");
  return {dedata, dx};
}

// the fused chain: returns (o, lse)
std::vector<Tensor> attention_forward(const Tensor& row, const Tensor& indptr, const Tensor& indices, const Tensor& q,
                                      const Tensor& k, const Tensor& v, double scale) {
  Call c(q);
  Tensor o = at::empty_like(q);
  const auto lse_type = q.scalar_type() == at::kDouble ? at::kDouble : at::kFloat;
  Tensor lse = q.dim() == 3 ? at::empty({q.size(0), q.size(1)}, q.options().dtype(lse_type))
                            : at::empty({q.size(0)}, q.options().dtype(lse_type));
  View vr(row, "row"), vp(indptr, "indptr"), vi(indices, "indices"), vq(q, "q"), vk(k, "k"), vv(v, "v"), vo(o, "o"),
      vl(lse, "lse"), vw;
  auto* ws = c.workspace(vw, GRAPHOP_OP_ATTENTION_FWD, indices.numel(), std::max(q.size(0), k.size(0)),
                         heads_of_node(q), (int)q.size(-1), q, row);
  c.check(graphop_dl_attention_forward(vr.p(), vp.p(), vi.p(), vq.p(), vk.p(), vv.p(), scale, vo.p(), vl.p(), ws,
                                       c.stream),
          "attention_forward");
  return {o, lse};
}

// gradients of the fused chain: returns (dq, dk, dv); pass eid_t = None to recompute in the transposed pass
std::vector<Tensor> attention_backward(const Tensor& row, const Tensor& indptr, const Tensor& indices,
                                       const Tensor& col, const Tensor& indptr_t,
                                       const c10::optional<Tensor>& eid_t, const Tensor& indices_t, const Tensor& q,
                                       const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& lse,
                                       const Tensor& d_o, double scale) {
  Call c(q);
  Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
  View v0(row, "row"), v1(indptr, "indptr"), v2(indices, "indices"), v3(col, "col"), v4(indptr_t, "indptr_t"),
      v6(indices_t, "indices_t"), vq(q, "q"), vk(k, "k"), vv(v, "v"), vo(o, "o"), vl(lse, "lse"), vg(d_o, "d_o"),
      vdq(dq, "dq"), vdk(dk, "dk"), vdv(dv, "dv"), v5, vw;
  graphop_dltensor_t* pairs = nullptr;
  if (eid_t.has_value()) {
    v5.set(*eid_t, "eid_t");
    pairs = v5.p();
  }
  auto* ws = c.workspace(vw, pairs ? GRAPHOP_OP_ATTENTION_BWD_PAIRS : GRAPHOP_OP_ATTENTION_BWD, indices.numel(),
                         std::max(q.size(0), k.size(0)), heads_of_node(q), (int)q.size(-1), q, row);
  c.check(graphop_dl_attention_backward(v0.p(), v1.p(), v2.p(), v3.p(), v4.p(), pairs, v6.p(), vq.p(), vk.p(), vv.p(),
                                        vo.p(), vl.p(), vg.p(), scale, vdq.p(), vdk.p(), vdv.p(), ws, c.stream),
          "attention_backward");
  return {dq, dk, dv};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "graphop for NVIDIA B200 (sm_100a): the eight operators of the graphop extension on the graphop_b200 C ABI";
  m.def("maskedmm_csr_forward", &maskedmm_csr_forward,
        "(row, indptr, eid, indices, A, B) -> y with y[eid[k]] = <A[row(k)], B[indices[k]]> per head");
  m.def("maskedmm_csr_backward", &maskedmm_csr_backward,
        "(row, indptr_r, eid_r, indices_r, col, indptr_c, eid_c, indices_c, A, B, dy) -> [dA, dB]");
  m.def("node_mul_edge_forward", &node_mul_edge_forward,
        "(row, indptr, eid, A, B) -> y with y[eid[k]] = <A[row(k)], B[eid[k]]> per head, B one row per edge");
  m.def("node_mul_edge_backward", &node_mul_edge_backward, "(row, indptr, eid, A, B, dy) -> [dA, dB]");
  m.def("sparse_softmax_forward", &sparse_softmax_forward,
        "(row, indptr, eid, x) -> y, the softmax of x over each node's edges, per head");
  m.def("sparse_softmax_backward", &sparse_softmax_backward, "(row, indptr, eid, y, dy) -> dx");
  m.def("vector_spmm_forward", &vector_spmm_forward,
        "(row, indptr, eid, indices, edata, x) -> y with y[n] = sum_k edata[eid[k]] * x[indices[k]] per head");
  m.def("vector_spmm_backward", &vector_spmm_backward,
        "(row, indptr, eid, indices, col, indptr_t, eid_t, indices_t, edata, dy, x) -> [dedata, dx]");
  m.def("attention_forward", &attention_forward,
        "(row, indptr, indices, q, k, v, scale) -> [o, lse]: maskedmm, scale, softmax and SpMM in one pass");
  m.def("attention_backward", &attention_backward,
        "(row, indptr, indices, col, indptr_t, eid_t | None, indices_t, q, k, v, o, lse, d_o, scale) -> [dq, dk, dv]");
  m.def("version", [] { return graphop_version(); }, "graphop_version() of the C library underneath");
}
