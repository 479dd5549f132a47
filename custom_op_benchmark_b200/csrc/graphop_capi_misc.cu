// C ABI entry points that do not depend on the element type: version, error text, the
// workspace size query and the graph-contract checker.
#include "gk_host.cuh"
#include "gk_plan.cuh"

namespace gk {
namespace {

// Scratch of one row-producing pass: per level 2 slots per tile, each `stride_bytes`, plus the
// next level's row stream.
size_t levels_bytes(long long len0, int tile0, size_t stride_bytes) {
  const Levels lv = make_levels(len0, tile0);
  size_t total = 0;
  for (int k = 0; k + 1 < lv.n; ++k) {
    total += align_up((size_t)(2 * lv.ntiles[k]) * stride_bytes);
    total += align_up((size_t)(2 * lv.ntiles[k]) * 4);
  }
  return total;
}

size_t graph_bytes(long long E, int index_bytes) {
  size_t b = align_up(sizeof(PlanHeader)) + align_up((size_t)E * 4);
  if (index_bytes == 8) b += 2 * align_up((size_t)E * 4);
  return b;
}

template <typename I>
__global__ void check_graph_kernel(const I* __restrict__ row, const I* __restrict__ indptr, const I* __restrict__ eid,
                                   const I* __restrict__ indices, long long C, long long E, long long n_nodes,
                                   long long n_other, int* __restrict__ flags) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int bad = 0;
  for (long long c = i0; c < C; c += stride) {
    const long long s = (long long)indptr[c], e = (long long)indptr[c + 1];
    if (e < s) bad |= 1;
    if (s < 0 || e > E) bad |= 16;
    const long long r = (long long)row[c];
    if (r < 0 || r >= n_nodes) bad |= 2;
    if (c > 0 && (long long)row[c - 1] > r) bad |= 2;
  }
  if (C > 0) {
    const long long lo = (long long)indptr[0], hi = (long long)indptr[C];
    for (long long j = i0; j < E; j += stride) {
      if (j < lo || j >= hi) continue;
      if (indices) { const long long v = (long long)indices[j]; if (v < 0 || v >= n_other) bad |= 4; }
      if (eid) { const long long v = (long long)eid[j]; if (v < 0 || v >= E) bad |= 8; }
    }
  }
  if (bad) atomicOr(flags, bad);
}

template <typename I>
int check_graph(const I* row, const I* indptr, const I* eid, const I* indices, long long C, long long E,
                long long n_nodes, long long n_other, int* violations, cudaStream_t st) {
  if (violations) *violations = 0;
  if (C < 0 || E < 0 || E >= (1LL << 31) || !indptr || (C > 0 && !row)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  int* flags = nullptr;
  GK_CUDA(cudaMallocAsync((void**)&flags, sizeof(int), st));
  GK_CUDA(cudaMemsetAsync(flags, 0, sizeof(int), st));
  const long long work = C > E ? C : E;
  const unsigned grid = (unsigned)((work + 255) / 256 < 4096 ? (work + 255) / 256 : 4096);
  check_graph_kernel<I><<<grid ? grid : 1, 256, 0, st>>>(row, indptr, eid, indices, C, E, n_nodes, n_other, flags);
  GK_LAUNCH_CHECK();
  int host = 0;
  GK_CUDA(cudaMemcpyAsync(&host, flags, sizeof(int), cudaMemcpyDeviceToHost, st));
  GK_CUDA(cudaStreamSynchronize(st));
  GK_CUDA(cudaFreeAsync(flags, st));
  if (violations) *violations = host;
  return host ? GRAPHOP_ERR_INVALID_ARGUMENT : GRAPHOP_OK;
}

}  // namespace
}  // namespace gk

extern "C" int graphop_version(void) { return 100; }

extern "C" const char* graphop_error_string(int code) {
  switch (code) {
    case GRAPHOP_OK: return "ok";
    case GRAPHOP_ERR_INVALID_ARGUMENT: return "invalid argument";
    case GRAPHOP_ERR_WORKSPACE: return "workspace too small or misaligned";
    case GRAPHOP_ERR_UNSUPPORTED: return "shape not supported by this entry point";
    case GRAPHOP_ERR_CUDA: return "CUDA call failed";
    default: return "unknown error code";
  }
}

extern "C" int graphop_last_cuda_error(void) { return gk::g_last_cuda_error; }

namespace gk {
// out[r] = table[idx[r]]: one warp per group of 4 rows, lanes copy 16-byte pieces; the 4 rows' loads are all
// issued before the first store.
__global__ void __launch_bounds__(256) gather_rows_kernel(const int32_t* __restrict__ idx, long long n_rows,
                                                         const uint4* __restrict__ table, int row_vec,
                                                         uint4* __restrict__ out) {
  constexpr int kRows = 4;
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * 8;
  for (long long g = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); g * kRows < n_rows; g += warps) {
    const long long r0 = g * kRows;
    long long src[kRows];
#pragma unroll
    for (int u = 0; u < kRows; ++u) src[u] = r0 + u < n_rows ? (long long)__ldg(idx + r0 + u) : -1;
    for (int j = lane; j < row_vec; j += 32) {
      uint4 v[kRows];
#pragma unroll
      for (int u = 0; u < kRows; ++u)
        if (src[u] >= 0) v[u] = __ldg(table + src[u] * row_vec + j);
#pragma unroll
      for (int u = 0; u < kRows; ++u)
        if (src[u] >= 0) out[(r0 + u) * row_vec + j] = v[u];
    }
  }
}
// out[r] = table_p[idx[r]] for the rows r of segment p (seg[p] <= r < seg[p + 1]): the tables are the blocks of a
// row-sharded tensor on this and on other GPUs, mapped into this process (peer pointers), so the loads of a remote
// segment cross NVLink - each needed row exactly once - and the stores are local.  Plain loads: no multicast, no
// waits; the caller orders the kernel after the owners' writes.  Same shape as gather_rows_kernel.
struct PullTables {
  const uint4* table[GRAPHOP_MAX_PEERS];
  long long seg[GRAPHOP_MAX_PEERS + 1];
  int n;
};
__global__ void __launch_bounds__(256) pull_rows_kernel(const __grid_constant__ PullTables tabs,
                                                       const int32_t* __restrict__ idx, long long n_rows,
                                                       int row_vec, uint4* __restrict__ out) {
  constexpr int kRows = 4;
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * 8;
  for (long long g = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); g * kRows < n_rows; g += warps) {
    const long long r0 = g * kRows;
    const uint4* src[kRows];
#pragma unroll
    for (int u = 0; u < kRows; ++u) {
      src[u] = nullptr;
      const long long r = r0 + u;
      if (r < n_rows) {
        int p = 0;
        while (p + 1 < tabs.n && r >= tabs.seg[p + 1]) ++p;
        src[u] = tabs.table[p] + (long long)__ldg(idx + r) * row_vec;
      }
    }
    for (int j = lane; j < row_vec; j += 32) {
      uint4 v[kRows];
#pragma unroll
      for (int u = 0; u < kRows; ++u)
        if (src[u]) v[u] = src[u][j];
#pragma unroll
      for (int u = 0; u < kRows; ++u)
        if (src[u]) out[(r0 + u) * row_vec + j] = v[u];
    }
  }
}
}  // namespace gk

extern "C" int graphop_pull_rows_i32(const void* const* tables, const int64_t* seg, int n_tables, const int32_t* idx,
                                     int64_t row_bytes, void* out, graphop_stream_t stream) {
  using namespace gk;
  if (n_tables < 1 || n_tables > GRAPHOP_MAX_PEERS || !tables || !seg || row_bytes <= 0) return GRAPHOP_ERR_INVALID_ARGUMENT;
  const long long n_rows = seg[n_tables];
  if (seg[0] != 0 || n_rows < 0) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (n_rows == 0) return GRAPHOP_OK;
  if (!idx || !out) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (row_bytes % 16 || row_bytes / 16 > 0x7fffffff || ((uintptr_t)out & 15)) return GRAPHOP_ERR_UNSUPPORTED;
  PullTables tabs{};
  tabs.n = n_tables;
  for (int p = 0; p < n_tables; ++p) {
    if (seg[p + 1] < seg[p]) return GRAPHOP_ERR_INVALID_ARGUMENT;
    if (seg[p + 1] > seg[p] && (!tables[p] || ((uintptr_t)tables[p] & 15))) return GRAPHOP_ERR_INVALID_ARGUMENT;
    tabs.table[p] = (const uint4*)tables[p];
    tabs.seg[p] = seg[p];
  }
  tabs.seg[n_tables] = n_rows;
  const long long groups = (n_rows + 3) / 4;
  const long long blocks = (groups + 7) / 8;
  const unsigned grid = (unsigned)(blocks < 148 * 64 ? blocks : 148 * 64);
  cudaStream_t st = (cudaStream_t)stream;
  pull_rows_kernel<<<grid, 256, 0, st>>>(tabs, idx, n_rows, (int)(row_bytes / 16), (uint4*)out);
  GK_LAUNCHED("pull_rows");
  return GRAPHOP_OK;
}

extern "C" int graphop_gather_rows_i32(const int32_t* idx, int64_t n_rows, const void* table, int64_t row_bytes,
                                       void* out, graphop_stream_t stream) {
  using namespace gk;
  if (n_rows < 0 || row_bytes <= 0) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (n_rows == 0) return GRAPHOP_OK;
  if (!idx || !table || !out) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (row_bytes % 16 || row_bytes / 16 > 0x7fffffff || (((uintptr_t)table | (uintptr_t)out) & 15))
    return GRAPHOP_ERR_UNSUPPORTED;
  const long long groups = (n_rows + 3) / 4;
  const long long blocks = (groups + 7) / 8;
  const unsigned grid = (unsigned)(blocks < 148 * 64 ? blocks : 148 * 64);
  cudaStream_t st = (cudaStream_t)stream;
  gather_rows_kernel<<<grid, 256, 0, st>>>(idx, n_rows, (const uint4*)table, (int)(row_bytes / 16), (uint4*)out);
  GK_LAUNCHED("gather_rows");
  return GRAPHOP_OK;
}

extern "C" size_t graphop_workspace_bytes(int op, int64_t n_edges, int64_t n_nodes, int H, int D, int elem_bytes,
                                          int index_bytes) {
  using namespace gk;
  if (n_edges < 0 || n_nodes < 0 || H < 1 || D < 1) return 0;
  const long long E = n_edges;
  const size_t acc = elem_bytes == 8 ? 8 : 4;
  const size_t HD = (size_t)H * D;
  const int tile0 = pick_tile(E);
  const size_t graph = graph_bytes(E, index_bytes);
  size_t need = graph;
  switch (op) {
    case GRAPHOP_OP_MASKEDMM_FWD:
    case GRAPHOP_OP_NODE_MUL_EDGE_FWD:
      break;
    case GRAPHOP_OP_MASKEDMM_BWD:
    case GRAPHOP_OP_NODE_MUL_EDGE_BWD:
    case GRAPHOP_OP_SPMM_FWD:
    case GRAPHOP_OP_SPMM_BWD:
      need += levels_bytes(E, tile0, HD * acc);
      break;
    case GRAPHOP_OP_SOFTMAX_FWD:
    case GRAPHOP_OP_SOFTMAX_BWD: {
      // level 0 tiles are 64 or 128 positions; size for 64, and for the widest specialised head count
      const int hh = H <= 8 ? H : 1;
      const size_t w = (op == GRAPHOP_OP_SOFTMAX_FWD ? 2 : 1) * (size_t)hh * acc;
      const long long nt0 = (E + 63) / 64;
      need += align_up((size_t)(2 * nt0) * w) + align_up((size_t)(2 * nt0) * 4);
      need += align_up((size_t)n_nodes * w);
      need += levels_bytes(2 * nt0, kCarryTile, w);
      break;
    }
    case GRAPHOP_OP_ATTENTION_FWD:
      need += levels_bytes(E, tile0, 3 * HD * acc);
      break;
    case GRAPHOP_OP_ATTENTION_BWD:
    case GRAPHOP_OP_ATTENTION_BWD_PAIRS:
      need += align_up((size_t)n_nodes * stat_heads(H, (int)acc) * 2 * acc) + levels_bytes(E, tile0, 2 * HD * acc);
      if (op == GRAPHOP_OP_ATTENTION_BWD_PAIRS) need += align_up((size_t)E * stat_heads(H, (int)acc) * 2 * acc);
      break;
    default:
      return 0;
  }
  return need + kAlign;
}

extern "C" int graphop_check_graph_i32(const int32_t* row, const int32_t* indptr, const int32_t* eid,
                                       const int32_t* indices, int64_t n_chunks, int64_t n_edges, int64_t n_nodes,
                                       int64_t n_other, int* violations, graphop_stream_t stream) {
  return gk::check_graph<int32_t>(row, indptr, eid, indices, n_chunks, n_edges, n_nodes, n_other, violations,
                                  (cudaStream_t)stream);
}
extern "C" int graphop_check_graph_i64(const int64_t* row, const int64_t* indptr, const int64_t* eid,
                                       const int64_t* indices, int64_t n_chunks, int64_t n_edges, int64_t n_nodes,
                                       int64_t n_other, int* violations, graphop_stream_t stream) {
  return gk::check_graph<int64_t>(row, indptr, eid, indices, n_chunks, n_edges, n_nodes, n_other, violations,
                                  (cudaStream_t)stream);
}

extern "C" size_t graphop_plan_bytes(int64_t n_chunks, int64_t n_edges, int64_t n_nodes, int index_bytes) {
  if (n_chunks < 0 || n_edges < 0 || n_nodes < 0) return 0;
  return gk::plan_bytes(n_chunks, n_edges, n_nodes, index_bytes);
}
extern "C" int graphop_plan_build_i32(const int32_t* row, const int32_t* indptr, const int32_t* eid,
                                      const int32_t* indices, int64_t n_chunks, int64_t n_edges, int64_t n_nodes,
                                      void* memory, size_t memory_bytes, graphop_plan_t* plan,
                                      graphop_stream_t stream) {
  return gk::plan_build<int32_t>(row, indptr, eid, indices, n_chunks, n_edges, n_nodes, memory, memory_bytes, plan,
                                 (cudaStream_t)stream);
}
extern "C" int graphop_plan_build_i64(const int64_t* row, const int64_t* indptr, const int64_t* eid,
                                      const int64_t* indices, int64_t n_chunks, int64_t n_edges, int64_t n_nodes,
                                      void* memory, size_t memory_bytes, graphop_plan_t* plan,
                                      graphop_stream_t stream) {
  return gk::plan_build<int64_t>(row, indptr, eid, indices, n_chunks, n_edges, n_nodes, memory, memory_bytes, plan,
                                 (cudaStream_t)stream);
}
