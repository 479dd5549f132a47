// Graph preprocessing as kernels: partition_csr, the chunk table every op of the reference takes, and the
// transposed CSR its backward passes take (built with scipy on the host in the reference's scripts,
// wrapper.py:96-112).
//
// The reference builds (row, indptr_) in a Python double loop on the host after copying indptr there
// (part_csr.py:13-27: for every row, for every start in range(indptr[r], indptr[r + 1], chunk_size)).  Here:
//   count:  chunks per row = ceil(degree / chunk_size), an exclusive prefix sum over the rows (CUB DeviceScan, a
//           library scan: this is set-up work, not the hot path) gives every row's first chunk and the total;
//   fill:   one thread per chunk finds its row by binary search in the prefix sums and writes
//           row[c] = r, indptr_[c] = indptr[r] + (c - first[r]) * chunk_size, and the closing sentinel indptr[n].
// Outputs are int64 whatever the input's integer type, as in the reference.  Rows without edges emit no chunk.
//
// transpose_csr: a stable sort of the positions by source id (CUB DeviceRadixSort over just the bits a source id
// needs; stable, so within one source the destinations ascend and the result is the same on every run, which an
// atomic counting sort would not give) yields eid_t; one pass over the sorted keys writes indptr_t at every key
// change (no histogram, no atomics) and looks every position's destination row up in indptr by binary search.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "gk_host.cuh"

namespace gk {
namespace {

template <typename I>
__global__ void chunk_counts_kernel(const I* __restrict__ indptr, long long n, long long cs, long long* __restrict__ out) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r <= n; r += stride) {
    long long c = 0;
    if (r < n) {
      const long long deg = (long long)indptr[r + 1] - (long long)indptr[r];
      c = deg > 0 ? (deg + cs - 1) / cs : 0;   // range(a, b, cs) is empty when b <= a
    }
    out[r] = c;   // out[n] = 0: after the exclusive scan it holds the total
  }
}

template <typename I>
__global__ void chunk_fill_kernel(const I* __restrict__ indptr, const long long* __restrict__ first, long long n,
                                  long long cs, long long C, long long* __restrict__ row,
                                  long long* __restrict__ out_ptr) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c <= C; c += stride) {
    if (c == C) {
      out_ptr[C] = (long long)indptr[n];
      continue;
    }
    // the last row whose first chunk is <= c: empty rows share their successor's value and are skipped by it
    long long lo = 0, hi = n;   // invariant: first[lo] <= c < first[hi]  (first[n] = C > c)
    while (hi - lo > 1) {
      const long long mid = (lo + hi) >> 1;
      if (first[mid] <= c) lo = mid; else hi = mid;
    }
    row[c] = lo;
    out_ptr[c] = (long long)indptr[lo] + (c - first[lo]) * cs;
  }
}

size_t scan_temp_bytes(long long items) {
  size_t bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, bytes, (long long*)nullptr, (long long*)nullptr, (int)(items > 0 ? items : 1));
  return bytes;
}

template <typename I>
int partition_count(const I* indptr, long long n, long long cs, void* ws, size_t wsb, long long* n_chunks,
                    cudaStream_t st) {
  if (!n_chunks) return GRAPHOP_ERR_INVALID_ARGUMENT;
  *n_chunks = 0;
  if (n < 0 || cs <= 0 || n >= (1LL << 31) - 1) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (n == 0) return GRAPHOP_OK;
  if (!indptr) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  long long* first = (long long*)ar.take((size_t)(n + 1) * 8);
  size_t temp_bytes = scan_temp_bytes(n + 1);
  void* temp = ar.take(temp_bytes);
  if (ar.overflow) return GRAPHOP_ERR_WORKSPACE;
  const unsigned grid = (unsigned)((n + 256) / 256 < 8192 ? (n + 256) / 256 : 8192);
  chunk_counts_kernel<I><<<grid, 256, 0, st>>>(indptr, n, cs, first);
  GK_LAUNCHED("partition_counts");
  GK_CUDA(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, first, first, (int)(n + 1), st));
  GK_CUDA(cudaMemcpyAsync(n_chunks, first + n, 8, cudaMemcpyDeviceToHost, st));
  GK_CUDA(cudaStreamSynchronize(st));
  return GRAPHOP_OK;
}

template <typename I>
int partition_fill(const I* indptr, long long n, long long cs, const void* ws, long long C, long long* row,
                   long long* out_ptr, cudaStream_t st) {
  if (n < 0 || cs <= 0 || C < 0 || !out_ptr || (C > 0 && !row)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (n == 0) {   // the reference's sentinel is indptr[-1] of a one-element indptr
    if (!indptr) return GRAPHOP_ERR_INVALID_ARGUMENT;
    chunk_fill_kernel<I><<<1, 32, 0, st>>>(indptr, nullptr, 0, cs, 0, row, out_ptr);
    GK_LAUNCHED("partition_fill");
    return GRAPHOP_OK;
  }
  if (!indptr) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  const long long* first = (const long long*)ws;   // the first item partition_count carved
  const unsigned grid = (unsigned)((C + 256) / 256 < 16384 ? (C + 256) / 256 : 16384);
  chunk_fill_kernel<I><<<grid, 256, 0, st>>>(indptr, first, n, cs, C, row, out_ptr);
  GK_LAUNCHED("partition_fill");
  return GRAPHOP_OK;
}

template <typename I>
__global__ void iota_kernel(I* __restrict__ out, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = (I)i;
}

// keys: the source ids in transposed order; eid_t: the row-CSR position of every transposed position.
template <typename I>
__global__ void transposed_fill_kernel(const I* __restrict__ keys, const I* __restrict__ eid_t,
                                       const I* __restrict__ indptr, long long n_dst, long long n_src, long long E,
                                       I* __restrict__ indptr_t, I* __restrict__ indices_t) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j <= E; j += stride) {
    // indptr_t[k] = j for every source k in (keys[j-1], keys[j]]: the first position whose key is >= k.  Keys
    // outside [0, n_src) break the graph contract; the clamps keep the stores inside the array all the same.
    long long prev = j > 0 ? (long long)keys[j - 1] : -1;
    long long cur = j < E ? (long long)keys[j] : n_src;
    prev = prev < -1 ? -1 : prev;
    cur = cur > n_src ? n_src : cur;
    for (long long k = prev + 1; k <= cur; ++k) indptr_t[k] = (I)j;
    if (j == E) continue;
    // the row that owns position e: the last r with indptr[r] <= e (rows without edges are skipped by it)
    const long long e = (long long)eid_t[j];
    long long lo = 0, hi = n_dst;
    while (hi - lo > 1) {
      const long long mid = (lo + hi) >> 1;
      if ((long long)indptr[mid] <= e) lo = mid; else hi = mid;
    }
    indices_t[j] = (I)lo;
  }
}

template <typename I>
size_t sort_temp_bytes(long long items) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const I*)nullptr, (I*)nullptr, (const I*)nullptr, (I*)nullptr,
                                  (int)(items > 0 ? items : 1), 0, (int)sizeof(I) * 8);
  return bytes;
}

template <typename I>
int transpose(const I* indptr, const I* indices, long long n_dst, long long n_src, long long E, I* indptr_t,
              I* indices_t, I* eid_t, void* ws, size_t wsb, cudaStream_t st) {
  if (n_dst < 0 || n_src < 0 || E < 0 || E >= (1LL << 31) - 1 || !indptr_t) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (sizeof(I) == 4 && (n_src >= (1LL << 31) || n_dst >= (1LL << 31))) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (E > 0 && (!indptr || !indices || !indices_t || !eid_t || n_dst == 0 || n_src == 0))
    return GRAPHOP_ERR_INVALID_ARGUMENT;
  I* keys = nullptr;
  if (E > 0) {
    GK_TRY(check_ws(ws));
    Arena ar(ws, wsb);
    keys = (I*)ar.take((size_t)E * sizeof(I));
    size_t temp_bytes = sort_temp_bytes<I>(E);
    void* temp = ar.take(temp_bytes);
    if (ar.overflow) return GRAPHOP_ERR_WORKSPACE;
    const unsigned grid = (unsigned)((E + 255) / 256 < 16384 ? (E + 255) / 256 : 16384);
    iota_kernel<I><<<grid, 256, 0, st>>>(indices_t, E);   // the output buffer doubles as the sort's value input
    GK_LAUNCHED("transpose_iota");
    int bits = 1;
    while (bits < (int)sizeof(I) * 8 && ((n_src - 1) >> bits) != 0) ++bits;
    GK_CUDA(cub::DeviceRadixSort::SortPairs(temp, temp_bytes, indices, keys, (const I*)indices_t, eid_t, (int)E, 0, bits,
                                            st));
  }
  const unsigned grid = (unsigned)((E + 256) / 256 < 16384 ? (E + 256) / 256 : 16384);
  transposed_fill_kernel<I><<<grid, 256, 0, st>>>(keys, eid_t, indptr, n_dst, n_src, E, indptr_t, indices_t);
  GK_LAUNCHED("transpose_fill");
  return GRAPHOP_OK;
}

}  // namespace
}  // namespace gk

extern "C" size_t graphop_partition_csr_workspace_bytes(int64_t n_rows) {
  if (n_rows < 0) return 0;
  return gk::align_up((size_t)(n_rows + 1) * 8) + gk::align_up(gk::scan_temp_bytes(n_rows + 1)) + gk::kAlign;
}
extern "C" int graphop_partition_csr_count_i32(const int32_t* indptr, int64_t n_rows, int64_t chunk_size, void* ws,
                                               size_t wsb, int64_t* n_chunks, graphop_stream_t stream) {
  long long c = 0;
  const int rc = gk::partition_count<int32_t>(indptr, n_rows, chunk_size, ws, wsb, &c, (cudaStream_t)stream);
  if (n_chunks) *n_chunks = c;
  return n_chunks ? rc : GRAPHOP_ERR_INVALID_ARGUMENT;
}
extern "C" int graphop_partition_csr_count_i64(const int64_t* indptr, int64_t n_rows, int64_t chunk_size, void* ws,
                                               size_t wsb, int64_t* n_chunks, graphop_stream_t stream) {
  long long c = 0;
  const int rc = gk::partition_count<int64_t>(indptr, n_rows, chunk_size, ws, wsb, &c, (cudaStream_t)stream);
  if (n_chunks) *n_chunks = c;
  return n_chunks ? rc : GRAPHOP_ERR_INVALID_ARGUMENT;
}
extern "C" int graphop_partition_csr_fill_i32(const int32_t* indptr, int64_t n_rows, int64_t chunk_size,
                                              const void* ws, int64_t n_chunks, int64_t* row, int64_t* indptr_out,
                                              graphop_stream_t stream) {
  return gk::partition_fill<int32_t>(indptr, n_rows, chunk_size, ws, n_chunks, (long long*)row, (long long*)indptr_out,
                                     (cudaStream_t)stream);
}
extern "C" int graphop_partition_csr_fill_i64(const int64_t* indptr, int64_t n_rows, int64_t chunk_size,
                                              const void* ws, int64_t n_chunks, int64_t* row, int64_t* indptr_out,
                                              graphop_stream_t stream) {
  return gk::partition_fill<int64_t>(indptr, n_rows, chunk_size, ws, n_chunks, (long long*)row, (long long*)indptr_out,
                                     (cudaStream_t)stream);
}

extern "C" size_t graphop_transpose_csr_workspace_bytes(int64_t n_edges, int index_bytes) {
  if (n_edges <= 0) return gk::kAlign;
  const size_t temp = index_bytes == 8 ? gk::sort_temp_bytes<int64_t>(n_edges) : gk::sort_temp_bytes<int32_t>(n_edges);
  return gk::align_up((size_t)n_edges * (size_t)(index_bytes == 8 ? 8 : 4)) + gk::align_up(temp) + gk::kAlign;
}
extern "C" int graphop_transpose_csr_i32(const int32_t* indptr, const int32_t* indices, int64_t n_dst, int64_t n_src,
                                         int64_t n_edges, int32_t* indptr_t, int32_t* indices_t, int32_t* eid_t,
                                         void* ws, size_t wsb, graphop_stream_t stream) {
  return gk::transpose<int32_t>(indptr, indices, n_dst, n_src, n_edges, indptr_t, indices_t, eid_t, ws, wsb,
                                (cudaStream_t)stream);
}
extern "C" int graphop_transpose_csr_i64(const int64_t* indptr, const int64_t* indices, int64_t n_dst, int64_t n_src,
                                         int64_t n_edges, int64_t* indptr_t, int64_t* indices_t, int64_t* eid_t,
                                         void* ws, size_t wsb, graphop_stream_t stream) {
  return gk::transpose<int64_t>(indptr, indices, n_dst, n_src, n_edges, indptr_t, indices_t, eid_t, ws, wsb,
                                (cudaStream_t)stream);
}
