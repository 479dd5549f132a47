// Graph plans: what the ops need from the graph alone, built once per graph in caller-provided memory
// (include/graphop_b200.h, "Graph plans").  The reference prepares its graphs on the host in Python loops
// (part_csr.py:18-21, wrapper.py:93-112); here the expansion of the chunk table, the 32-bit index copies, the
// per-node ranges and the shape analysis are kernels.
#pragma once
#include <climits>

#include "gk_host.cuh"

namespace gk {

struct BandVerdict {
  int not_contiguous;  // some node's neighbours are not one run of consecutive ids
  int max_span;        // most different neighbours any 128 consecutive nodes reach
  int row_crosses;     // some node's positions cross a row-aligned tile boundary
};

constexpr int kBandTileRows = 128;

template <typename V>
__global__ void fill_words_kernel(V* __restrict__ out, V value, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = value;
}

// first position and number of positions of every node, from the chunk table (integer atomics: the result does
// not depend on their order)
template <typename I>
__global__ void node_ranges_kernel(const I* __restrict__ row, const I* __restrict__ indptr, long long C,
                                   long long n_nodes, int32_t* __restrict__ first, int32_t* __restrict__ deg) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < C; c += stride) {
    const long long r = (long long)row[c];
    const long long s = (long long)indptr[c], e = (long long)indptr[c + 1];
    if (r < 0 || r >= n_nodes || e <= s) continue;
    atomicMin(first + r, (int)s);
    atomicAdd(deg + r, (int)(e - s));
  }
}

// every covered position must hold (first neighbour of its node) + (its offset inside the node)
__global__ void band_positions_kernel(const int32_t* __restrict__ erow, const int32_t* __restrict__ other, long long E,
                                      const int32_t* __restrict__ first, BandVerdict* __restrict__ verdict) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  int bad = 0;
  for (long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x; j < E; j += stride) {
    const int r = erow[j];
    if (r < 0) continue;
    const int f = first[r];
    if (other[j] != other[f] + (int)(j - f)) bad = 1;
  }
  if (bad) atomicOr(&verdict->not_contiguous, 1);
}

// first neighbour per node, and the widest range of neighbours any tile of 128 consecutive nodes reaches
__global__ void __launch_bounds__(kBandTileRows)
band_tiles_kernel(const int32_t* __restrict__ other, const int32_t* __restrict__ first,
                  const int32_t* __restrict__ deg, long long n_nodes, int32_t* __restrict__ node_lo,
                  BandVerdict* __restrict__ verdict) {
  __shared__ int s_lo[kBandTileRows / 32], s_hi[kBandTileRows / 32];
  const long long r = (long long)blockIdx.x * kBandTileRows + threadIdx.x;
  int lo = INT_MAX, hi = INT_MIN;
  if (r < n_nodes) {
    const int d = deg[r];
    const int l = d > 0 ? other[first[r]] : 0;
    node_lo[r] = l;
    if (d > 0) { lo = l; hi = l + d - 1; }
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(kFull, lo, o));
    hi = max(hi, __shfl_xor_sync(kFull, hi, o));
  }
  if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo; s_hi[threadIdx.x >> 5] = hi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kBandTileRows / 32; ++w) { lo = min(lo, s_lo[w]); hi = max(hi, s_hi[w]); }
    if (hi >= lo) atomicMax(&verdict->max_span, hi - lo + 1);
  }
}

// Boundaries of the level-0 work tiles, moved up to row starts: tile t nominally begins at position t * tile; if a
// node starts at one of the positions t * tile .. (t + 1) * tile - 1, the tile begins at the first such position
// instead, so that no short node is cut in two.  A node longer than a tile still crosses: reported in the verdict.
__global__ void tile_bounds_kernel(const int32_t* __restrict__ erow, long long E, int tile, long long n_tiles,
                                   int32_t* __restrict__ tile_start, BandVerdict* __restrict__ verdict) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  int crosses = 0;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t <= n_tiles; t += stride) {
    long long b = t * tile;
    if (t == 0) b = 0;
    else if (t == n_tiles) b = E;
    else {
      const long long limit = b + tile < E ? b + tile : E;
      int prev = erow[b - 1];
      long long q = b;
      for (; q < limit; ++q) {
        const int r = erow[q];
        if (r != prev) break;
        prev = r;
      }
      if (q < limit) b = q;                       // a row start inside the tile
      else if (erow[b] >= 0) crosses = 1;         // one node fills the whole tile and began before it
    }
    tile_start[t] = (int32_t)b;
  }
  if (crosses) atomicOr(&verdict->row_crosses, 1);
}

inline size_t plan_bytes(long long C, long long E, long long n_nodes, int index_bytes) {
  (void)C;
  size_t b = align_up(sizeof(PlanHeader)) + align_up((size_t)E * 4) + align_up(sizeof(BandVerdict));
  b += align_up((size_t)((E + 31) / 32 + 2) * 4);   // tile boundaries, sized for the smallest tile
  if (index_bytes == 8) b += 2 * align_up((size_t)E * 4);
  b += 3 * align_up((size_t)(n_nodes > 0 ? n_nodes : 1) * 4);
  return b + kAlign;
}

template <typename I>
inline int plan_build(const I* row, const I* indptr, const I* eid, const I* indices, long long C, long long E,
                      long long n_nodes, void* memory, size_t bytes, graphop_plan_t* plan, cudaStream_t st) {
  if (!plan) return GRAPHOP_ERR_INVALID_ARGUMENT;
  *plan = graphop_plan_t{};
  if (C < 0 || E < 0 || n_nodes < 0 || E >= (1LL << 31) || n_nodes >= (1LL << 31)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (!indptr || (C > 0 && !row)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(memory));
  Arena ar(memory, bytes);
  auto* verdict = (BandVerdict*)ar.take(sizeof(BandVerdict));
  GraphView g{};
  int32_t* first = (int32_t*)ar.take((size_t)(n_nodes > 0 ? n_nodes : 1) * 4);
  int32_t* deg = (int32_t*)ar.take((size_t)(n_nodes > 0 ? n_nodes : 1) * 4);
  int32_t* node_lo = (int32_t*)ar.take((size_t)(n_nodes > 0 ? n_nodes : 1) * 4);
  if (ar.overflow) return GRAPHOP_ERR_WORKSPACE;
  plan->n_chunks = C;
  plan->n_edges = E;
  plan->n_nodes = n_nodes;
  if (E == 0) {  // nothing to expand: the ops return before they look at a plan's arrays
    GK_CUDA(cudaMemsetAsync(deg, 0, (size_t)(n_nodes > 0 ? n_nodes : 1) * 4, st));
    plan->node_deg = deg;
    plan->node_lo = node_lo;
    return GRAPHOP_OK;
  }
  GK_TRY(prepare_graph<I>(ar, row, indptr, eid, indices, C, E, st, &g));
  plan->header = g.hdr;
  plan->erow = g.erow;
  plan->other = g.other;
  plan->eid = g.eid;
  plan->node_lo = node_lo;
  plan->node_deg = deg;
  GK_CUDA(cudaMemsetAsync(verdict, 0, sizeof(BandVerdict), st));
  GK_CUDA(cudaMemsetAsync(deg, 0, (size_t)n_nodes * 4, st));
  if (n_nodes > 0) {
    const unsigned gn = (unsigned)((n_nodes + 255) / 256 < 4096 ? (n_nodes + 255) / 256 : 4096);
    fill_words_kernel<int32_t><<<gn, 256, 0, st>>>(first, INT_MAX, n_nodes);
    GK_LAUNCHED("plan_fill");
    const unsigned gc = (unsigned)((C + 255) / 256 < 8192 ? (C + 255) / 256 : 8192);
    node_ranges_kernel<I><<<gc ? gc : 1, 256, 0, st>>>(row, indptr, C, n_nodes, first, deg);
    GK_LAUNCHED("plan_node_ranges");
  }
  // row-aligned boundaries of the work tiles the ops will use for this many positions
  const int tile = pick_tile(E);
  const long long n_tiles = (E + tile - 1) / tile;
  int32_t* tile_start = (int32_t*)ar.take((size_t)(n_tiles + 1) * 4);
  if (ar.overflow) return GRAPHOP_ERR_WORKSPACE;
  {
    const unsigned gb = (unsigned)((n_tiles + 256) / 256 < 4096 ? (n_tiles + 256) / 256 : 4096);
    tile_bounds_kernel<<<gb, 256, 0, st>>>(g.erow, E, tile, n_tiles, tile_start, verdict);
    GK_LAUNCHED("plan_tile_bounds");
  }
  BandVerdict host{1, 0, 1};
  if (g.other && n_nodes > 0) {
    const unsigned ge = (unsigned)((E + 255) / 256 < 8192 ? (E + 255) / 256 : 8192);
    band_positions_kernel<<<ge, 256, 0, st>>>(g.erow, g.other, E, first, verdict);
    GK_LAUNCHED("plan_band_positions");
    const unsigned gt = (unsigned)((n_nodes + kBandTileRows - 1) / kBandTileRows);
    band_tiles_kernel<<<gt, kBandTileRows, 0, st>>>(g.other, first, deg, n_nodes, node_lo, verdict);
    GK_LAUNCHED("plan_band_tiles");
  }
  const bool analysed = g.other && n_nodes > 0;
  GK_CUDA(cudaMemcpyAsync(&host, verdict, sizeof(host), cudaMemcpyDeviceToHost, st));
  GK_CUDA(cudaStreamSynchronize(st));
  plan->band_span = analysed ? host.max_span : 0;
  if (analysed && !host.not_contiguous && host.max_span > 0 && host.max_span <= GRAPHOP_BAND_MAX_SPAN)
    plan->flags |= GRAPHOP_PLAN_DENSE_BAND;
  // Row-aligned tiles are used only where they remove the carry levels altogether.  Where long rows still cross
  // (R-MAT 21: hubs of 10^5 positions) the uneven tiles cost the level-0 kernels more than the fewer partial rows
  // save: the fused step got about 4 % slower, measured.
  plan->tile = tile;
  if (!host.row_crosses) {
    plan->tile_start = tile_start;
    plan->flags |= GRAPHOP_PLAN_ROW_TILES | GRAPHOP_PLAN_NO_CARRY;
  }
  return GRAPHOP_OK;
}

}  // namespace gk
