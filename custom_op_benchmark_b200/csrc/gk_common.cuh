// Shared device machinery of the graphop kernels for sm_100a.
//
// Work decomposition.  Every op sees the graph as a flat stream of CSR positions
// 0..E-1.  A one-pass "expansion" turns the caller's chunk table (row[c], indptr[c]),
// in which several consecutive chunks may belong to one node, into erow[j] = owner node
// of position j (-1 where no chunk covers j).  All other kernels cut the position stream
// into fixed tiles of `tile` positions, one warp per tile, so the work per warp is the
// same whatever the degree distribution looks like: a node with a million in-edges is
// simply spread over thousands of warps, and a thousand one-edge nodes share one warp.
//
// Row-owned reductions without atomics.  Inside a tile a warp walks the positions in
// order; all 32 lanes work on one edge at a time, each lane owning R vector slots of the
// node's H*D feature row, and a run of equal erow[] values is one segment.  A segment
// that lies wholly inside the tile is reduced in registers and stored once.  The first
// segment of a tile whose node already started in an earlier tile ("open head") and the
// last segment of a tile whose node continues in the next one ("open tail") are stored
// as partials in a per-tile carry slot; a second small kernel lets the tile in which the
// node starts fold the carries of the following tiles in ascending tile order.  The sum
// order is therefore a function of (E, tile) only: results are bit-reproducible.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gk {

constexpr int kWarpsPerCta = 8;
constexpr unsigned kFull = 0xffffffffu;

struct PlanHeader {
  long long cover_lo;  // first CSR position any chunk covers  (= indptr[0])
  long long cover_hi;  // one past the last covered position   (= indptr[C])
};

// ---------------------------------------------------------------------------------------
// element types: storage type T, accumulation type AccOf<T>
// ---------------------------------------------------------------------------------------
template <typename T> struct AccOf { using type = float; };
template <> struct AccOf<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename AccOf<T>::type to_acc(T v) { return v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_acc(typename AccOf<T>::type v) { return (T)v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float gk_exp(float x) { return expf(x); }
__device__ __forceinline__ double gk_exp(double x) { return exp(x); }
__device__ __forceinline__ float gk_log(float x) { return logf(x); }
__device__ __forceinline__ double gk_log(double x) { return log(x); }
template <typename A> __device__ __forceinline__ A neg_inf();
template <> __device__ __forceinline__ float neg_inf<float>() { return -INFINITY; }
template <> __device__ __forceinline__ double neg_inf<double>() { return -(double)INFINITY; }

// V consecutive elements of T moved with one load/store of V*sizeof(T) bytes (4, 8 or 16).
template <typename T, int V> struct alignas(sizeof(T) * V) Pack { T v[V]; };

template <int BYTES> struct Mover;
template <> struct Mover<16> { using type = uint4; };
template <> struct Mover<8> { using type = uint2; };
template <> struct Mover<4> { using type = uint32_t; };
template <> struct Mover<2> { using type = uint16_t; };

template <typename T, int V>
__device__ __forceinline__ void load_acc(typename AccOf<T>::type (&dst)[V], const T* __restrict__ p) {
  using M = typename Mover<sizeof(T) * V>::type;
  union { M m; T t[V]; } u;
  u.m = __ldg(reinterpret_cast<const M*>(p));
#pragma unroll
  for (int i = 0; i < V; ++i) dst[i] = to_acc<T>(u.t[i]);
}

template <typename T, int V>
__device__ __forceinline__ void store_acc(T* __restrict__ p, const typename AccOf<T>::type (&src)[V]) {
  using M = typename Mover<sizeof(T) * V>::type;
  union { M m; T t[V]; } u;
#pragma unroll
  for (int i = 0; i < V; ++i) u.t[i] = from_acc<T>(src[i]);
  *reinterpret_cast<M*>(p) = u.m;
}

// plain (non-converting) vector moves for the accumulation type itself: carries
template <typename A, int V>
__device__ __forceinline__ void load_raw(A (&dst)[V], const A* p) {
#pragma unroll
  for (int i = 0; i < V; ++i) dst[i] = p[i];
}
template <typename A, int V>
__device__ __forceinline__ void store_raw(A* p, const A (&src)[V]) {
#pragma unroll
  for (int i = 0; i < V; ++i) p[i] = src[i];
}

// Every cross-lane sum in these kernels is a butterfly over lane distances 1, 2, 4, ... in that order, whichever
// routine forms it: two kernels that reduce the same per-lane partials (delta in the destination pass, dO . v in
// the source pass) then agree bit for bit.
template <typename A> __device__ __forceinline__ A warp_sum(A v) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}

// One value per lane summed over the LPH lanes of a head, lane distances 1, 2, 4, ... in that order.
template <int LPH, typename A>
__device__ __forceinline__ A reduce_ascending(A v) {
#pragma unroll
  for (int o = 1; o < LPH; o <<= 1) v += __shfl_xor_sync(kFull, v, o);
  return v;
}

// Per-lane view of a node's feature row: lane owns slots lane, lane+32, ..., each V elements.
template <int R> struct SlotMap {
  int head[R];  // head index of the slot
  int feat[R];  // element offset of the slot inside the H*D row
  int efeat[R]; // element offset inside one head's D-vector (edge-feature operands)
  bool ok[R];   // slot exists (slot < S)
  __device__ __forceinline__ void init(int lane, int S, int V, int D, int feat0) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int s = lane + 32 * i;
      ok[i] = s < S;
      const int el = feat0 + (ok[i] ? s : 0) * V;
      feat[i] = el;
      head[i] = el / D;
      efeat[i] = el - head[i] * D;
    }
  }
};

// Sums the per-register partial dot products over the lanes (and registers) that hold the
// same head; afterwards every lane holds the head's total in each of its registers.
// lph = lanes (vector slots) per head, a power of two.
template <typename A, int R>
__device__ __forceinline__ void reduce_heads(A (&p)[R], int lph) {
  if (lph >= 32) {
    const int rph = lph >> 5;  // registers per head
#pragma unroll
    for (int s = 1; s < R; s <<= 1) {
      if (s < rph) {
        A t[R];
#pragma unroll
        for (int i = 0; i < R; ++i) t[i] = p[i ^ s];
#pragma unroll
        for (int i = 0; i < R; ++i) p[i] += t[i];
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) p[i] = warp_sum(p[i]);
  } else {
    for (int o = 1; o < lph; o <<= 1) {
#pragma unroll
      for (int i = 0; i < R; ++i) p[i] += __shfl_xor_sync(kFull, p[i], o);
    }
  }
}

// ---------------------------------------------------------------------------------------
// expansion: chunk table -> erow[], optional int64 -> int32 copies of indices / eid
// ---------------------------------------------------------------------------------------
constexpr int kExpandTile = 256;  // positions per warp

template <typename I>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
expand_rows_kernel(const I* __restrict__ row, const I* __restrict__ indptr, long long C, long long E,
                   int32_t* __restrict__ erow, PlanHeader* __restrict__ hdr) {
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  const long long p0 = t * kExpandTile;
  const long long base = (long long)indptr[0];
  const long long end = (long long)indptr[C];
  if (t == 0 && lane == 0) {
    hdr->cover_lo = base;
    hdr->cover_hi = end < base ? base : end;
  }
  if (p0 >= E) return;
  const long long p1 = p0 + kExpandTile < E ? p0 + kExpandTile : E;
  const long long lo = p0 > base ? p0 : base;
  const long long hi = p1 < end ? p1 : end;
  // positions of this tile outside [base, end) belong to no chunk
  for (long long p = p0 + lane; p < p1; p += 32)
    if (p < lo || p >= hi) erow[p] = -1;
  if (lo >= hi) return;
  // chunk that contains position lo: the last c with indptr[c] <= lo
  // 32-way search: every lane probes one pivot strictly inside (a, b), the ballot picks the sub-range;
  // 5 dependent loads for a million chunks instead of 20
  long long a = 0, b = C;  // invariant: indptr[a] <= lo < indptr[b] (indptr[C] = end > lo)
  while (b - a > 1) {
    const long long span = b - a;
    long long m = a + (span * (lane + 1)) / 33;  // non-decreasing in the lane index
    m = m <= a ? a + 1 : (m >= b ? b - 1 : m);
    const unsigned le = __ballot_sync(kFull, (long long)indptr[m] <= lo);  // a prefix of the lanes
    const int cnt = __popc(le);
    const long long below = __shfl_sync(kFull, m, cnt ? cnt - 1 : 0);
    const long long above = __shfl_sync(kFull, m, cnt < 32 ? cnt : 31);
    if (cnt) a = below;
    if (cnt < 32) b = above;
  }
  // 32 chunks at a time: lane l holds chunk a + l; every position of the part of the tile they cover
  // finds its chunk by a 5-step search over the lanes' start positions, so that the stores are
  // coalesced whatever the chunk lengths are
  for (long long c = a; c < C; c += 32) {
    const long long cc = c + lane;
    long long s = hi, e = hi;
    int r = -1;
    if (cc < C) {
      s = (long long)indptr[cc];
      e = (long long)indptr[cc + 1];
      r = (int)row[cc];
    }
    const bool past = s >= hi;  // this chunk starts at or beyond the end of the tile
    s = s < lo ? lo : (s > hi ? hi : s);
    e = e < lo ? lo : (e > hi ? hi : e);
    const int s_rel = (int)(s - lo);  // 0 .. kExpandTile, non-decreasing over the lanes
    const long long from = __shfl_sync(kFull, s, 0);
    const long long to = __shfl_sync(kFull, e, 31);
    for (long long q = from; q < to; q += 32) {
      const long long p = q + lane;
      const int p_rel = (int)(p - lo);
      int owner = 0;  // the last lane whose chunk starts at or before p
#pragma unroll
      for (int step = 16; step; step >>= 1) {
        const int cand = owner + step;
        const int start = __shfl_sync(kFull, s_rel, cand & 31);
        if (cand < 32 && start <= p_rel) owner = cand;
      }
      const int rr = __shfl_sync(kFull, r, owner);
      if (p < to) erow[p] = rr;
    }
    if (__any_sync(kFull, past)) break;
  }
}

template <typename I>
__global__ void narrow_index_kernel(const I* __restrict__ src, int32_t* __restrict__ dst, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = (int32_t)src[i];
}

// Edge outputs start from zero in the reference (at::zeros); only edge ids that some chunk
// covers are written by the kernels here, so when the chunk table does not cover all E
// positions the output is cleared first.  With full coverage this kernel returns at once.
template <typename W>
__global__ void zero_uncovered_kernel(const PlanHeader* __restrict__ hdr, long long E, W* __restrict__ out,
                                      long long n_words) {
  if (hdr->cover_hi - hdr->cover_lo >= E) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_words; i += stride) out[i] = W(0);
}

// ---------------------------------------------------------------------------------------
// the tile walker
// ---------------------------------------------------------------------------------------
// Op interface (all members __device__):
//   static constexpr bool kRowOut;   // produces one output row per node (needs carries, gap fill)
//   static constexpr int  kUnroll;   // edges fetched ahead of the consuming loop
//   struct State; struct Fetched;
//   void setup(State&, int lane)                       once per warp
//   void begin(State&, int node, int lane)             a segment of `node` starts
//   void fetch(const State&, Fetched&, int other, int edge, int lane)   issue the edge's loads
//   void consume(State&, const Fetched&, int lane)     fold the edge into the state
//   -- kRowOut only --
//   struct CarryIn;
//   void store_row(const State&, int node, int lane)   the state is the node's final value
//   void store_carry(const State&, long long slot, int lane)    partial of an open segment
//   void store_identity(const State&, long long slot, int lane) neutral partial
//   void begin_merge(State&, int node, int lane)       neutral state, nothing loaded
//   void fetch_carry(const State&, CarryIn&, long long slot, int lane)   issue the loads of a stored partial
//   void merge_carry(State&, const CarryIn&, int lane)          fold it into the state
//   void zero_rows(long long lo, long long hi, int lane)        nodes [lo, hi) have no edge
//
// Level 0 (kCarryLevel = false) walks CSR positions.  A node whose positions cross a tile
// boundary is never stored at level 0: every tile writes the partial of its open first
// segment to carry slot 2t and of its open last segment to slot 2t+1, and rows_next[2t],
// rows_next[2t+1] name the node each slot belongs to (-1: slot unused).  A tile that lies
// wholly inside one node writes its partial to slot 2t and a neutral partial to 2t+1, so
// the slots of one node are always consecutive.  Level k+1 (kCarryLevel = true) walks that
// slot stream with the same code, merging partials instead of edges, stores the nodes whose
// slots end inside one of its tiles and emits the next, 128-times shorter stream, until a
// level fits one tile.  Every merge order is a function of (E, tile sizes) only.
template <class Op, bool kCarryLevel>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
walk_kernel(Op op, const PlanHeader* __restrict__ hdr, const int32_t* __restrict__ erow,
            const int32_t* __restrict__ other, const int32_t* __restrict__ eid, long long E, int tile,
            long long n_rows, int32_t* __restrict__ rows_next, const int32_t* __restrict__ tile_start) {
  constexpr int U = Op::kUnroll;
  constexpr bool kOut = Op::kRowOut;
  constexpr bool kFill = Op::kRowOut && !kCarryLevel;
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  // tile t covers positions [t * tile, (t + 1) * tile), or, with a plan's row-aligned boundaries,
  // [tile_start[t], tile_start[t + 1]): the same number of tiles, each boundary moved up to the next row start
  if (t * tile >= E) return;
  const long long j0 = tile_start ? (long long)__ldg(tile_start + t) : t * tile;
  const long long j1 = tile_start ? (long long)__ldg(tile_start + t + 1) : (j0 + tile < E ? j0 + tile : E);

  if constexpr (kFill) {
    if (t == 0 && hdr->cover_hi <= hdr->cover_lo) {  // no covered position at all
      op.zero_rows(0, n_rows, lane);
      if (rows_next && lane == 0) { rows_next[0] = -1; rows_next[1] = -1; }
      return;
    }
  }

  typename Op::State st;
  op.setup(st, lane);
  const int before = j0 > 0 ? __ldg(erow + j0 - 1) : -1;
  const int first = __ldg(erow + j0);
  const bool head_open = before >= 0 && before == first;
  bool first_seg = true;    // the segment being built is the tile's first one
  int cur = -1;             // node of the segment being built, -1: none
  int last_valid = before;  // last node seen so far in position order (-1: none yet)
  int head_row = -1;        // node whose partial went to slot 2t

  for (long long jb = j0; jb < j1; jb += 32) {
    const long long j = jb + lane;
    const bool inb = j < j1;
    const int my_row = inb ? __ldg(erow + j) : -1;
    const int my_other = (!kCarryLevel && inb && other) ? __ldg(other + j) : 0;
    const int my_eid = (!kCarryLevel && inb && eid) ? __ldg(eid + j) : (int)j;
    const int n = (int)(j1 - jb < 32 ? j1 - jb : 32);
    // 32 positions without a node and no segment open: nothing to do (most slots of a carry level)
    if (cur < 0 && __ballot_sync(kFull, my_row >= 0) == 0u) continue;
    for (int k = 0; k < n; k += U) {
      typename Op::Fetched f[U];
      typename Op::CarryIn ci[U];
      int rr[U];
      (void)f; (void)ci;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int kk = (k + u) & 31;
        const int r = __shfl_sync(kFull, my_row, kk);
        rr[u] = (k + u < n) ? r : -2;  // -2: beyond the tile, ignore
        if constexpr (kCarryLevel) {
          if (rr[u] >= 0) op.fetch_carry(st, ci[u], jb + k + u, lane);
        } else {
          const int c = __shfl_sync(kFull, my_other, kk);
          const int e = __shfl_sync(kFull, my_eid, kk);
          if (rr[u] >= 0) op.fetch(st, f[u], c, e, lane);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int r = rr[u];
        if (r == -2) continue;
        if (r != cur) {
          if (cur >= 0) {
            if constexpr (kOut) {
              if (first_seg && head_open) { op.store_carry(st, 2 * t, lane); head_row = cur; }
              else op.store_row(st, cur, lane);
            }
            first_seg = false;
            if constexpr (kFill) {
              if (r < 0) op.zero_rows((long long)cur + 1, n_rows, lane);  // coverage ended
            }
          }
          if (r >= 0) {
            if constexpr (kFill) {
              if (!(first_seg && head_open)) op.zero_rows((long long)last_valid + 1, r, lane);
            }
            if constexpr (kCarryLevel) op.begin_merge(st, r, lane); else op.begin(st, r, lane);
            last_valid = r;
          }
          cur = r;
        }
        if (r >= 0) {
          if constexpr (kCarryLevel) op.merge_carry(st, ci[u], lane); else op.consume(st, f[u], lane);
        }
      }
    }
  }
  int tail_row = -1;
  if constexpr (kOut) {
   if (cur >= 0) {
    const int next = j1 < E ? __ldg(erow + j1) : -1;
    const bool tail_open = next == cur;
    if (first_seg && head_open) {  // the whole tile lies inside one node that started earlier
      op.store_carry(st, 2 * t, lane);
      head_row = cur;
      if (tail_open) { op.store_identity(st, 2 * t + 1, lane); tail_row = cur; }
    } else if (tail_open) {
      op.store_carry(st, 2 * t + 1, lane);
      tail_row = cur;
    } else {
      op.store_row(st, cur, lane);
    }
    if constexpr (kFill) {
      if (next < 0) op.zero_rows((long long)cur + 1, n_rows, lane);  // last covered position
    }
   }
   if (rows_next && lane == 0) { rows_next[2 * t] = head_row; rows_next[2 * t + 1] = tail_row; }
  }
}

}  // namespace gk
