// Sparse row softmax over each node's edges, forward and backward
// (reference: graphop_kernel.cu:170-202 and :208-230, three and two launches of h-thread
// blocks with one atomic per edge; here one streaming pass with segmented warp scans).
//
// Mapping: one lane per CSR position, all H heads of the edge in that lane, so a warp moves
// 32 consecutive (E, H) rows per step with vector loads.  A tile is kSteps steps.  Runs of
// equal erow[] inside the tile are segments; segment boundaries are ballots, a lane finds
// its segment's first and last lane with bit scans, and max / sum over a segment is a
// Hillis-Steele scan that stops at the segment's first lane.  Per-segment results live in
// shared memory (one slot per local segment, written by the segment's last lane of each
// step, steps in order), so the order of every sum is fixed.
//
// Nodes whose positions cross a tile boundary: the tile writes the partial statistics of
// its open first / last segment to carry slots 2t / 2t+1 exactly like the vector walker,
// the carry levels (walk_kernel with SegStatOp) merge them into stats[node], and
// softmax_*_finish_kernel revisits only the positions of open segments.
#pragma once
#include "gk_common.cuh"

namespace gk {

constexpr int kSoftmaxWarps = 4;

template <typename T, int N>
__device__ __forceinline__ void load_vec(typename AccOf<T>::type (&dst)[N], const T* __restrict__ p) {
  constexpr int kPer = (N * (int)sizeof(T) <= 16) ? N : 16 / (int)sizeof(T);
#pragma unroll
  for (int c = 0; c < N / kPer; ++c) {
    typename AccOf<T>::type tmp[kPer];
    load_acc<T, kPer>(tmp, p + c * kPer);
#pragma unroll
    for (int i = 0; i < kPer; ++i) dst[c * kPer + i] = tmp[i];
  }
}
template <typename T, int N>
__device__ __forceinline__ void store_vec(T* __restrict__ p, const typename AccOf<T>::type (&src)[N]) {
  constexpr int kPer = (N * (int)sizeof(T) <= 16) ? N : 16 / (int)sizeof(T);
#pragma unroll
  for (int c = 0; c < N / kPer; ++c) {
    typename AccOf<T>::type tmp[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) tmp[i] = src[c * kPer + i];
    store_acc<T, kPer>(p + c * kPer, tmp);
  }
}

// Segment geometry of one 32-position step.
struct StepSeg {
  int sid;          // tile-local segment index of this lane's position
  int lo;           // first lane of the segment inside this step
  bool last;        // this lane is the segment's last lane inside this step
  bool starts;      // the segment starts inside this step (else it continues the previous step)
};

__device__ __forceinline__ StepSeg step_geometry(unsigned mask, int sbase, int lane) {
  const unsigned le = 0xffffffffu >> (31 - lane);  // bits 0..lane
  StepSeg g;
  g.sid = sbase + __popc(mask & le) - 1;
  g.lo = 31 - __clz((mask | 1u) & le);
  const unsigned upper = mask & ~le;
  const int hi = upper ? __ffs(upper) - 1 : 32;
  g.last = lane == hi - 1;
  g.starts = (mask >> g.lo) & 1u;
  return g;
}

template <typename A, int H, bool kMax>
__device__ __forceinline__ void seg_scan(A (&v)[H], int lo, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const A t = __shfl_up_sync(kFull, v[h], d);
      if (lane - d >= lo) v[h] = kMax ? (t > v[h] ? t : v[h]) : v[h] + t;
    }
  }
}

template <int H> struct SoftmaxSteps { static constexpr int value = H <= 4 ? 4 : 2; };

// Forward (kBackward = false):  y = exp(x - max) / sum exp(x - max) per (node, head).
//   in0 = x, in1 unused; carry slot = [H max][H sum]
// Backward (kBackward = true):  dx = y * (dy - sum_node dy * y).
//   in0 = y, in1 = dy;   carry slot = [H sum]
// hs / h0: the (E, hs) tensors are read at columns h0 .. h0 + H - 1.
template <typename T, int H, bool kBackward>
__global__ void __launch_bounds__(kSoftmaxWarps * 32)
softmax_tile_kernel(const int32_t* __restrict__ erow, const int32_t* __restrict__ eid, const T* __restrict__ in0,
                    const T* __restrict__ in1, T* __restrict__ out, typename AccOf<T>::type* __restrict__ carry,
                    int32_t* __restrict__ rows_next, long long E, int hs, int h0) {
  using A = typename AccOf<T>::type;
  constexpr int kSteps = SoftmaxSteps<H>::value;
  constexpr int kTile = kSteps * 32;
  constexpr int kCarry = kBackward ? H : 2 * H;
  __shared__ A s_a[kSoftmaxWarps][kTile][H];                       // max (fwd) / sum (bwd)
  __shared__ A s_b[kBackward ? 1 : kSoftmaxWarps][kBackward ? 1 : kTile][H];  // sum (fwd)
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  const long long t = (long long)blockIdx.x * kSoftmaxWarps + w;
  const long long j0 = t * kTile;
  if (j0 >= E) return;
  const long long j1 = j0 + kTile < E ? j0 + kTile : E;
  const int before = j0 > 0 ? __ldg(erow + j0 - 1) : -1;
  const int next = j1 < E ? __ldg(erow + j1) : -1;

  int rw[kSteps];
  long long ed[kSteps];
  A a[kSteps][H];   // x (fwd) / y (bwd); later exp(x - max) (fwd)
  A b[kSteps][H];   // dy (bwd)
  unsigned mask[kSteps];
  int prev_last = before;
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const long long j = j0 + 32 * s + lane;
    const bool inb = j < j1;
    rw[s] = inb ? __ldg(erow + j) : -1;
    ed[s] = inb ? (eid ? (long long)__ldg(eid + j) : j) : 0;
    if (rw[s] >= 0) {
      load_vec<T, H>(a[s], in0 + ed[s] * hs + h0);
      if (kBackward) load_vec<T, H>(b[s], in1 + ed[s] * hs + h0);
    } else {
#pragma unroll
      for (int h = 0; h < H; ++h) { a[s][h] = A(0); b[s][h] = A(0); }
    }
    int up = __shfl_up_sync(kFull, rw[s], 1);
    if (lane == 0) up = prev_last;
    mask[s] = __ballot_sync(kFull, rw[s] != up || (s == 0 && lane == 0));
    prev_last = __shfl_sync(kFull, rw[s], 31);
  }
  const int row0 = __shfl_sync(kFull, rw[0], 0);
  const bool head_open = before >= 0 && before == row0;
  // last position of the tile: its node and its segment
  const int last_off = (int)(j1 - 1 - j0);
  int last_row = -1, last_sid = 0;

  StepSeg g[kSteps];
  int sbase = 0;
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    g[s] = step_geometry(mask[s], sbase, lane);
    sbase += __popc(mask[s]);
    if ((last_off >> 5) == s) {
      last_row = __shfl_sync(kFull, rw[s], last_off & 31);
      last_sid = __shfl_sync(kFull, g[s].sid, last_off & 31);
    }
  }
  const bool tail_open = last_row >= 0 && next == last_row;

  if (!kBackward) {
    // pass 1: segment maxima
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      A v[H];
#pragma unroll
      for (int h = 0; h < H; ++h) v[h] = rw[s] >= 0 ? a[s][h] : neg_inf<A>();
      seg_scan<A, H, true>(v, g[s].lo, lane);
      if (g[s].last) {
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const A old = g[s].starts ? neg_inf<A>() : s_a[w][g[s].sid][h];
          s_a[w][g[s].sid][h] = old > v[h] ? old : v[h];
        }
      }
      __syncwarp();
    }
    // pass 2: exponentials and their segment sums
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      A v[H];
#pragma unroll
      for (int h = 0; h < H; ++h) {
        a[s][h] = rw[s] >= 0 ? gk_exp(a[s][h] - s_a[w][g[s].sid][h]) : A(0);
        v[h] = a[s][h];
      }
      seg_scan<A, H, false>(v, g[s].lo, lane);
      if (g[s].last) {
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const A old = g[s].starts ? A(0) : s_b[w][g[s].sid][h];
          s_b[w][g[s].sid][h] = old + v[h];
        }
      }
      __syncwarp();
    }
  } else {
#pragma unroll
    for (int s = 0; s < kSteps; ++s) {
      A v[H];
#pragma unroll
      for (int h = 0; h < H; ++h) v[h] = a[s][h] * b[s][h];
      seg_scan<A, H, false>(v, g[s].lo, lane);
      if (g[s].last) {
#pragma unroll
        for (int h = 0; h < H; ++h) {
          const A old = g[s].starts ? A(0) : s_a[w][g[s].sid][h];
          s_a[w][g[s].sid][h] = old + v[h];
        }
      }
      __syncwarp();
    }
  }

  // pass 3: positions of closed segments are final
#pragma unroll
  for (int s = 0; s < kSteps; ++s) {
    const int sid = g[s].sid;
    const bool open = (sid == 0 && head_open) || (sid == last_sid && tail_open);
    if (rw[s] >= 0 && !open) {
      A r[H];
#pragma unroll
      for (int h = 0; h < H; ++h) {
        if (kBackward) r[h] = a[s][h] * (b[s][h] - s_a[w][sid][h]);
        else r[h] = a[s][h] / s_b[w][sid][h];
      }
      store_vec<T, H>(out + ed[s] * hs + h0, r);
    }
  }

  // partial statistics of the open segments -> carry slots, same slot rules as walk_kernel
  if (lane < H) {
    const int h = lane;
    A* c0 = carry + (2 * t) * kCarry;
    A* c1 = carry + (2 * t + 1) * kCarry;
    const bool whole = head_open && last_sid == 0;  // the tile lies inside one node that started earlier
    if (head_open) {
      c0[h] = s_a[w][0][h];
      if (!kBackward) c0[H + h] = s_b[w][0][h];
    }
    if (tail_open) {
      if (whole) {
        c1[h] = kBackward ? A(0) : neg_inf<A>();
        if (!kBackward) c1[H + h] = A(0);
      } else {
        c1[h] = s_a[w][last_sid][h];
        if (!kBackward) c1[H + h] = s_b[w][last_sid][h];
      }
    }
  }
  if (lane == 0) {
    rows_next[2 * t] = head_open ? row0 : -1;
    rows_next[2 * t + 1] = tail_open ? last_row : -1;
  }
}

// Revisits the positions of open segments once stats[node] holds the node's merged
// statistics: forward stats = [H max][H sum] per node, backward stats = [H sum].
template <typename T, int H, bool kBackward>
__global__ void __launch_bounds__(kSoftmaxWarps * 32)
softmax_finish_kernel(const int32_t* __restrict__ erow, const int32_t* __restrict__ eid, const T* __restrict__ in0,
                      const T* __restrict__ in1, T* __restrict__ out,
                      const typename AccOf<T>::type* __restrict__ stats, long long n_nodes, long long E, int hs,
                      int h0) {
  using A = typename AccOf<T>::type;
  constexpr int kSteps = SoftmaxSteps<H>::value;
  constexpr int kTile = kSteps * 32;
  constexpr int kStat = kBackward ? H : 2 * H;
  const int lane = threadIdx.x & 31;
  const long long t = (long long)blockIdx.x * kSoftmaxWarps + (threadIdx.x >> 5);
  const long long j0 = t * kTile;
  if (j0 >= E) return;
  const long long j1 = j0 + kTile < E ? j0 + kTile : E;
  const int before = j0 > 0 ? __ldg(erow + j0 - 1) : -1;
  const int next = j1 < E ? __ldg(erow + j1) : -1;
  const int row0 = __ldg(erow + j0);
  const int last_row = __ldg(erow + j1 - 1);
  const bool head_open = before >= 0 && before == row0;
  const bool tail_open = last_row >= 0 && next == last_row;
  if (!head_open && !tail_open) return;
  for (long long j = j0 + lane; j < j1; j += 32) {
    const int r = __ldg(erow + j);
    if (r < 0 || r >= n_nodes) continue;  // a node id beyond the caller's bound has no statistics slot
    if (!((head_open && r == row0) || (tail_open && r == last_row))) continue;
    const long long e = eid ? (long long)__ldg(eid + j) : j;
    A a[H], o[H];
    load_vec<T, H>(a, in0 + e * hs + h0);
    const A* st = stats + (long long)r * kStat;
    if (kBackward) {
      A b[H];
      load_vec<T, H>(b, in1 + e * hs + h0);
#pragma unroll
      for (int h = 0; h < H; ++h) o[h] = a[h] * (b[h] - st[h]);
    } else {
#pragma unroll
      for (int h = 0; h < H; ++h) o[h] = gk_exp(a[h] - st[h]) / st[H + h];
    }
    store_vec<T, H>(out + e * hs + h0, o);
  }
}

// Carry-level op for the softmax statistics: lane h owns head h.
template <typename A, bool kPair>
struct SegStatOp {
  static constexpr bool kRowOut = true;
  static constexpr int kUnroll = 8;
  A* __restrict__ stats;      // (n_nodes, kPair ? 2H : H)
  A* __restrict__ carry;
  const A* carry_in;
  int H;
  long long n_nodes;          // rows of `stats`
  static constexpr int kW = kPair ? 2 : 1;
  struct State { A m, l; };
  struct Fetched {};
  struct CarryIn { A m, l; };
  __device__ __forceinline__ void setup(State&, int) const {}
  __device__ __forceinline__ void begin(State&, int, int) const {}
  __device__ __forceinline__ void fetch(const State&, Fetched&, int, int, int) const {}
  __device__ __forceinline__ void consume(State&, const Fetched&, int) const {}
  __device__ __forceinline__ void begin_merge(State& st, int, int) const {
    st.m = kPair ? neg_inf<A>() : A(0);
    st.l = A(0);
  }
  __device__ __forceinline__ void fetch_carry(const State&, CarryIn& c, long long slot, int lane) const {
    if (lane < H) {
      c.m = carry_in[slot * kW * H + lane];
      c.l = kPair ? carry_in[slot * kW * H + H + lane] : A(0);
    }
  }
  __device__ __forceinline__ void merge_carry(State& st, const CarryIn& c, int lane) const {
    if (lane >= H) return;
    if (kPair) {
      const A mn = c.m > st.m ? c.m : st.m;
      const A wa = st.m == neg_inf<A>() ? A(0) : gk_exp(st.m - mn);
      const A wb = c.m == neg_inf<A>() ? A(0) : gk_exp(c.m - mn);
      st.l = st.l * wa + c.l * wb;
      st.m = mn;
    } else {
      st.m += c.m;
    }
  }
  __device__ __forceinline__ void store_row(const State& st, int node, int lane) const {
    if (lane < H && node < n_nodes) {
      stats[(long long)node * kW * H + lane] = st.m;
      if (kPair) stats[(long long)node * kW * H + H + lane] = st.l;
    }
  }
  __device__ __forceinline__ void store_carry(const State& st, long long slot, int lane) const {
    if (lane < H) {
      carry[slot * kW * H + lane] = st.m;
      if (kPair) carry[slot * kW * H + H + lane] = st.l;
    }
  }
  __device__ __forceinline__ void store_identity(const State&, long long slot, int lane) const {
    if (lane < H) {
      carry[slot * kW * H + lane] = kPair ? neg_inf<A>() : A(0);
      if (kPair) carry[slot * kW * H + H + lane] = A(0);
    }
  }
  __device__ __forceinline__ void zero_rows(long long, long long, int) const {}
};

}  // namespace gk
