// The per-edge bodies ("ops") that the tile walker of gk_common.cuh drives, one per
// reference kernel family.  Each op cites the reference kernel whose arithmetic it computes
// (graphop/graphop_kernel.cu); none of them shares its scheduling: no transposed copies of
// the node tensors, no atomics, 128-bit loads of whole feature rows.
#pragma once
#include "gk_common.cuh"

namespace gk {

// ---------------------------------------------------------------------------------------
// Edge-weighted aggregation of gathered feature rows:
//     out[node, h, :] = sum over the node's positions k of  w[eid[k], h] * feat(k)[h, :]
// feat(k) = x[other[k]]            (kEdgeFeat = false)  -> vector_spmm forward
//                                   (graphop_kernel.cu:123-128), vector_spmm backward dx over
//                                   the transposed CSR (:156-161), maskedmm backward dA / dB
//                                   (:105-110, w = dy, x = B or A)
// feat(k) = xe[eid[k]] (one D-vector shared by all heads, kEdgeFeat = true)
//                                   -> node_mul_edge backward dA (graphop_kernel.cu:66-71)
// ---------------------------------------------------------------------------------------
template <typename T, int V, int R, bool kEdgeFeat>
struct AggregateOp {
  using A = typename AccOf<T>::type;
  static constexpr const char* kName = kEdgeFeat ? "aggregate_edge_feat" : "aggregate";
  static constexpr bool kRowOut = true;
  static constexpr int kUnroll = (R * V * (int)sizeof(A) <= 16) ? 8 : (R * V * (int)sizeof(A) <= 32 ? 4 : 2);
  const T* __restrict__ w;    // (E, H)
  const T* __restrict__ x;    // (n_src, H, D) or (E, D)
  T* __restrict__ y;          // (n_dst, H, D)
  A* __restrict__ carry;      // (2 * n_tiles, HD) partial rows written by this level
  const A* carry_in;          // partial rows of the level below (carry levels only)
  int H, D, HD, S, feat0;

  struct State { SlotMap<R> sm; A acc[R][V]; };
  struct Fetched { A w[R]; A x[R][V]; };
  struct CarryIn { A x[R][V]; };

  __device__ __forceinline__ void setup(State& st, int lane) const { st.sm.init(lane, S, V, D, feat0); }
  __device__ __forceinline__ void begin(State& st, int, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int v = 0; v < V; ++v) st.acc[i][v] = A(0);
  }
  __device__ __forceinline__ void fetch(const State& st, Fetched& f, int c, int e, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (st.sm.ok[i]) {
        f.w[i] = to_acc<T>(__ldg(w + (long long)e * H + st.sm.head[i]));
        const T* src = kEdgeFeat ? x + (long long)e * D + st.sm.efeat[i] : x + (long long)c * HD + st.sm.feat[i];
        load_acc<T, V>(f.x[i], src);
      }
    }
  }
  __device__ __forceinline__ void consume(State& st, const Fetched& f, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int v = 0; v < V; ++v) st.acc[i][v] += f.w[i] * f.x[i][v];
  }
  __device__ __forceinline__ void store_row(const State& st, int node, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) store_acc<T, V>(y + (long long)node * HD + st.sm.feat[i], st.acc[i]);
  }
  __device__ __forceinline__ void store_carry(const State& st, long long slot, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) store_raw<A, V>(carry + slot * HD + st.sm.feat[i], st.acc[i]);
  }
  __device__ __forceinline__ void store_identity(const State& st, long long slot, int) const {
    A z[V];
#pragma unroll
    for (int v = 0; v < V; ++v) z[v] = A(0);
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) store_raw<A, V>(carry + slot * HD + st.sm.feat[i], z);
  }
  __device__ __forceinline__ void begin_merge(State& st, int node, int lane) const { begin(st, node, lane); }
  __device__ __forceinline__ void fetch_carry(const State& st, CarryIn& c, long long slot, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) load_raw<A, V>(c.x[i], carry_in + slot * HD + st.sm.feat[i]);
  }
  __device__ __forceinline__ void merge_carry(State& st, const CarryIn& c, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
#pragma unroll
        for (int v = 0; v < V; ++v) st.acc[i][v] += c.x[i][v];
      }
  }
  __device__ __forceinline__ void zero_rows(long long lo, long long hi, int lane) const {
    if (hi <= lo) return;
    A z[V];
#pragma unroll
    for (int v = 0; v < V; ++v) z[v] = A(0);
    const long long n = (hi - lo) * S;
    for (long long k = lane; k < n; k += 32) {
      const long long node = lo + k / S;
      const int s = (int)(k % S);
      store_acc<T, V>(y + node * HD + feat0 + s * V, z);
    }
  }
};

// ---------------------------------------------------------------------------------------
// Sampled dot products on the edges:
//     y[eid[k], h] = sum_d a[node(k), h, d] * feat(k)[h, d]
// feat(k) = b[other[k]]  -> maskedmm forward (graphop_kernel.cu:45-53) and the dedata half of
//                           vector_spmm backward (:140-147, a = dy, b = x)
// feat(k) = be[eid[k]]   -> node_mul_edge forward (graphop_kernel.cu:24-32)
// The node's row of `a` stays in registers for the whole segment.
// ---------------------------------------------------------------------------------------
template <typename T, int V, int R, bool kEdgeFeat>
struct EdgeDotOp {
  using A = typename AccOf<T>::type;
  static constexpr const char* kName = "edge_dot";
  static constexpr bool kRowOut = false;
  static constexpr int kUnroll = (R * V * (int)sizeof(A) <= 16) ? 8 : (R * V * (int)sizeof(A) <= 32 ? 4 : 2);
  const T* __restrict__ a;  // (n_dst, H, D)
  const T* __restrict__ b;  // (n_src, H, D) or (E, D)
  T* __restrict__ y;        // (E, H)
  int H, D, HD, S, lph;

  struct State { SlotMap<R> sm; A a[R][V]; };
  struct Fetched { A b[R][V]; int e; };
  struct CarryIn {};

  __device__ __forceinline__ void setup(State& st, int lane) const { st.sm.init(lane, S, V, D, 0); }
  __device__ __forceinline__ void begin(State& st, int node, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (st.sm.ok[i]) load_acc<T, V>(st.a[i], a + (long long)node * HD + st.sm.feat[i]);
      else
#pragma unroll
        for (int v = 0; v < V; ++v) st.a[i][v] = A(0);
    }
  }
  __device__ __forceinline__ void fetch(const State& st, Fetched& f, int c, int e, int) const {
    f.e = e;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (st.sm.ok[i]) {
        const T* src = kEdgeFeat ? b + (long long)e * D + st.sm.efeat[i] : b + (long long)c * HD + st.sm.feat[i];
        load_acc<T, V>(f.b[i], src);
      } else {
#pragma unroll
        for (int v = 0; v < V; ++v) f.b[i][v] = A(0);
      }
    }
  }
  __device__ __forceinline__ void consume(State& st, const Fetched& f, int lane) const {
    A p[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      p[i] = A(0);
#pragma unroll
      for (int v = 0; v < V; ++v) p[i] += st.a[i][v] * f.b[i][v];
    }
    reduce_heads<A, R>(p, lph);
    // one lane per head writes: the first lane of the head's lane group, from the first
    // register that holds the head
    if (lph >= 32) {
      const int rph = lph >> 5;
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < R; ++i)
          if (st.sm.ok[i] && (i % rph) == 0) y[(long long)f.e * H + st.sm.head[i]] = from_acc<T>(p[i]);
      }
    } else if ((lane & (lph - 1)) == 0) {
#pragma unroll
      for (int i = 0; i < R; ++i)
        if (st.sm.ok[i]) y[(long long)f.e * H + st.sm.head[i]] = from_acc<T>(p[i]);
    }
  }
};

// Any-shape fallback of EdgeDotOp: scalar loads, a full-warp reduction per head.  Used when
// D is not a power-of-two number of vector slots or H*D exceeds the register-resident limit.
template <typename T, bool kEdgeFeat>
struct EdgeDotAnyOp {
  using A = typename AccOf<T>::type;
  static constexpr bool kRowOut = false;
  static constexpr int kUnroll = 1;
  const T* __restrict__ a;
  const T* __restrict__ b;
  T* __restrict__ y;
  int H, D, HD;
  struct State { int node; };
  struct Fetched { int c, e; };
  struct CarryIn {};
  __device__ __forceinline__ void setup(State&, int) const {}
  __device__ __forceinline__ void begin(State& st, int node, int) const { st.node = node; }
  __device__ __forceinline__ void fetch(const State&, Fetched& f, int c, int e, int) const { f.c = c; f.e = e; }
  __device__ __forceinline__ void consume(State& st, const Fetched& f, int lane) const {
    const T* ar = a + (long long)st.node * HD;
    for (int h = 0; h < H; ++h) {
      const T* br = kEdgeFeat ? b + (long long)f.e * D : b + (long long)f.c * HD + h * D;
      A p = A(0);
      for (int d = lane; d < D; d += 32) p += to_acc<T>(__ldg(ar + h * D + d)) * to_acc<T>(__ldg(br + d));
      p = warp_sum(p);
      if (lane == 0) y[(long long)f.e * H + h] = from_acc<T>(p);
    }
  }
};

// ---------------------------------------------------------------------------------------
// node_mul_edge backward, edge half:  dB[eid[k], :] = sum_h dy[eid[k], h] * A[node(k), h, :]
// (graphop_kernel.cu:84-92).  One thread per (position, D-slot); no reduction across edges.
// ---------------------------------------------------------------------------------------
// kH: the head count when it is 1, 2, 4 or 8 (all of an edge's loads are then issued before the first use),
// 0: read it from H.  ds_shift >= 0: D / V is that power of two (no 64-bit division per element).
template <typename T, int V, int kH>
__global__ void __launch_bounds__(256)
edge_mix_heads_kernel(const int32_t* __restrict__ erow, const int32_t* __restrict__ eid, const T* __restrict__ dy,
                      const T* __restrict__ a, T* __restrict__ db, long long E, int H, int D, int ds_shift) {
  using A = typename AccOf<T>::type;
  const int ds = D / V;
  const int nh = kH ? kH : H;
  const long long total = E * ds;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const long long j = ds_shift >= 0 ? (idx >> ds_shift) : idx / ds;
    const int s = (int)(idx - j * ds);
    const int node = __ldg(erow + j);
    if (node < 0) continue;
    const long long e = eid ? (long long)__ldg(eid + j) : j;
    const T* arow = a + (long long)node * nh * D + s * V;
    const T* grow = dy + e * nh;
    A acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = A(0);
    if constexpr (kH != 0) {
      A g[kH], av[kH][V];
#pragma unroll
      for (int h = 0; h < kH; ++h) {
        g[h] = to_acc<T>(__ldg(grow + h));
        load_acc<T, V>(av[h], arow + (long long)h * D);
      }
#pragma unroll
      for (int h = 0; h < kH; ++h)
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] += g[h] * av[h][v];
    } else {
      for (int h = 0; h < nh; ++h) {
        const A g = to_acc<T>(__ldg(grow + h));
        A av[V];
        load_acc<T, V>(av, arow + (long long)h * D);
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] += g * av[v];
      }
    }
    store_acc<T, V>(db + e * D + s * V, acc);
  }
}

// ---------------------------------------------------------------------------------------
// Fused attention over the in-edges of every node (no counterpart kernel in the reference;
// it computes what the chain maskedmm -> scale -> sparse_softmax -> vector_spmm computes,
// graphop_kernel.cu:45-53, 175-200, 123-128, without materialising the (E, H) scores):
//     s_k = scale * q[node] . k[other[k]],  p = softmax over the node's edges,
//     o[node] = sum_k p_k v[other[k]],      lse[node] = log sum_k exp(s_k)
// Streaming softmax: running maximum m, running sum l and the running weighted sum are
// rescaled whenever the maximum grows; partials of split nodes merge with the same rule.
// ---------------------------------------------------------------------------------------
// kBias: the score of an edge is scale * q . (k[other] + rel[edge]), rel an (n_edges, D) tensor shared by the
// heads - the node_mul_edge term (graphop_kernel.cu:16-34, "relative positional encoding") folded into the scores.
template <typename T, int V, int R, bool kBias = false>
struct AttnFwdOp {
  using A = typename AccOf<T>::type;
  static constexpr const char* kName = kBias ? "attention_bias_fwd" : "attention_fwd";
  const T* __restrict__ rel = nullptr;   // (n_edges, D), kBias only
  static constexpr bool kRowOut = true;
  static constexpr int kUnroll = (R * V * (int)sizeof(A) <= 16) ? 4 : 2;
  const T* __restrict__ q;   // (n_dst, H, D)
  const T* __restrict__ k;   // (n_src, H, D)
  const T* __restrict__ v;   // (n_src, H, D)
  T* __restrict__ o;         // (n_dst, H, D)
  A* __restrict__ lse;       // (n_dst, H)
  A* __restrict__ carry;     // (2 * n_tiles, cstride) partials written by this level
  const A* carry_in;         // partials of the level below (carry levels only)
  A scale;
  int H, D, HD, S, lph;
  long long cstride;         // HD + 2 * S elements per carry slot

  struct State { SlotMap<R> sm; A q[R][V]; A acc[R][V]; A m[R]; A l[R]; };
  struct Fetched { A k[R][V]; A v[R][V]; };
  struct CarryIn { A acc[R][V]; A m[R]; A l[R]; };

  __device__ __forceinline__ void setup(State& st, int lane) const { st.sm.init(lane, S, V, D, 0); }
  __device__ __forceinline__ void begin(State& st, int node, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.m[i] = neg_inf<A>();
      st.l[i] = A(0);
#pragma unroll
      for (int e = 0; e < V; ++e) { st.acc[i][e] = A(0); st.q[i][e] = A(0); }
      if (st.sm.ok[i]) load_acc<T, V>(st.q[i], q + (long long)node * HD + st.sm.feat[i]);
    }
  }
  __device__ __forceinline__ void fetch(const State& st, Fetched& f, int c, int edge, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (st.sm.ok[i]) {
        load_acc<T, V>(f.k[i], k + (long long)c * HD + st.sm.feat[i]);
        load_acc<T, V>(f.v[i], v + (long long)c * HD + st.sm.feat[i]);
        if constexpr (kBias) {
          A b[V];
          load_acc<T, V>(b, rel + (long long)edge * D + st.sm.efeat[i]);
#pragma unroll
          for (int e = 0; e < V; ++e) f.k[i][e] += b[e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) { f.k[i][e] = A(0); f.v[i][e] = A(0); }
      }
    }
  }
  __device__ __forceinline__ void consume(State& st, const Fetched& f, int) const {
    A s[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      s[i] = A(0);
#pragma unroll
      for (int e = 0; e < V; ++e) s[i] += st.q[i][e] * f.k[i][e];
    }
    reduce_heads<A, R>(s, lph);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const A sc = s[i] * scale;
      const A mn = sc > st.m[i] ? sc : st.m[i];
      const A corr = gk_exp(st.m[i] - mn);
      const A p = gk_exp(sc - mn);
      st.l[i] = st.l[i] * corr + p;
#pragma unroll
      for (int e = 0; e < V; ++e) st.acc[i][e] = st.acc[i][e] * corr + p * f.v[i][e];
      st.m[i] = mn;
    }
  }
  __device__ __forceinline__ void store_row(const State& st, int node, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (st.sm.ok[i]) {
        const A inv = A(1) / st.l[i];
        A out[V];
#pragma unroll
        for (int e = 0; e < V; ++e) out[e] = st.acc[i][e] * inv;
        store_acc<T, V>(o + (long long)node * HD + st.sm.feat[i], out);
        if (st.sm.efeat[i] == 0) lse[(long long)node * H + st.sm.head[i]] = st.m[i] + gk_log(st.l[i]);
      }
    }
  }
  __device__ __forceinline__ void store_carry(const State& st, long long slot, int lane) const {
    A* c = carry + slot * cstride;
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        store_raw<A, V>(c + st.sm.feat[i], st.acc[i]);
        c[HD + lane + 32 * i] = st.m[i];
        c[HD + S + lane + 32 * i] = st.l[i];
      }
  }
  __device__ __forceinline__ void store_identity(const State& st, long long slot, int lane) const {
    A* c = carry + slot * cstride;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        store_raw<A, V>(c + st.sm.feat[i], z);
        c[HD + lane + 32 * i] = neg_inf<A>();
        c[HD + S + lane + 32 * i] = A(0);
      }
  }
  __device__ __forceinline__ void begin_merge(State& st, int, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.m[i] = neg_inf<A>();
      st.l[i] = A(0);
#pragma unroll
      for (int e = 0; e < V; ++e) st.acc[i][e] = A(0);
    }
  }
  __device__ __forceinline__ void fetch_carry(const State& st, CarryIn& ci, long long slot, int lane) const {
    const A* c = carry_in + slot * cstride;
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        load_raw<A, V>(ci.acc[i], c + st.sm.feat[i]);
        ci.m[i] = c[HD + lane + 32 * i];
        ci.l[i] = c[HD + S + lane + 32 * i];
      }
  }
  __device__ __forceinline__ void merge_carry(State& st, const CarryIn& ci, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        const A mc = ci.m[i];
        const A mn = mc > st.m[i] ? mc : st.m[i];
        // a neutral partial has m = -inf: its weight is zero, never exp(-inf - -inf)
        const A wa = st.m[i] == neg_inf<A>() ? A(0) : gk_exp(st.m[i] - mn);
        const A wb = mc == neg_inf<A>() ? A(0) : gk_exp(mc - mn);
        st.l[i] = st.l[i] * wa + ci.l[i] * wb;
#pragma unroll
        for (int e = 0; e < V; ++e) st.acc[i][e] = st.acc[i][e] * wa + ci.acc[i][e] * wb;
        st.m[i] = mn;
      }
  }
  __device__ __forceinline__ void zero_rows(long long lo, long long hi, int lane) const {
    if (hi <= lo) return;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    const long long n = (hi - lo) * S;
    for (long long kk = lane; kk < n; kk += 32) store_acc<T, V>(o + lo * HD + kk * V, z);
    const long long nl = (hi - lo) * H;
    for (long long kk = lane; kk < nl; kk += 32) lse[lo * H + kk] = neg_inf<A>();
  }
};

// ---------------------------------------------------------------------------------------
// Fused attention backward, destination side:  for every node, with dO, O and lse given,
//     delta = dO . O (per head),  p_k = exp(scale * q.k_k - lse),
//     ds_k = p_k * (dO . v_k - delta) * scale,     dq[node] = sum_k ds_k * k_k
// which is sparse_softmax backward (graphop_kernel.cu:214-228) composed with the dA half of
// maskedmm backward (:105-110), probabilities recomputed instead of stored.  delta is also
// written out for the source-side pass.
// (lse, delta) of one (destination node, head), written side by side by the destination pass so that the
// source pass fetches both with one load.  Rows hold `stat_heads(H)` pairs: H rounded up so that a row is
// a whole number of 16-byte pieces.
template <typename A> struct alignas(2 * sizeof(A)) StatPair { A lse, delta; };
// (p, ds) of one (edge, head): the probability and the score gradient the destination pass computed, kept
// for the source pass when the caller gives the transposed CSR's edge ids.  Rows hold stat_heads(H) pairs.
template <typename A> struct alignas(2 * sizeof(A)) EdgePair { A p, ds; };
__host__ __device__ constexpr int stat_heads(int H, int acc_bytes) { return acc_bytes >= 8 ? H : ((H + 1) & ~1); }

// ---------------------------------------------------------------------------------------
// kBias: scores with the edge term (see AttnFwdOp); dq then sums ds * (k + rel), and (p, ds) of every edge
// are left in `pairs` for the source pass and for the gradient of rel.
template <typename T, int V, int R, bool kBias = false>
struct AttnBwdDstOp {
  using A = typename AccOf<T>::type;
  static constexpr const char* kName = kBias ? "attention_bias_bwd_dst" : "attention_bwd_dst";
  const T* __restrict__ rel = nullptr;          // (n_edges, D), kBias only
  EdgePair<A>* __restrict__ pairs = nullptr;    // (n_edges, Hp) out, kBias only
  static constexpr bool kRowOut = true;
  static constexpr int kUnroll = (R * V * (int)sizeof(A) <= 16) ? 4 : 2;
  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const T* __restrict__ o;
  const T* __restrict__ dout;
  const A* __restrict__ lse;
  StatPair<A>* __restrict__ stat;  // (n_dst, Hp) out: lse copied, delta computed; Hp = stat_heads(H)
  T* __restrict__ dq;        // (n_dst, H, D) out
  A* __restrict__ carry;     // (2 * n_tiles, HD) partials written by this level
  const A* carry_in;         // partials of the level below (carry levels only)
  A scale;
  int H, Hp, D, HD, S, lph;

  struct State { SlotMap<R> sm; A q[R][V]; A g[R][V]; A acc[R][V]; A lse[R]; A delta[R]; };
  struct Fetched { A k[R][V]; A v[R][V]; int edge; };
  struct CarryIn { A x[R][V]; };

  __device__ __forceinline__ void setup(State& st, int lane) const { st.sm.init(lane, S, V, D, 0); }
  __device__ __forceinline__ void begin(State& st, int node, int lane) const { begin_ordered<0>(st, node, lane); }
  // kAscLph > 0: that many lanes per head (a head inside one of the lane's slots), delta summed in the ascending butterfly order
  // (the order in which the staged fast path sums dO . v)
  template <int kAscLph>
  __device__ __forceinline__ void begin_ordered(State& st, int node, int) const {
    A dl[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      dl[i] = A(0);
      st.lse[i] = A(0);
#pragma unroll
      for (int e = 0; e < V; ++e) { st.acc[i][e] = A(0); st.q[i][e] = A(0); st.g[i][e] = A(0); }
      if (st.sm.ok[i]) {
        const long long off = (long long)node * HD + st.sm.feat[i];
        A ov[V];
        load_acc<T, V>(st.q[i], q + off);
        load_acc<T, V>(st.g[i], dout + off);
        load_acc<T, V>(ov, o + off);
#pragma unroll
        for (int e = 0; e < V; ++e) dl[i] += st.g[i][e] * ov[e];
        st.lse[i] = __ldg(lse + (long long)node * H + st.sm.head[i]);
      }
    }
    if constexpr (kAscLph > 0) {
#pragma unroll
      for (int i = 0; i < R; ++i) dl[i] = reduce_ascending<kAscLph, A>(dl[i]);
    } else {
      reduce_heads<A, R>(dl, lph);
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.delta[i] = dl[i];
      if (st.sm.ok[i] && st.sm.efeat[i] == 0) stat[(long long)node * Hp + st.sm.head[i]] = StatPair<A>{st.lse[i], dl[i]};
    }
  }
  __device__ __forceinline__ void fetch(const State& st, Fetched& f, int c, int edge, int) const {
    f.edge = edge;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (st.sm.ok[i]) {
        load_acc<T, V>(f.k[i], k + (long long)c * HD + st.sm.feat[i]);
        load_acc<T, V>(f.v[i], v + (long long)c * HD + st.sm.feat[i]);
        if constexpr (kBias) {
          A b[V];
          load_acc<T, V>(b, rel + (long long)edge * D + st.sm.efeat[i]);
#pragma unroll
          for (int e = 0; e < V; ++e) f.k[i][e] += b[e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) { f.k[i][e] = A(0); f.v[i][e] = A(0); }
      }
    }
  }
  __device__ __forceinline__ void consume(State& st, const Fetched& f, int) const {
    A s[R], dp[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      s[i] = A(0);
      dp[i] = A(0);
#pragma unroll
      for (int e = 0; e < V; ++e) { s[i] += st.q[i][e] * f.k[i][e]; dp[i] += st.g[i][e] * f.v[i][e]; }
    }
    reduce_heads<A, R>(s, lph);
    reduce_heads<A, R>(dp, lph);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const A p = gk_exp(s[i] * scale - st.lse[i]);
      const A ds = p * (dp[i] - st.delta[i]) * scale;
#pragma unroll
      for (int e = 0; e < V; ++e) st.acc[i][e] += ds * f.k[i][e];
      if constexpr (kBias) {
        if (st.sm.ok[i] && st.sm.efeat[i] == 0) pairs[(long long)f.edge * Hp + st.sm.head[i]] = EdgePair<A>{p, ds};
      }
    }
  }
  __device__ __forceinline__ void store_row(const State& st, int node, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) store_acc<T, V>(dq + (long long)node * HD + st.sm.feat[i], st.acc[i]);
  }
  __device__ __forceinline__ void store_carry(const State& st, long long slot, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) store_raw<A, V>(carry + slot * HD + st.sm.feat[i], st.acc[i]);
  }
  __device__ __forceinline__ void store_identity(const State& st, long long slot, int) const {
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) store_raw<A, V>(carry + slot * HD + st.sm.feat[i], z);
  }
  __device__ __forceinline__ void begin_merge(State& st, int, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int e = 0; e < V; ++e) st.acc[i][e] = A(0);
  }
  __device__ __forceinline__ void fetch_carry(const State& st, CarryIn& c, long long slot, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) load_raw<A, V>(c.x[i], carry_in + slot * HD + st.sm.feat[i]);
  }
  __device__ __forceinline__ void merge_carry(State& st, const CarryIn& c, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
#pragma unroll
        for (int e = 0; e < V; ++e) st.acc[i][e] += c.x[i][e];
      }
  }
  __device__ __forceinline__ void zero_rows(long long lo, long long hi, int lane) const {
    if (hi <= lo) return;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    const long long n = (hi - lo) * S;
    for (long long kk = lane; kk < n; kk += 32) store_acc<T, V>(dq + lo * HD + kk * V, z);
    const long long nl = (hi - lo) * Hp;
    for (long long kk = lane; kk < nl; kk += 32) stat[lo * Hp + kk] = StatPair<A>{A(0), A(0)};
  }
};

// ---------------------------------------------------------------------------------------
// Fused attention backward, source side, over the transposed CSR: for every source node c
//     dv[c] = sum_k p_k * dO[dst_k],     dk[c] = sum_k ds_k * q[dst_k]
// with p_k and ds_k recomputed from q[dst_k], dO[dst_k], lse[dst_k] and delta[dst_k]: the dx
// half of vector_spmm backward (graphop_kernel.cu:156-161) and the dB half of maskedmm
// backward (:105-110 over the column CSR) in one pass.
// ---------------------------------------------------------------------------------------
template <typename T, int V, int R>
struct AttnBwdSrcOp {
  using A = typename AccOf<T>::type;
  static constexpr const char* kName = "attention_bwd_src";
  static constexpr bool kRowOut = true;
  static constexpr int kUnroll = (R * V * (int)sizeof(A) <= 16) ? 4 : 2;
  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const T* __restrict__ dout;
  const StatPair<A>* __restrict__ stat;  // (n_dst, Hp) from the destination pass
  T* __restrict__ dk;
  T* __restrict__ dv;
  A* __restrict__ carry;     // (2 * n_tiles, 2 * HD): dk partial then dv partial, written by this level
  const A* carry_in;         // partials of the level below (carry levels only)
  A scale;
  int H, Hp, D, HD, S, lph;

  struct State { SlotMap<R> sm; A k[R][V]; A v[R][V]; A ak[R][V]; A av[R][V]; };
  struct Fetched { A q[R][V]; A g[R][V]; A lse[R]; A delta[R]; };
  struct CarryIn { A k[R][V]; A v[R][V]; };

  __device__ __forceinline__ void setup(State& st, int lane) const { st.sm.init(lane, S, V, D, 0); }
  __device__ __forceinline__ void begin(State& st, int node, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
#pragma unroll
      for (int e = 0; e < V; ++e) { st.ak[i][e] = A(0); st.av[i][e] = A(0); st.k[i][e] = A(0); st.v[i][e] = A(0); }
      if (st.sm.ok[i]) {
        load_acc<T, V>(st.k[i], k + (long long)node * HD + st.sm.feat[i]);
        load_acc<T, V>(st.v[i], v + (long long)node * HD + st.sm.feat[i]);
      }
    }
  }
  __device__ __forceinline__ void fetch(const State& st, Fetched& f, int c, int, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (st.sm.ok[i]) {
        load_acc<T, V>(f.q[i], q + (long long)c * HD + st.sm.feat[i]);
        load_acc<T, V>(f.g[i], dout + (long long)c * HD + st.sm.feat[i]);
        const StatPair<A> pr = stat[(long long)c * Hp + st.sm.head[i]];
        f.lse[i] = pr.lse;
        f.delta[i] = pr.delta;
      } else {
        f.lse[i] = A(0);
        f.delta[i] = A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) { f.q[i][e] = A(0); f.g[i][e] = A(0); }
      }
    }
  }
  __device__ __forceinline__ void consume(State& st, const Fetched& f, int) const {
    A s[R], dp[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
      s[i] = A(0);
      dp[i] = A(0);
#pragma unroll
      for (int e = 0; e < V; ++e) { s[i] += f.q[i][e] * st.k[i][e]; dp[i] += f.g[i][e] * st.v[i][e]; }
    }
    reduce_heads<A, R>(s, lph);
    reduce_heads<A, R>(dp, lph);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const A p = gk_exp(s[i] * scale - f.lse[i]);
      const A ds = p * (dp[i] - f.delta[i]) * scale;
#pragma unroll
      for (int e = 0; e < V; ++e) { st.av[i][e] += p * f.g[i][e]; st.ak[i][e] += ds * f.q[i][e]; }
    }
  }
  __device__ __forceinline__ void store_row(const State& st, int node, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        store_acc<T, V>(dk + (long long)node * HD + st.sm.feat[i], st.ak[i]);
        store_acc<T, V>(dv + (long long)node * HD + st.sm.feat[i], st.av[i]);
      }
  }
  __device__ __forceinline__ void store_carry(const State& st, long long slot, int) const {
    A* c = carry + slot * 2 * HD;
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        store_raw<A, V>(c + st.sm.feat[i], st.ak[i]);
        store_raw<A, V>(c + HD + st.sm.feat[i], st.av[i]);
      }
  }
  __device__ __forceinline__ void store_identity(const State& st, long long slot, int) const {
    A* c = carry + slot * 2 * HD;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        store_raw<A, V>(c + st.sm.feat[i], z);
        store_raw<A, V>(c + HD + st.sm.feat[i], z);
      }
  }
  __device__ __forceinline__ void begin_merge(State& st, int, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int e = 0; e < V; ++e) { st.ak[i][e] = A(0); st.av[i][e] = A(0); }
  }
  __device__ __forceinline__ void fetch_carry(const State& st, CarryIn& ci, long long slot, int) const {
    const A* c = carry_in + slot * 2 * HD;
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        load_raw<A, V>(ci.k[i], c + st.sm.feat[i]);
        load_raw<A, V>(ci.v[i], c + HD + st.sm.feat[i]);
      }
  }
  __device__ __forceinline__ void merge_carry(State& st, const CarryIn& ci, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
#pragma unroll
        for (int e = 0; e < V; ++e) { st.ak[i][e] += ci.k[i][e]; st.av[i][e] += ci.v[i][e]; }
      }
  }
  __device__ __forceinline__ void zero_rows(long long lo, long long hi, int lane) const {
    if (hi <= lo) return;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    const long long n = (hi - lo) * S;
    for (long long kk = lane; kk < n; kk += 32) {
      store_acc<T, V>(dk + lo * HD + kk * V, z);
      store_acc<T, V>(dv + lo * HD + kk * V, z);
    }
  }
};

// Gradient of the edge term of the biased attention:  d_rel[j, :] = sum_h ds[j, h] * q[node(j), h, :]
// (the dB half of node_mul_edge backward, graphop_kernel.cu:79-93, with the score gradients the destination
// pass left in `pairs`).  One thread per (position, slot of V features); consecutive threads cover a position's
// features, consecutive positions of a node re-read its q row from L1 / L2; positions no chunk covers get 0.
// shift = log2(D / V) when that is a power of two, else -1.
template <typename T, int V>
__global__ void __launch_bounds__(256)
bias_grad_kernel(const int32_t* __restrict__ erow, const EdgePair<typename AccOf<T>::type>* __restrict__ pairs,
                 const T* __restrict__ q, T* __restrict__ d_rel, long long E, int H, int Hp, int D, int shift) {
  using A = typename AccOf<T>::type;
  const int slots = D / V;
  const long long stride = (long long)gridDim.x * blockDim.x, total = E * slots;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long j = shift >= 0 ? (i >> shift) : i / slots;
    const int d = (int)(i - j * slots) * V;
    const int r = __ldg(erow + j);
    A sum[V];
#pragma unroll
    for (int e = 0; e < V; ++e) sum[e] = A(0);
    if (r >= 0) {
      const T* qrow = q + (long long)r * H * D + d;
      const EdgePair<A>* pr = pairs + j * Hp;
      for (int h = 0; h < H; ++h) {
        const A ds = pr[h].ds;
        A qv[V];
        load_acc<T, V>(qv, qrow + (long long)h * D);
#pragma unroll
        for (int e = 0; e < V; ++e) sum[e] += ds * qv[e];
      }
    }
    store_acc<T, V>(d_rel + j * D + d, sum);
  }
}

}  // namespace gk
