// Fused attention kernels for node rows of exactly 512 bytes (32 vector slots, one per lane:
// 4 heads x 32 fp32, 2 x 64, 1 x 128, or the bf16 shapes of the same byte size), driven by
// walk_staged_kernel.  Two lane mappings alternate inside a batch of four edges:
//
//   dot mapping    lane = (head, part, u): the lane multiplies slots (lane & ~3) .. +3 of the
//                  node-resident row, kept in registers, with the same slots of edge u = lane & 3
//                  read from the shared-memory ring, and the partial dot products of one head meet
//                  with log2(LPH / 4) shuffles.  Every (edge, head) score therefore exists once
//                  per batch, and one ex2 per lane turns it into a probability.
//   slot mapping   lane = slot: the lane owns 16 bytes of the output row and accumulates the four
//                  edges' contributions, fetching each edge's scalar (probability or score
//                  gradient) from the dot-mapping lane that holds it with one shuffle.
//
// Both mappings keep the LPH lanes of a head together, so per-head running values (maximum, sum,
// lse, delta) are simply held by every lane of the head.  Edges past the end of the node in a
// short batch are masked to probability 0; their ring entries hold some other edge's rows, which
// are finite numbers.  Ring entries are padded so that consecutive entries start 16 bytes apart
// modulo 128: the four edges a quarter-warp reads in the dot mapping hit different banks.
//
// Partial results of nodes that span tiles use the carry-slot format of the generic ops
// (AttnFwdOp etc. in gk_ops.cuh), so the carry levels run unchanged.
#pragma once
#include "gk_staged.cuh"

namespace gk {

#ifndef GK_TUNE_CTAS3
#define GK_TUNE_CTAS3 5   // blocks of 4 warps per SM aimed at
#endif
#ifndef GK_TUNE_DEPTH3
#define GK_TUNE_DEPTH3 8  // ring entries per warp
#endif

template <typename T, int V, int LPH>
struct Attn3Base {
  using A = typename AccOf<T>::type;
  static_assert(sizeof(T) * V == 16 && sizeof(A) == 4, "512-byte rows of 16-byte slots, fp32 accumulation");
  static_assert(LPH == 8 || LPH == 16 || LPH == 32, "lanes per head");
  static constexpr int H = 32 / LPH;
  static constexpr int HD = 32 * V;
  static constexpr bool kRowOut = true;
  static constexpr bool kUsesEid = false;
  static constexpr int kBatch = 4, kDepth = GK_TUNE_DEPTH3, kWarps = 4, kMinCtas = GK_TUNE_CTAS3;
  static constexpr int kUnroll = 1;
  struct Fetched {};
  struct CarryIn {};

  __device__ static __forceinline__ const unsigned char* entry_of(const unsigned char* ring, int pos, int eb) {
    return ring + (size_t)(pos & (kDepth - 1)) * eb;
  }
  // sum over the lanes of one head that hold different parts of the dot product
  __device__ static __forceinline__ A sum_parts(A v) {
#pragma unroll
    for (int o = 4; o < LPH; o <<= 1) v += __shfl_xor_sync(kFull, v, o);
    return v;
  }
  // sum over the four edges of a batch (lanes that differ in u)
  __device__ static __forceinline__ A sum_edges(A v) {
    v += __shfl_xor_sync(kFull, v, 1);
    v += __shfl_xor_sync(kFull, v, 2);
    return v;
  }
  // value of edge uu held by the dot-mapping lanes of this lane's head
  __device__ static __forceinline__ A from_edge(A v, int uu, int lane) {
    return __shfl_sync(kFull, v, (lane & ~(LPH - 1)) + uu);
  }
  // the four slots of a node row this lane multiplies in the dot mapping
  __device__ static __forceinline__ void load_dot_slots(A (&dst)[4][V], const T* row, int lane) {
#pragma unroll
    for (int c = 0; c < 4; ++c) load_acc<T, V>(dst[c], row + ((lane & ~3) + c) * V);
  }
  __device__ static __forceinline__ A dot_slots(const A (&a)[4][V], const unsigned char* row_in_ring, int lane) {
    A s = A(0);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      A b[V];
      lds_acc<T, V>(b, row_in_ring + ((lane & ~3) + c) * 16);
#pragma unroll
      for (int e = 0; e < V; ++e) s += a[c][e] * b[e];
    }
    return s;
  }
};

// ---------------------------------------------------------------------------------------
// forward: ring entry = [k row 512][v row 512][16 pad]
// ---------------------------------------------------------------------------------------
template <typename T, int V, int LPH>
struct AttnFwd3 : Attn3Base<T, V, LPH> {
  using B = Attn3Base<T, V, LPH>;
  using A = typename B::A;
  static constexpr const char* kName = "attention_fwd";
  static constexpr int kEdgeBytes = 1040;
  static constexpr int H = B::H, HD = B::HD;
  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  T* __restrict__ o;
  A* __restrict__ lse;
  A* __restrict__ carry;   // (2 * n_tiles, cstride), format of AttnFwdOp: [acc HD][m 32][l 32]
  A scale;
  long long cstride;

  struct State { A q[4][V]; A acc[V]; A m, l; };

  __device__ __forceinline__ void setup(State&, int) const {}
  __device__ __forceinline__ void begin(State& st, int node, int lane) const {
    B::load_dot_slots(st.q, q + (long long)node * HD, lane);
    const A c = scale * A(kLog2e);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc)
#pragma unroll
      for (int e = 0; e < V; ++e) st.q[cc][e] *= c;
#pragma unroll
    for (int e = 0; e < V; ++e) st.acc[e] = A(0);
    st.m = neg_inf<A>();
    st.l = A(0);
  }
  __device__ __forceinline__ void stage(const State&, unsigned char* entry, int c, int, int lane) const {
    cp_async16(entry + lane * 16, k + (long long)c * HD + lane * V);
    cp_async16(entry + 512 + lane * 16, v + (long long)c * HD + lane * V);
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt, const int*,
                                                int lane) const {
    const int u = lane & 3;
    A s = B::sum_parts(B::dot_slots(st.q, B::entry_of(ring, i0 + u, kEdgeBytes), lane));
    if (!kFullBatch && u >= cnt) s = neg_inf<A>();
    A bm = s;
    bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, 1));
    bm = fmaxf(bm, __shfl_xor_sync(kFull, bm, 2));
    const A mn = fmaxf(st.m, bm);
    const A corr = gk_exp2(st.m - mn);  // first batch of a node: 2^-inf = 0
    const A p = gk_exp2(s - mn);
    st.l = st.l * corr + p;             // this lane's edges only; summed over u when the node ends
    st.m = mn;
#pragma unroll
    for (int e = 0; e < V; ++e) st.acc[e] *= corr;
#pragma unroll
    for (int uu = 0; uu < 4; ++uu) {
      const A pu = B::from_edge(p, uu, lane);
      A vv[V];
      lds_acc<T, V>(vv, B::entry_of(ring, i0 + uu, kEdgeBytes) + 512 + lane * 16);
#pragma unroll
      for (int e = 0; e < V; ++e) st.acc[e] += pu * vv[e];
    }
  }
  __device__ __forceinline__ void store_row(const State& st, int node, int lane) const {
    const A l = B::sum_edges(st.l);
    const A inv = A(1) / l;
    A out[V];
#pragma unroll
    for (int e = 0; e < V; ++e) out[e] = st.acc[e] * inv;
    store_acc<T, V>(o + (long long)node * HD + lane * V, out);
    if ((lane & (LPH - 1)) == 0) lse[(long long)node * H + lane / LPH] = (st.m + gk_log2(l)) * A(kLn2);
  }
  __device__ __forceinline__ void store_carry(const State& st, long long slot, int lane) const {
    A* c = carry + slot * cstride;
    store_raw<A, V>(c + lane * V, st.acc);
    c[HD + lane] = st.m;
    c[HD + 32 + lane] = B::sum_edges(st.l);
  }
  __device__ __forceinline__ void store_identity(const State&, long long slot, int lane) const {
    A* c = carry + slot * cstride;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    store_raw<A, V>(c + lane * V, z);
    c[HD + lane] = neg_inf<A>();
    c[HD + 32 + lane] = A(0);
  }
  __device__ __forceinline__ void zero_rows(long long lo, long long hi, int lane) const {
    if (hi <= lo) return;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    for (long long kk = lane; kk < (hi - lo) * 32; kk += 32) store_acc<T, V>(o + lo * HD + kk * V, z);
    for (long long kk = lane; kk < (hi - lo) * H; kk += 32) lse[lo * H + kk] = neg_inf<A>();
  }
};

// ---------------------------------------------------------------------------------------
// backward, destination side: ring entry = [k row 512][v row 512][16 pad]
// ---------------------------------------------------------------------------------------
template <typename T, int V, int LPH>
struct AttnBwdDst3 : Attn3Base<T, V, LPH> {
  using B = Attn3Base<T, V, LPH>;
  using A = typename B::A;
  static constexpr const char* kName = "attention_bwd_dst";
  static constexpr int kEdgeBytes = 1040;
  static constexpr int H = B::H, HD = B::HD;
  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const T* __restrict__ o;
  const T* __restrict__ dout;
  const A* __restrict__ lse;
  A* __restrict__ delta;
  T* __restrict__ dq;
  A* __restrict__ carry;   // (2 * n_tiles, HD)
  A scale;

  struct State { A q[4][V]; A g[4][V]; A acc[V]; A lse2, delta; };

  __device__ __forceinline__ void setup(State&, int) const {}
  __device__ __forceinline__ void begin(State& st, int node, int lane) const {
    const long long off = (long long)node * HD;
    A ov[4][V];
    B::load_dot_slots(st.q, q + off, lane);
    B::load_dot_slots(st.g, dout + off, lane);
    B::load_dot_slots(ov, o + off, lane);
    const A c = scale * A(kLog2e);
    A d = A(0);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc)
#pragma unroll
      for (int e = 0; e < V; ++e) { d += st.g[cc][e] * ov[cc][e]; st.q[cc][e] *= c; }
    st.delta = B::sum_parts(d);
    st.lse2 = __ldg(lse + (long long)node * H + lane / LPH) * A(kLog2e);
    if ((lane & (LPH - 1)) == 0) delta[(long long)node * H + lane / LPH] = st.delta;
#pragma unroll
    for (int e = 0; e < V; ++e) st.acc[e] = A(0);
  }
  __device__ __forceinline__ void stage(const State&, unsigned char* entry, int c, int, int lane) const {
    cp_async16(entry + lane * 16, k + (long long)c * HD + lane * V);
    cp_async16(entry + 512 + lane * 16, v + (long long)c * HD + lane * V);
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt, const int*,
                                                int lane) const {
    const int u = lane & 3;
    const unsigned char* mine = B::entry_of(ring, i0 + u, kEdgeBytes);
    const A s = B::sum_parts(B::dot_slots(st.q, mine, lane));
    const A dp = B::sum_parts(B::dot_slots(st.g, mine + 512, lane));
    A ds = gk_exp2(s - st.lse2) * (dp - st.delta) * scale;
    if (!kFullBatch && u >= cnt) ds = A(0);
#pragma unroll
    for (int uu = 0; uu < 4; ++uu) {
      const A du = B::from_edge(ds, uu, lane);
      A kv[V];
      lds_acc<T, V>(kv, B::entry_of(ring, i0 + uu, kEdgeBytes) + lane * 16);
#pragma unroll
      for (int e = 0; e < V; ++e) st.acc[e] += du * kv[e];
    }
  }
  __device__ __forceinline__ void store_row(const State& st, int node, int lane) const {
    store_acc<T, V>(dq + (long long)node * HD + lane * V, st.acc);
  }
  __device__ __forceinline__ void store_carry(const State& st, long long slot, int lane) const {
    store_raw<A, V>(carry + slot * HD + lane * V, st.acc);
  }
  __device__ __forceinline__ void store_identity(const State&, long long slot, int lane) const {
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    store_raw<A, V>(carry + slot * HD + lane * V, z);
  }
  __device__ __forceinline__ void zero_rows(long long lo, long long hi, int lane) const {
    if (hi <= lo) return;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    for (long long kk = lane; kk < (hi - lo) * 32; kk += 32) store_acc<T, V>(dq + lo * HD + kk * V, z);
    for (long long kk = lane; kk < (hi - lo) * H; kk += 32) delta[lo * H + kk] = A(0);
  }
};

// ---------------------------------------------------------------------------------------
// backward, source side, over the transposed CSR:
// ring entry = [q row of the destination 512][dO row 512][lse H][delta H][pad to 1072]
// ---------------------------------------------------------------------------------------
template <typename T, int V, int LPH>
struct AttnBwdSrc3 : Attn3Base<T, V, LPH> {
  using B = Attn3Base<T, V, LPH>;
  using A = typename B::A;
  static constexpr const char* kName = "attention_bwd_src";
  static constexpr int kEdgeBytes = 1072;  // 67 * 16: consecutive entries 48 bytes apart modulo 128
  static constexpr int H = B::H, HD = B::HD;
  const T* __restrict__ q;
  const T* __restrict__ k;
  const T* __restrict__ v;
  const T* __restrict__ dout;
  const A* __restrict__ lse;
  const A* __restrict__ delta;
  T* __restrict__ dk;
  T* __restrict__ dv;
  A* __restrict__ carry;   // (2 * n_tiles, 2 * HD)
  A scale;

  struct State { A k[4][V]; A v[4][V]; A ak[V]; A av[V]; };

  __device__ __forceinline__ void setup(State&, int) const {}
  __device__ __forceinline__ void begin(State& st, int node, int lane) const {
    const long long off = (long long)node * HD;
    B::load_dot_slots(st.k, k + off, lane);
    B::load_dot_slots(st.v, v + off, lane);
    const A c = scale * A(kLog2e);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc)
#pragma unroll
      for (int e = 0; e < V; ++e) st.k[cc][e] *= c;
#pragma unroll
    for (int e = 0; e < V; ++e) { st.ak[e] = A(0); st.av[e] = A(0); }
  }
  __device__ __forceinline__ void stage(const State&, unsigned char* entry, int c, int, int lane) const {
    cp_async16(entry + lane * 16, q + (long long)c * HD + lane * V);
    cp_async16(entry + 512 + lane * 16, dout + (long long)c * HD + lane * V);
    // the destination's H log-sum-exps and H deltas: one small copy each, by lanes 0 and 1
    if (lane < 2) {
      const A* src = (lane == 0 ? lse : delta) + (long long)c * H;
      unsigned char* dst = entry + 1024 + lane * 16;
      if constexpr (H == 4) cp_async16(dst, src);
      else cp_async_small<H * 4>(dst, src);
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt, const int*,
                                                int lane) const {
    const int u = lane & 3;
    const unsigned char* mine = B::entry_of(ring, i0 + u, kEdgeBytes);
    const A s = B::sum_parts(B::dot_slots(st.k, mine, lane));
    const A dp = B::sum_parts(B::dot_slots(st.v, mine + 512, lane));
    const A* sc = reinterpret_cast<const A*>(mine + 1024);
    A p = gk_exp2(s - sc[lane / LPH] * A(kLog2e));
    A ds = p * (dp - sc[4 + lane / LPH]) * scale;
    if (!kFullBatch && u >= cnt) { p = A(0); ds = A(0); }
#pragma unroll
    for (int uu = 0; uu < 4; ++uu) {
      const A pu = B::from_edge(p, uu, lane);
      const A du = B::from_edge(ds, uu, lane);
      const unsigned char* e_uu = B::entry_of(ring, i0 + uu, kEdgeBytes);
      A qv[V], gv[V];
      lds_acc<T, V>(qv, e_uu + lane * 16);
      lds_acc<T, V>(gv, e_uu + 512 + lane * 16);
#pragma unroll
      for (int e = 0; e < V; ++e) { st.av[e] += pu * gv[e]; st.ak[e] += du * qv[e]; }
    }
  }
  __device__ __forceinline__ void store_row(const State& st, int node, int lane) const {
    store_acc<T, V>(dk + (long long)node * HD + lane * V, st.ak);
    store_acc<T, V>(dv + (long long)node * HD + lane * V, st.av);
  }
  __device__ __forceinline__ void store_carry(const State& st, long long slot, int lane) const {
    A* c = carry + slot * 2 * HD;
    store_raw<A, V>(c + lane * V, st.ak);
    store_raw<A, V>(c + HD + lane * V, st.av);
  }
  __device__ __forceinline__ void store_identity(const State&, long long slot, int lane) const {
    A* c = carry + slot * 2 * HD;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    store_raw<A, V>(c + lane * V, z);
    store_raw<A, V>(c + HD + lane * V, z);
  }
  __device__ __forceinline__ void zero_rows(long long lo, long long hi, int lane) const {
    if (hi <= lo) return;
    A z[V];
#pragma unroll
    for (int e = 0; e < V; ++e) z[e] = A(0);
    for (long long kk = lane; kk < (hi - lo) * 32; kk += 32) {
      store_acc<T, V>(dk + lo * HD + kk * V, z);
      store_acc<T, V>(dv + lo * HD + kk * V, z);
    }
  }
};

}  // namespace gk
