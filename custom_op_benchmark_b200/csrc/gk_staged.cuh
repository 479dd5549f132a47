// Level-0 walker with shared-memory staging, and the ops written for it.
//
// Same decomposition and the same carry / gap-fill rules as walk_kernel (gk_common.cuh); what
// changes is how the gathered rows reach the math:
//   * each warp owns a ring of kDepth edge entries in shared memory and keeps it full with
//     cp.async (16 bytes per lane per operand row, straight from global memory to shared
//     memory, no registers held while the load is in flight), so a warp has kDepth edges of
//     gathers outstanding at all times whatever its register budget;
//   * the tile's (node, other endpoint, edge id) triples are loaded once, coalesced, into
//     shared memory together with one byte per position that says how many of the following
//     positions belong to the same node;
//   * up to kBatch consecutive edges of one node are folded together, which gives the
//     scheduler kBatch independent dot-product / shuffle chains instead of one.
// A lane reads back the bytes it copied itself, so no barrier is needed between the asynchronous
// copies and their use beyond cp.async.wait_group (ops that share entry bytes between lanes say so
// and get a warp barrier, see SharesEntries).
#pragma once
#include <type_traits>

#include "gk_ops.cuh"

// Build-time tunables.
#ifndef GK_TUNE_CTAS_NARROW
#define GK_TUNE_CTAS_NARROW 4   // resident blocks per SM aimed at when a node row fits one slot per lane
#endif
#ifndef GK_TUNE_CTAS_SRC
#define GK_TUNE_CTAS_SRC 3      // the same for the attention backward over the transposed CSR: it keeps two
#endif                          // accumulator rows and two resident rows, which 64 registers do not hold
#ifndef GK_TUNE_TILE
#define GK_TUNE_TILE 256        // largest level-0 tile of the staged walker
#endif
#ifndef GK_TUNE_BATCH_MAX
#define GK_TUNE_BATCH_MAX 8     // most edges of one node folded together
#endif

namespace gk {

__device__ __forceinline__ void cp_async16(void* smem, const void* g) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(g) : "memory");
}
template <int BYTES>
__device__ __forceinline__ void cp_async_small(void* smem, const void* g) {
  static_assert(BYTES == 4 || BYTES == 8, "cp.async.ca moves 4, 8 or 16 bytes");
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2;\n" ::"r"(s), "l"(g), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Address of a lane's 16 bytes of row `c`: the lane's own base pointer (row 0, its slot) plus c rows.
// One 32 x 32 -> 64-bit multiply-add instead of a 64-bit index computation per copy.
__device__ __forceinline__ const unsigned char* row_ptr(const unsigned char* lane_base, int c, unsigned row_bytes) {
  return lane_base + (unsigned long long)(unsigned)c * row_bytes;
}

// 2^x.  float: the hardware approximation (relative error about 2^-22); double: exp2().
__device__ __forceinline__ float gk_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ double gk_exp2(double x) { return exp2(x); }
__device__ __forceinline__ float gk_log2(float x) { return log2f(x); }
__device__ __forceinline__ double gk_log2(double x) { return log2(x); }
constexpr double kLog2e = 1.4426950408889634074;
constexpr double kLn2 = 0.69314718055994530942;

// V elements of T from shared memory (16 bytes), widened to the accumulation type.
template <typename T, int V>
__device__ __forceinline__ void lds_acc(typename AccOf<T>::type (&dst)[V], const void* p) {
  static_assert(sizeof(T) * V == 16, "staged slots are 16 bytes");
  union { uint4 m; T t[V]; } u;
  u.m = *reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < V; ++i) dst[i] = to_acc<T>(u.t[i]);
}

// Staged op interface, on top of the walk_kernel interface (the carry levels of a staged op run
// through walk_kernel<Op, true>):
//   static constexpr int kBatch, kDepth, kEdgeBytes, kWarps (per block), kMinCtas (blocks per SM aimed at);
//   void stage(const State&, unsigned char* entry, int other, int edge, int lane)   cp.async the edge's operands
//   void prefetch_node(State&, int node, int lane)   start loading what begin(node) will need (may be a no-op)
//   template <bool kFullBatch>
//   void consume_batch(State&, const unsigned char* ring, int i, int cnt, const int* eids, int lane)
//        fold ring entries i .. i+cnt-1 (entry of position p at ring + (p & (kDepth-1)) * kEdgeBytes);
//        kFullBatch: cnt == kBatch, known at compile time
// Lanes whose slot does not exist (slot >= S) are not masked in stage / consume_batch: their slot map
// points at slot 0, so their copies and arithmetic are harmless duplicates, their node-resident
// operand is zero, and only stores test `ok`.
constexpr int kMetaPad = 32;  // metadata entries past the tile that the prefetcher may read

// Shared memory of one warp: metadata of tile + kMetaPad positions (node, other endpoint, edge id if
// the op uses it, one run-length byte), rounded to 16 bytes, then kDepth ring entries.
template <class Op>
__host__ __device__ constexpr size_t staged_warp_bytes(int tile) {
  return (((size_t)(tile + kMetaPad) * (Op::kUsesEid ? 13 : 9)) + 15) / 16 * 16 + (size_t)Op::kDepth * Op::kEdgeBytes;
}

// Ops whose lanes read ring bytes copied by other lanes declare `kSharedEntry = true`; the walker
// then puts a warp barrier between the copies' completion and the reads, and between the reads and
// the refill.  Every other op reads back only the bytes the same lane copied and needs neither.
template <class Op, class = void> struct SharesEntries : std::false_type {};
template <class Op> struct SharesEntries<Op, std::void_t<decltype(Op::kSharedEntry)>> : std::true_type {};

// Ops that need the global position of the edges they fold declare `kTileBase = true` and get the tile's
// first position in `State::tile_base` (positions stay below 2^31).
template <class Op, class = void> struct WantsTileBase : std::false_type {};
template <class Op> struct WantsTileBase<Op, std::void_t<decltype(Op::kTileBase)>> : std::true_type {};

template <class Op>
__global__ void __launch_bounds__(Op::kWarps * 32, Op::kMinCtas)
walk_staged_kernel(Op op, const PlanHeader* __restrict__ hdr, const int32_t* __restrict__ erow,
                   const int32_t* __restrict__ other, const int32_t* __restrict__ eid, long long E, int tile,
                   long long n_rows, int32_t* __restrict__ rows_next) {
  constexpr int U = Op::kBatch;
  constexpr int DEPTH = Op::kDepth;
  constexpr int EB = Op::kEdgeBytes;
  constexpr bool kOut = Op::kRowOut;
  constexpr bool kShared = SharesEntries<Op>::value;
  static_assert((DEPTH & (DEPTH - 1)) == 0 && DEPTH >= U && U <= 32, "ring depth: a power of two >= batch");
  extern __shared__ uint4 gk_smem[];
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  const long long t = (long long)blockIdx.x * Op::kWarps + w;
  const long long j0 = t * tile;
  if (j0 >= E) return;
  const int nt = (int)(j0 + tile < E ? tile : E - j0);
  const long long j1 = j0 + nt;

  if constexpr (kOut) {
    if (t == 0 && hdr->cover_hi <= hdr->cover_lo) {  // no covered position at all
      op.zero_rows(0, n_rows, lane);
      if (rows_next && lane == 0) { rows_next[0] = -1; rows_next[1] = -1; }
      return;
    }
  }

  // per warp: node and other-endpoint (and, for ops that use it, edge id) of tile + kMetaPad
  // positions, one byte of run length per position, then the ring
  const int cap = tile + kMetaPad;
  unsigned char* mine = reinterpret_cast<unsigned char*>(gk_smem) + (size_t)w * staged_warp_bytes<Op>(tile);
  int* m_row = reinterpret_cast<int*>(mine);
  int* m_oth = m_row + cap;
  int* m_eid = m_oth + cap;  // present only when Op::kUsesEid
  unsigned char* m_rem = reinterpret_cast<unsigned char*>(m_oth + (Op::kUsesEid ? 2 : 1) * cap);
  unsigned char* ring = mine + staged_warp_bytes<Op>(tile) - (size_t)DEPTH * EB;

  // Tile metadata -> shared memory.  m_rem[i] = number of consecutive positions from i on that have
  // the same node as i (at most 255, never past the tile): blocks of 32 are filled from the last to
  // the first so that a run that continues into the next block can add that block's first count.
  // Positions past the tile get node -2, and every position without a node points at node 0 / edge 0,
  // so that the prefetcher can issue its copies without looking at the node.
  const int before = j0 > 0 ? __ldg(erow + j0 - 1) : -1;
  {
    // all global loads of the tile's metadata are issued before any is used: one memory latency
    // per tile instead of one per 32 positions
    constexpr int kMaxBlocks = (GK_TUNE_TILE + kMetaPad) / 32;
    int r_[kMaxBlocks], o_[kMaxBlocks], e_[kMaxBlocks];
#pragma unroll
    for (int b = 0; b < kMaxBlocks; ++b) {
      const int i = b * 32 + lane;
      const bool inb = i < nt;
      r_[b] = inb ? __ldg(erow + j0 + i) : -2;
      o_[b] = (inb && other) ? __ldg(other + j0 + i) : 0;
      e_[b] = (Op::kUsesEid && inb) ? (eid ? __ldg(eid + j0 + i) : (int)(j0 + i)) : 0;
    }
    int next_first_row = -3, next_first_rem = 0;  // node and run length of the first position of block b + 1
#pragma unroll
    for (int b = kMaxBlocks - 1; b >= 0; --b) {
      const int i = b * 32 + lane;
      const int r = r_[b];
      if (i < cap) {
        m_row[i] = r;
        m_oth[i] = r >= 0 ? o_[b] : 0;
        if constexpr (Op::kUsesEid) m_eid[i] = r >= 0 ? e_[b] : 0;
      }
      int down = __shfl_down_sync(kFull, r, 1);
      if (lane == 31) down = next_first_row;
      const unsigned ends = __ballot_sync(kFull, r != down);   // bit l: the run ends at lane l
      const unsigned at_or_after = ends >> lane;                // bit 0 <-> this lane
      int rem;
      if (at_or_after) rem = __ffs(at_or_after);               // run ends inside this block
      else rem = (32 - lane) + next_first_rem;                  // runs on into block b + 1
      rem = rem > 255 ? 255 : rem;
      if (i < cap) m_rem[i] = (unsigned char)(i < nt ? rem : 1);
      next_first_row = __shfl_sync(kFull, r, 0);
      next_first_rem = __shfl_sync(kFull, rem, 0);
    }
  }
  __syncwarp();

  typename Op::State st;
  op.setup(st, lane);
  if constexpr (WantsTileBase<Op>::value) st.tile_base = (int)j0;
  const int first = m_row[0];
  const bool head_open = before >= 0 && before == first;
  bool first_seg = true;
  int cur = -1;
  int last_valid = before;
  int head_row = -1;

  // one commit group per position, copies issued whether or not the position carries an edge
  auto issue = [&](int i) {
    op.stage(st, ring + (size_t)(i & (DEPTH - 1)) * EB, m_oth[i], Op::kUsesEid ? m_eid[i] : 0, lane);
    cp_async_commit();
  };
#pragma unroll
  for (int i = 0; i < DEPTH; ++i) issue(i);

  bool new_seg = true;
  int i = 0;
  while (i < nt) {
    const int r = m_row[i];
    const int rem = m_rem[i];
    if (new_seg) {  // a segment starts here
      if (cur >= 0) {
        if constexpr (kOut) {
          if (first_seg && head_open) { op.store_carry(st, 2 * t, lane); head_row = cur; }
          else op.store_row(st, cur, lane);
          if (r < 0) op.zero_rows((long long)cur + 1, n_rows, lane);  // coverage ended
        }
        first_seg = false;
      }
      if (r >= 0) {
        if constexpr (kOut) {
          if (!(first_seg && head_open)) op.zero_rows((long long)last_valid + 1, r, lane);
        }
        op.begin(st, r, lane);
        last_valid = r;
        // the node that starts next in this tile: fetch its resident rows while this one is processed
        const int nx = i + rem;
        if (nx < nt) {
          const int rn = m_row[nx];
          if (rn >= 0 && rn != r) op.prefetch_node(st, rn, lane);
        }
      }
      cur = r;
    }
    cp_async_wait<DEPTH - U>();
    if constexpr (kShared) __syncwarp();  // every lane's copies of these entries have landed
    if (rem >= U) {  // the common case: a full batch of one node's edges
      if (r >= 0) op.template consume_batch<true>(st, ring, i, U, Op::kUsesEid ? m_eid + i : nullptr, lane);
      if constexpr (kShared) __syncwarp();  // all lanes have read the entries about to be refilled
#pragma unroll
      for (int u = 0; u < U; ++u) issue(i + u + DEPTH);
      new_seg = rem == U;
      i += U;
    } else {
      if (r >= 0) op.template consume_batch<false>(st, ring, i, rem, Op::kUsesEid ? m_eid + i : nullptr, lane);
      if constexpr (kShared) __syncwarp();
      for (int u = 0; u < rem; ++u) issue(i + u + DEPTH);
      new_seg = true;
      i += rem;
    }
  }
  cp_async_wait<0>();

  if constexpr (kOut) {
    int tail_row = -1;
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
      if (next < 0) op.zero_rows((long long)cur + 1, n_rows, lane);  // last covered position
    }
    if (rows_next && lane == 0) { rows_next[2 * t] = head_row; rows_next[2 * t + 1] = tail_row; }
  }
}

// Ring geometry shared by the staged ops: entries of `kOperands` feature rows (32*R slots of
// 16 bytes each) plus `kScalars` per-lane scalars of the accumulation type per register.
// Ring depth: the largest power of two (<= 16) whose ring, next to the tile metadata, lets
// `min_ctas` blocks of kWarpsPerCta warps share one SM's shared memory.
constexpr int pick_depth(int edge_bytes, int min_ctas, bool uses_eid) {
  const int budget = 216 * 1024 / min_ctas / kWarpsPerCta - (GK_TUNE_TILE + kMetaPad) * (uses_eid ? 13 : 9) - 16;
  int d = 16;
  while (d > 2 && d * edge_bytes > budget) d >>= 1;
  return d;
}
// Edges folded together; at most half the ring, so that the other half is in flight meanwhile.
constexpr int pick_batch(int r, int depth) {
  const int b0 = r == 1 ? 8 : (r == 2 ? 4 : 2);
  const int b = b0 < GK_TUNE_BATCH_MAX ? b0 : GK_TUNE_BATCH_MAX;
  const int half = depth / 2 > 1 ? depth / 2 : 1;
  return b < half ? b : half;
}

template <typename T, int R, int kOperands, int kScalars, bool kEid, int kCtasNarrow = GK_TUNE_CTAS_NARROW>
struct RingShape {
  using A = typename AccOf<T>::type;
  static constexpr int kRowBytes = 32 * R * 16;
  static constexpr int kScalarBytes = 32 * R * (int)sizeof(A);
  static constexpr int kEdgeBytes = kOperands * kRowBytes + kScalars * kScalarBytes;
  // 4-byte elements: 16 bytes of accumulator per slot, 64 registers are enough; 2-byte elements
  // (8 accumulators per slot) and doubles need the 80 registers of 3 resident blocks
  static constexpr int kMinCtas = R == 1 ? (sizeof(T) == 4 ? kCtasNarrow : (kCtasNarrow < 3 ? kCtasNarrow : 3))
                                         : (R == 2 ? 2 : 1);
  static constexpr int kDepth = pick_depth(kEdgeBytes, kMinCtas, kEid);
  static constexpr int kBatch = pick_batch(R, kDepth);
};

// Sum of per-register partial dot products over the lanes of one head, lanes-per-head known at
// compile time (LPH = 1, 2, 4, 8, 16 or 32; LPH = 0: read it from `lph`, any power of two).
template <int LPH, typename A, int R>
__device__ __forceinline__ void reduce_heads_ct(A (&p)[R], int lph) {
  if constexpr (LPH == 0) {
    reduce_heads<A, R>(p, lph);
  } else {
#pragma unroll
    for (int o = LPH >> 1; o; o >>= 1)
#pragma unroll
      for (int i = 0; i < R; ++i) p[i] += __shfl_xor_sync(kFull, p[i], o);
  }
}

#define GK_RING_ENTRY(pos) (ring + (size_t)((pos) & (kDepth - 1)) * kEdgeBytes)
#define GK_BATCH_LOOP(u) _Pragma("unroll") for (int u = 0; u < kBatch; ++u) if (kFullBatch || u < cnt)

// ---------------------------------------------------------------------------------------
// AggregateOp, staged: ring entry = [feature row][weights]
// ---------------------------------------------------------------------------------------
// kMode >= 0: the weight staging mode is known at compile time (the host instantiates the packed-pieces mode
// that way: no mode tests per edge); -1: read it from `wmode`.
template <typename T, int V, int R, bool kEdgeFeat, int kMode = -1>
struct AggregateStaged : AggregateOp<T, V, R, kEdgeFeat> {
  using Base = AggregateOp<T, V, R, kEdgeFeat>;
  using A = typename Base::A;
  struct State : Base::State { const unsigned char* xb[R]; };
  using Ring = RingShape<T, R, 1, 0, true>;
  // weights: one 4- or 8-byte word per lane and register (2-byte elements travel as the aligned
  // 4-byte word that contains them; the word's last 2 bytes may lie past an odd-sized tensor's end,
  // inside the allocation's padding)
  using WWord = typename std::conditional<sizeof(T) == 8, double, uint32_t>::type;
  static constexpr int kEdgeBytes = Ring::kRowBytes + 32 * R * (int)sizeof(WWord);
  static constexpr int kMinCtas = Ring::kMinCtas;
  static constexpr int kWarps = kWarpsPerCta;
  static constexpr bool kUsesEid = true;
  static constexpr bool kSharedEntry = true;  // in the packed modes lanes read weights that other lanes copied
  static constexpr int kDepth = pick_depth(kEdgeBytes, kMinCtas, true);
  static constexpr int kBatch = pick_batch(R, kDepth);
  // How an edge's H weights reach the ring entry (set by the host):
  //   kWeightsPerLane  every lane copies the word of its own head (any H, any element size);
  //   kWeightsWords    lane j < H copies weight j, lanes read the weight of their head (4- and 8-byte
  //                    elements, H <= 32 * R);
  //   kWeightsPieces   the H weights travel as 16-byte pieces copied by the first lanes (the weight
  //                    row is a whole number of aligned 16-byte pieces).
  // One scattered copy per edge instead of one per lane is what the packed modes buy.
  enum { kWeightsPerLane = 0, kWeightsWords = 1, kWeightsPieces = 2 };
  int wmode = kWeightsPerLane;
  __device__ __forceinline__ int mode() const { return kMode >= 0 ? kMode : wmode; }

  __host__ static int pick_wmode(const void* w, int H, int feat0, int HD, int block_elems) {
    const bool whole = feat0 == 0 && HD <= block_elems && H <= 32 * R;  // one feature block sees every head
    if (!whole) return kWeightsPerLane;
    if ((H * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) return kWeightsPieces;
    return sizeof(T) >= 4 ? kWeightsWords : kWeightsPerLane;
  }

  __device__ __forceinline__ void setup(State& st, int lane) const {
    Base::setup(st, lane);
#pragma unroll
    for (int i = 0; i < R; ++i)
      st.xb[i] = reinterpret_cast<const unsigned char*>(this->x + (kEdgeFeat ? st.sm.efeat[i] : st.sm.feat[i]));
  }
  __device__ __forceinline__ void stage(const State& st, unsigned char* entry, int c, int e, int lane) const {
    const int wbytes = this->H * (int)sizeof(T);
    const unsigned char* wrow = row_ptr(reinterpret_cast<const unsigned char*>(this->w), e, (unsigned)wbytes);
    const unsigned rowb = (unsigned)(kEdgeFeat ? this->D : this->HD) * (unsigned)sizeof(T);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.xb[i], kEdgeFeat ? e : c, rowb));
      const int j = lane + 32 * i;
      if (mode() == kWeightsPieces) {
        if (j * 16 < wbytes) cp_async16(entry + Ring::kRowBytes + j * 16, wrow + j * 16);
      } else if (mode() == kWeightsWords) {
        if constexpr (sizeof(T) >= 4) {
          if (j < this->H)
            cp_async_small<sizeof(T)>(entry + Ring::kRowBytes + j * sizeof(T), wrow + j * sizeof(T));
        }
      } else {
        const T* wsrc = this->w + (long long)e * this->H + st.sm.head[i];
        WWord* wdst = reinterpret_cast<WWord*>(entry + Ring::kRowBytes) + lane + 32 * i;
        if constexpr (sizeof(T) == 2)
          cp_async_small<4>(wdst, reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(wsrc) & ~uintptr_t(3)));
        else
          cp_async_small<sizeof(T)>(wdst, wsrc);
      }
    }
  }
  __device__ __forceinline__ void prefetch_node(State&, int, int) const {}
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt,
                                                const int* eids, int lane) const {
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        A xv[V];
        lds_acc<T, V>(xv, entry + (lane + 32 * i) * 16);
        A wv;
        if (mode() != kWeightsPerLane) {
          wv = to_acc<T>(reinterpret_cast<const T*>(entry + Ring::kRowBytes)[st.sm.head[i]]);
        } else if constexpr (sizeof(T) == 2) {
          const WWord word = reinterpret_cast<const WWord*>(entry + Ring::kRowBytes)[lane + 32 * i];
          const bool hi = (((long long)eids[u] * this->H + st.sm.head[i]) & 1) != 0;
          union { uint16_t b; T t; } cvt;
          cvt.b = (uint16_t)(hi ? (word >> 16) : (word & 0xffffu));
          wv = to_acc<T>(cvt.t);
        } else {
          union { WWord wd; T t; } cvt;
          cvt.wd = reinterpret_cast<const WWord*>(entry + Ring::kRowBytes)[lane + 32 * i];
          wv = to_acc<T>(cvt.t);
        }
#pragma unroll
        for (int v = 0; v < V; ++v) st.acc[i][v] += wv * xv[v];
      }
    }
  }
};

// ---------------------------------------------------------------------------------------
// EdgeDotOp, staged: ring entry = [gathered row]
// ---------------------------------------------------------------------------------------
template <typename T, int V, int R, bool kEdgeFeat, int LPH>
struct EdgeDotStaged : EdgeDotOp<T, V, R, kEdgeFeat> {
  using Base = EdgeDotOp<T, V, R, kEdgeFeat>;
  using A = typename Base::A;
  struct State : Base::State { A an[R][V]; int next_node; const unsigned char* bb[R]; };
  // the next node\'s resident rows are fetched ahead only while they fit 16 bytes per lane: wider rows need
  // the registers for the node being processed
  static constexpr bool kPrefetch = R * V * (int)sizeof(A) <= 16;
  using Ring = RingShape<T, R, 1, 0, true>;
  static constexpr int kEdgeBytes = Ring::kEdgeBytes, kDepth = Ring::kDepth, kBatch = Ring::kBatch,
                       kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr bool kUsesEid = true;

  __device__ __forceinline__ void setup(State& st, int lane) const {
    Base::setup(st, lane);
    st.next_node = -1;
#pragma unroll
    for (int i = 0; i < R; ++i)
      st.bb[i] = reinterpret_cast<const unsigned char*>(this->b + (kEdgeFeat ? st.sm.efeat[i] : st.sm.feat[i]));
  }
  __device__ __forceinline__ void prefetch_node(State& st, int node, int) const {
    if constexpr (!kPrefetch) return;
#pragma unroll
    for (int i = 0; i < R; ++i) load_acc<T, V>(st.an[i], this->a + (long long)node * this->HD + st.sm.feat[i]);
    st.next_node = node;
  }
  __device__ __forceinline__ void begin(State& st, int node, int lane) const {
    if (kPrefetch && st.next_node == node) {
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int v = 0; v < V; ++v) st.a[i][v] = st.sm.ok[i] ? st.an[i][v] : A(0);
    } else {
      Base::begin(st, node, lane);
    }
  }
  __device__ __forceinline__ void stage(const State& st, unsigned char* entry, int c, int e, int lane) const {
    const unsigned rowb = (unsigned)(kEdgeFeat ? this->D : this->HD) * (unsigned)sizeof(T);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.bb[i], kEdgeFeat ? e : c, rowb));
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt,
                                                const int* eids, int lane) const {
    A p[kBatch][R];
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        A bv[V];
        lds_acc<T, V>(bv, entry + (lane + 32 * i) * 16);
        p[u][i] = A(0);
#pragma unroll
        for (int v = 0; v < V; ++v) p[u][i] += st.a[i][v] * bv[v];
      }
    }
    GK_BATCH_LOOP(u) reduce_heads_ct<LPH, A, R>(p[u], this->lph);
    const int lph = LPH ? LPH : this->lph;
    const int rph = lph >= 32 ? lph >> 5 : 1;
    const bool writer = lph >= 32 ? lane == 0 : (lane & (lph - 1)) == 0;
    if (writer) {
      GK_BATCH_LOOP(u) {
        const long long e = eids[u];
#pragma unroll
        for (int i = 0; i < R; ++i)
          if (st.sm.ok[i] && (i % rph) == 0) this->y[e * this->H + st.sm.head[i]] = from_acc<T>(p[u][i]);
      }
    }
  }
};

// ---------------------------------------------------------------------------------------
// Fused attention forward, staged.  Scores are kept in base-2 units: q is multiplied by
// scale * log2(e) when a node starts, so a probability is one ex2 of a difference.
// ring entry = [k row][v row]
// ---------------------------------------------------------------------------------------
template <typename T, int V, int R, int LPH>
struct AttnFwdStaged : AttnFwdOp<T, V, R> {
  using Base = AttnFwdOp<T, V, R>;
  using A = typename Base::A;
  struct State : Base::State { A qn[R][V]; int next_node; const unsigned char* kb[R]; const unsigned char* vb[R]; };
  // the next node\'s resident rows are fetched ahead only while they fit 16 bytes per lane: wider rows need
  // the registers for the node being processed
  static constexpr bool kPrefetch = R * V * (int)sizeof(A) <= 16;
  using CarryIn = typename Base::CarryIn;
  using Ring = RingShape<T, R, 2, 0, false>;
  static constexpr int kEdgeBytes = Ring::kEdgeBytes, kDepth = Ring::kDepth, kBatch = Ring::kBatch,
                       kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr bool kUsesEid = false;

  __device__ __forceinline__ void setup(State& st, int lane) const {
    Base::setup(st, lane);
    st.next_node = -1;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.kb[i] = reinterpret_cast<const unsigned char*>(this->k + st.sm.feat[i]);
      st.vb[i] = reinterpret_cast<const unsigned char*>(this->v + st.sm.feat[i]);
    }
  }
  __device__ __forceinline__ void prefetch_node(State& st, int node, int) const {
    if constexpr (!kPrefetch) return;
#pragma unroll
    for (int i = 0; i < R; ++i) load_acc<T, V>(st.qn[i], this->q + (long long)node * this->HD + st.sm.feat[i]);
    st.next_node = node;
  }
  __device__ __forceinline__ void begin(State& st, int node, int lane) const {
    const A c = this->scale * A(kLog2e);
    if (kPrefetch && st.next_node == node) {
#pragma unroll
      for (int i = 0; i < R; ++i) {
        st.m[i] = neg_inf<A>();
        st.l[i] = A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) { st.acc[i][e] = A(0); st.q[i][e] = st.sm.ok[i] ? st.qn[i][e] * c : A(0); }
      }
      return;
    }
    Base::begin(st, node, lane);
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int e = 0; e < V; ++e) st.q[i][e] *= c;
  }
  __device__ __forceinline__ void stage(const State& st, unsigned char* entry, int c, int, int lane) const {
    const unsigned rowb = (unsigned)this->HD * (unsigned)sizeof(T);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.kb[i], c, rowb));
      cp_async16(entry + Ring::kRowBytes + (lane + 32 * i) * 16, row_ptr(st.vb[i], c, rowb));
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt, const int*,
                                                int lane) const {
    A s[kBatch][R];
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        A kv[V];
        lds_acc<T, V>(kv, entry + (lane + 32 * i) * 16);
        s[u][i] = A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) s[u][i] += st.q[i][e] * kv[e];
      }
    }
    GK_BATCH_LOOP(u) reduce_heads_ct<LPH, A, R>(s[u], this->lph);
    // one rescale per batch: new maximum over the batch, then the batch's terms
#pragma unroll
    for (int i = 0; i < R; ++i) {
      A mn = st.m[i];
      GK_BATCH_LOOP(u) mn = s[u][i] > mn ? s[u][i] : mn;
      const A corr = gk_exp2(st.m[i] - mn);  // m = -inf at a node's first batch: 2^-inf = 0
      st.m[i] = mn;
      st.l[i] *= corr;
#pragma unroll
      for (int e = 0; e < V; ++e) st.acc[i][e] *= corr;
    }
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u) + Ring::kRowBytes;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const A p = gk_exp2(s[u][i] - st.m[i]);
        st.l[i] += p;
        A vv[V];
        lds_acc<T, V>(vv, entry + (lane + 32 * i) * 16);
#pragma unroll
        for (int e = 0; e < V; ++e) st.acc[i][e] += p * vv[e];
      }
    }
  }
  // m is a base-2 exponent here: lse = (m + log2 l) * ln 2, and partials merge with ex2
  __device__ __forceinline__ void store_row(const State& st, int node, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (st.sm.ok[i]) {
        const A inv = A(1) / st.l[i];
        A out[V];
#pragma unroll
        for (int e = 0; e < V; ++e) out[e] = st.acc[i][e] * inv;
        store_acc<T, V>(this->o + (long long)node * this->HD + st.sm.feat[i], out);
        if (st.sm.efeat[i] == 0)
          this->lse[(long long)node * this->H + st.sm.head[i]] = (st.m[i] + gk_log2(st.l[i])) * A(kLn2);
      }
    }
  }
  __device__ __forceinline__ void merge_carry(State& st, const CarryIn& ci, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (st.sm.ok[i]) {
        const A mc = ci.m[i];
        const A mn = mc > st.m[i] ? mc : st.m[i];
        const A wa = st.m[i] == neg_inf<A>() ? A(0) : gk_exp2(st.m[i] - mn);
        const A wb = mc == neg_inf<A>() ? A(0) : gk_exp2(mc - mn);
        st.l[i] = st.l[i] * wa + ci.l[i] * wb;
#pragma unroll
        for (int e = 0; e < V; ++e) st.acc[i][e] = st.acc[i][e] * wa + ci.acc[i][e] * wb;
        st.m[i] = mn;
      }
  }
};

// ---------------------------------------------------------------------------------------
// Fused attention backward, destination side, staged.  ring entry = [k row][v row]
// ---------------------------------------------------------------------------------------
template <typename T, int V, int R, int LPH>
struct AttnBwdDstStaged : AttnBwdDstOp<T, V, R> {
  using Base = AttnBwdDstOp<T, V, R>;
  using A = typename Base::A;
  struct State : Base::State {
    A qn[R][V]; A gn[R][V]; A on[R][V]; A lsen[R]; int next_node; int tile_base;
    const unsigned char* kb[R]; const unsigned char* vb[R];
    unsigned char* pdw[R];  // where this lane writes its head's (p, ds) of edge 0, or null: not the head's writer
  };
  static constexpr bool kTileBase = true;
  EdgePair<A>* __restrict__ pd = nullptr;  // (n_edges, Hp) out when not null: (p, ds) of every edge, by position
  // the next node\'s resident rows are fetched ahead only while they fit 16 bytes per lane: wider rows need
  // the registers for the node being processed
  static constexpr bool kPrefetch = R * V * (int)sizeof(A) <= 16;
  using Ring = RingShape<T, R, 2, 0, false>;
  static constexpr int kEdgeBytes = Ring::kEdgeBytes, kDepth = Ring::kDepth, kBatch = Ring::kBatch,
                       kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr bool kUsesEid = false;

  __device__ __forceinline__ void setup(State& st, int lane) const {
    Base::setup(st, lane);
    st.next_node = -1;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.kb[i] = reinterpret_cast<const unsigned char*>(this->k + st.sm.feat[i]);
      st.vb[i] = reinterpret_cast<const unsigned char*>(this->v + st.sm.feat[i]);
      st.pdw[i] = (pd && st.sm.ok[i] && st.sm.efeat[i] == 0) ? reinterpret_cast<unsigned char*>(pd + st.sm.head[i])
                                                              : nullptr;
    }
  }
  __device__ __forceinline__ void prefetch_node(State& st, int node, int) const {
    if constexpr (!kPrefetch) return;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const long long off = (long long)node * this->HD + st.sm.feat[i];
      load_acc<T, V>(st.qn[i], this->q + off);
      load_acc<T, V>(st.gn[i], this->dout + off);
      load_acc<T, V>(st.on[i], this->o + off);
      st.lsen[i] = __ldg(this->lse + (long long)node * this->H + st.sm.head[i]);
    }
    st.next_node = node;
  }
  // q scaled to base-2 score units, lse converted to base 2
  __device__ __forceinline__ void begin(State& st, int node, int lane) const {
    const A c = this->scale * A(kLog2e);
    if (kPrefetch && st.next_node == node) {
      A dl[R];
#pragma unroll
      for (int i = 0; i < R; ++i) {
        dl[i] = A(0);
        st.lse[i] = st.sm.ok[i] ? st.lsen[i] * A(kLog2e) : A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) {
          st.acc[i][e] = A(0);
          st.q[i][e] = st.sm.ok[i] ? st.qn[i][e] * c : A(0);
          st.g[i][e] = st.sm.ok[i] ? st.gn[i][e] : A(0);
          dl[i] += st.g[i][e] * st.on[i][e];
        }
      }
      reduce_heads_ct<LPH, A, R>(dl, this->lph);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        st.delta[i] = dl[i];
        if (st.sm.ok[i] && st.sm.efeat[i] == 0)
          this->stat[(long long)node * this->Hp + st.sm.head[i]] = StatPair<A>{st.lsen[i], dl[i]};
      }
      return;
    }
    Base::begin(st, node, lane);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.lse[i] *= A(kLog2e);
#pragma unroll
      for (int e = 0; e < V; ++e) st.q[i][e] *= c;
    }
  }
  __device__ __forceinline__ void stage(const State& st, unsigned char* entry, int c, int, int lane) const {
    const unsigned rowb = (unsigned)this->HD * (unsigned)sizeof(T);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.kb[i], c, rowb));
      cp_async16(entry + Ring::kRowBytes + (lane + 32 * i) * 16, row_ptr(st.vb[i], c, rowb));
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt, const int*,
                                                int lane) const {
    const unsigned pairb = (unsigned)this->Hp * (unsigned)sizeof(EdgePair<A>);
    A s[kBatch][R], dp[kBatch][R];
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        A kv[V], vv[V];
        lds_acc<T, V>(kv, entry + (lane + 32 * i) * 16);
        lds_acc<T, V>(vv, entry + Ring::kRowBytes + (lane + 32 * i) * 16);
        s[u][i] = A(0);
        dp[u][i] = A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) { s[u][i] += st.q[i][e] * kv[e]; dp[u][i] += st.g[i][e] * vv[e]; }
      }
    }
    GK_BATCH_LOOP(u) { reduce_heads_ct<LPH, A, R>(s[u], this->lph); reduce_heads_ct<LPH, A, R>(dp[u], this->lph); }
    // the k row is read again rather than kept: registers matter more than the second read
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const A p = gk_exp2(s[u][i] - st.lse[i]);
        const A ds = p * (dp[u][i] - st.delta[i]) * this->scale;
        if (st.pdw[i])
          *reinterpret_cast<EdgePair<A>*>(st.pdw[i] + (unsigned long long)(unsigned)(st.tile_base + i0 + u) * pairb) =
              EdgePair<A>{p, ds};
        A kv[V];
        lds_acc<T, V>(kv, entry + (lane + 32 * i) * 16);
#pragma unroll
        for (int e = 0; e < V; ++e) st.acc[i][e] += ds * kv[e];
      }
    }
  }
};

// ---------------------------------------------------------------------------------------
// Fused attention backward, source side, staged.
// ring entry = [q row of the destination][dO row][lse][delta]
// ---------------------------------------------------------------------------------------
template <typename T, int V, int R, int LPH>
struct AttnBwdSrcStaged : AttnBwdSrcOp<T, V, R> {
  using Base = AttnBwdSrcOp<T, V, R>;
  using A = typename Base::A;
  struct State : Base::State { A kn[R][V]; A vn[R][V]; int next_node; };
  // the next node\'s resident rows are fetched ahead only while they fit 16 bytes per lane: wider rows need
  // the registers for the node being processed
  static constexpr bool kPrefetch = R * V * (int)sizeof(A) <= 16;
  using Ring = RingShape<T, R, 2, 0, false, GK_TUNE_CTAS_SRC>;
  // (lse, delta) pairs of the most heads this instantiation can see: 32 * R / LPH (every head when the
  // lanes per head are only known at run time), at least one 16-byte piece
  static constexpr int kMaxHeads = LPH ? (32 * R / LPH > 2 ? 32 * R / LPH : 2) : 32 * R;
  static constexpr int kPairBytes = (kMaxHeads * (int)sizeof(StatPair<A>) + 15) / 16 * 16;
  static constexpr int kEdgeBytes = 2 * Ring::kRowBytes + kPairBytes;
  static constexpr int kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr int kDepth = pick_depth(kEdgeBytes, kMinCtas, false);
  static constexpr int kBatch = pick_batch(R, kDepth);
  static constexpr bool kUsesEid = false;
  static constexpr bool kSharedEntry = true;  // lanes read pair bytes that other lanes copied

  __device__ __forceinline__ void setup(State& st, int lane) const { Base::setup(st, lane); st.next_node = -1; }
  __device__ __forceinline__ void prefetch_node(State& st, int node, int) const {
    if constexpr (!kPrefetch) return;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const long long off = (long long)node * this->HD + st.sm.feat[i];
      load_acc<T, V>(st.kn[i], this->k + off);
      load_acc<T, V>(st.vn[i], this->v + off);
    }
    st.next_node = node;
  }
  // k scaled to base-2 score units
  __device__ __forceinline__ void begin(State& st, int node, int lane) const {
    const A c = this->scale * A(kLog2e);
    if (kPrefetch && st.next_node == node) {
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int e = 0; e < V; ++e) {
          st.ak[i][e] = A(0);
          st.av[i][e] = A(0);
          st.k[i][e] = st.sm.ok[i] ? st.kn[i][e] * c : A(0);
          st.v[i][e] = st.sm.ok[i] ? st.vn[i][e] : A(0);
        }
      return;
    }
    Base::begin(st, node, lane);
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int e = 0; e < V; ++e) st.k[i][e] *= c;
  }
  __device__ __forceinline__ void stage(const State& st, unsigned char* entry, int c, int, int lane) const {
    // the node's (lse, delta) pairs: Hp pairs = `pieces` copies of 16 bytes, one per low lane
    const unsigned pairb = (unsigned)this->Hp * (unsigned)sizeof(StatPair<A>);
    const unsigned char* pairs = row_ptr(reinterpret_cast<const unsigned char*>(this->stat), c, pairb);
    const int pieces = (int)(pairb / 16);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      // plain index arithmetic here: the per-lane base pointers of the other two kernels would cost this
      // one, which is at its register limit, more than they save
      cp_async16(entry + (lane + 32 * i) * 16, this->q + (long long)c * this->HD + st.sm.feat[i]);
      cp_async16(entry + Ring::kRowBytes + (lane + 32 * i) * 16, this->dout + (long long)c * this->HD + st.sm.feat[i]);
      const int piece = lane + 32 * i;
      if (piece < pieces) cp_async16(entry + 2 * Ring::kRowBytes + piece * 16, pairs + piece * 16);
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt, const int*,
                                                int lane) const {
    A s[kBatch][R], dp[kBatch][R];
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        A qv[V], gv[V];
        lds_acc<T, V>(qv, entry + (lane + 32 * i) * 16);
        lds_acc<T, V>(gv, entry + Ring::kRowBytes + (lane + 32 * i) * 16);
        s[u][i] = A(0);
        dp[u][i] = A(0);
#pragma unroll
        for (int e = 0; e < V; ++e) { s[u][i] += qv[e] * st.k[i][e]; dp[u][i] += gv[e] * st.v[i][e]; }
      }
    }
    GK_BATCH_LOOP(u) { reduce_heads_ct<LPH, A, R>(s[u], this->lph); reduce_heads_ct<LPH, A, R>(dp[u], this->lph); }
    // the q and dout rows are read again rather than kept: registers matter more than the second read
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u);
      const StatPair<A>* sc = reinterpret_cast<const StatPair<A>*>(entry + 2 * Ring::kRowBytes);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const StatPair<A> pr = sc[st.sm.head[i]];
        const A p = gk_exp2(s[u][i] - pr.lse * A(kLog2e));
        const A ds = p * (dp[u][i] - pr.delta) * this->scale;
        A qv[V], gv[V];
        lds_acc<T, V>(qv, entry + (lane + 32 * i) * 16);
        lds_acc<T, V>(gv, entry + Ring::kRowBytes + (lane + 32 * i) * 16);
#pragma unroll
        for (int e = 0; e < V; ++e) { st.av[i][e] += p * gv[e]; st.ak[i][e] += ds * qv[e]; }
      }
    }
  }
  // dk accumulated against k in base-2 units would be wrong: ak sums ds * q, which does not involve k,
  // so nothing to undo at store time.
};

// ---------------------------------------------------------------------------------------
// Source side of the attention backward when the destination pass left (p, ds) of every edge:
//     dv[c] = sum_k p_k * dO[dst_k],     dk[c] = sum_k ds_k * q[dst_k]
// Two weighted aggregations: no dot products, no k / v rows.  Ring entry = [q row][dO row][(p, ds) pairs of the
// edge], the pairs fetched by edge id (the transposed CSR's eid).  Row output, carries and gap fill are the
// base op's.
// ---------------------------------------------------------------------------------------
template <typename T, int V, int R, int LPH>
struct AttnBwdSrcPairsStaged : AttnBwdSrcOp<T, V, R> {
  using Base = AttnBwdSrcOp<T, V, R>;
  using A = typename Base::A;
  struct State : Base::State { const unsigned char* qb[R]; const unsigned char* gb[R]; };
  using Ring = RingShape<T, R, 2, 0, true, GK_TUNE_CTAS_SRC>;
  static constexpr int kMaxHeads = LPH ? (32 * R / LPH > 2 ? 32 * R / LPH : 2) : 32 * R;
  static constexpr int kPairBytes = (kMaxHeads * (int)sizeof(EdgePair<A>) + 15) / 16 * 16;
  static constexpr int kEdgeBytes = 2 * Ring::kRowBytes + kPairBytes;
  static constexpr int kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr int kDepth = pick_depth(kEdgeBytes, kMinCtas, true);
  static constexpr int kBatch = pick_batch(R, kDepth);
  static constexpr bool kUsesEid = true;
  static constexpr bool kSharedEntry = true;  // lanes read pair bytes that other lanes copied
  const EdgePair<A>* __restrict__ pd;          // (n_edges, Hp) by edge id, from the destination pass

  __device__ __forceinline__ void setup(State& st, int lane) const {
    Base::setup(st, lane);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.qb[i] = reinterpret_cast<const unsigned char*>(this->q + st.sm.feat[i]);
      st.gb[i] = reinterpret_cast<const unsigned char*>(this->dout + st.sm.feat[i]);
    }
  }
  __device__ __forceinline__ void prefetch_node(State&, int, int) const {}
  __device__ __forceinline__ void begin(State& st, int, int) const {
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int e = 0; e < V; ++e) { st.ak[i][e] = A(0); st.av[i][e] = A(0); }
  }
  __device__ __forceinline__ void stage(const State& st, unsigned char* entry, int c, int e, int lane) const {
    const unsigned rowb = (unsigned)this->HD * (unsigned)sizeof(T);
    const unsigned pairb = (unsigned)this->Hp * (unsigned)sizeof(EdgePair<A>);
    const unsigned char* pairs = row_ptr(reinterpret_cast<const unsigned char*>(pd), e, pairb);
    const int pieces = (int)(pairb / 16);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.qb[i], c, rowb));
      cp_async16(entry + Ring::kRowBytes + (lane + 32 * i) * 16, row_ptr(st.gb[i], c, rowb));
      const int piece = lane + 32 * i;
      if (piece < pieces) cp_async16(entry + 2 * Ring::kRowBytes + piece * 16, pairs + piece * 16);
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int i0, int cnt, const int*,
                                                int lane) const {
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_ENTRY(i0 + u);
      const EdgePair<A>* pr = reinterpret_cast<const EdgePair<A>*>(entry + 2 * Ring::kRowBytes);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const EdgePair<A> w = pr[st.sm.head[i]];
        A qv[V], gv[V];
        lds_acc<T, V>(qv, entry + (lane + 32 * i) * 16);
        lds_acc<T, V>(gv, entry + Ring::kRowBytes + (lane + 32 * i) * 16);
#pragma unroll
        for (int e = 0; e < V; ++e) { st.av[i][e] += w.p * gv[e]; st.ak[i][e] += w.ds * qv[e]; }
      }
    }
  }
};

}  // namespace gk
