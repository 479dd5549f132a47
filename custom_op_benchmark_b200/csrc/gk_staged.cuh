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

// Launch shape of the staged kernels, chosen by measurement on a B200 (R-MAT scale 21, 4 heads x 32, fp32).
// All of them are bound by how many gathered rows the shared-memory rings keep in flight per SM, so the numbers
// below trade resident warps against ring depth.
#define GK_CTAS_NARROW 4     // resident blocks per SM aimed at when a node row fits one 16-byte slot per lane
#define GK_CTAS_DST 3        // attention backward, destination side: its state needs the 80 registers of 3 blocks
#define GK_CTAS_SRC 4        // attention backward, source side
#define GK_TILE 256          // largest level-0 tile (positions per warp)
#define GK_FAST_BATCH 2      // batch of the transposed-reduction paths (2 or 4)

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
//   void consume_batch(State&, const unsigned char* first, int cnt, const int* eids, int lane)
//        fold cnt positions whose ring entries are first, first + kEdgeBytes, ...;
//        kFullBatch: cnt == kBatch, known at compile time
// Lanes whose slot does not exist (slot >= S) copy nothing in stage (32 lanes fetching slot 0 again cost a
// narrow row - one head of 32 floats - more than the row itself: the kernels ran 2.5x slower on it than on a
// 512-byte row); the walker zeroes every ring once per tile, so what those lanes read in consume_batch is zero,
// their node-resident operand is zero as well, and only stores test `ok`.

// Ops that hand a batch's per-edge scalars from their owner lanes to all lanes of a head through shared memory
// declare `kScratchBytes` (a multiple of 16): that many bytes per warp follow the ring.
template <class Op, class = void> struct ScratchBytes { static constexpr int value = 0; };
template <class Op> struct ScratchBytes<Op, std::void_t<decltype(Op::kScratchBytes)>> {
  static constexpr int value = Op::kScratchBytes;
};

// Tile metadata lives in a window of two blocks of 32 positions per warp (node, other endpoint, edge id if the
// op uses it, one run-length byte), refilled block by block while the tile is walked: a few hundred bytes per
// warp instead of the whole tile's, which leaves the shared memory to the rings.
constexpr int kWinBlock = 32, kWin = 2 * kWinBlock;

// Shared memory of one warp: the metadata window rounded to 16 bytes, kDepth ring entries, the op's scratch.
template <class Op>
__host__ __device__ constexpr size_t staged_meta_bytes() {
  return ((size_t)kWin * (Op::kUsesEid ? 13 : 9) + 15) / 16 * 16;
}
template <class Op>
__host__ __device__ constexpr size_t staged_warp_bytes() {
  return staged_meta_bytes<Op>() + (size_t)Op::kDepth * Op::kEdgeBytes + (size_t)ScratchBytes<Op>::value;
}

// Ops whose lanes read ring bytes copied by other lanes declare `kSharedEntry = true`; the walker
// then puts a warp barrier between the copies' completion and the reads, and between the reads and
// the refill.  Every other op reads back only the bytes the same lane copied and needs neither.
template <class Op, class = void> struct SharesEntries : std::false_type {};
template <class Op> struct SharesEntries<Op, std::void_t<decltype(Op::kSharedEntry)>> : std::true_type {};

// Ops that need the global position of the edges they fold declare `kTileBase = true` and get the tile's
// first position in `State::tile_base` (positions stay below 2^31) and the batch's offset in `State::batch_pos`.
template <class Op, class = void> struct WantsTileBase : std::false_type {};
template <class Op> struct WantsTileBase<Op, std::void_t<decltype(Op::kTileBase)>> : std::true_type {};

// Ops whose begin(node) reads rows of node tensors declare `kNodeRows = true` and implement
// prefetch_rows_l2(node): the walker calls it for every node that starts in a metadata block when the block
// enters the window, 32 to 64 positions before the node is reached, so that begin() finds the rows in the L2
// cache instead of paying a DRAM round trip per node (a graph with millions of short rows is otherwise bound
// by exactly that latency).  One request per 128-byte line: a few per node, nothing beside the gathers.
template <class Op, class = void> struct NodeRows : std::false_type {};
template <class Op> struct NodeRows<Op, std::void_t<decltype(Op::kNodeRows)>> : std::true_type {};
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
__device__ __forceinline__ void prefetch_row_l2(const void* row, unsigned row_bytes) {
  for (unsigned off = 0; off < row_bytes; off += 128) prefetch_l2(reinterpret_cast<const unsigned char*>(row) + off);
}

// U consecutive ints from shared memory (U a power of two up to 8, the address a multiple of 4 U bytes).
template <int U>
__device__ __forceinline__ void load_meta(int (&d)[U], const int* p) {
  if constexpr (U == 1) {
    d[0] = p[0];
  } else if constexpr (U == 2) {
    const int2 t = *reinterpret_cast<const int2*>(p);
    d[0] = t.x; d[1] = t.y;
  } else {
#pragma unroll
    for (int k = 0; k < U / 4; ++k) {
      const int4 t = reinterpret_cast<const int4*>(p)[k];
      d[4 * k] = t.x; d[4 * k + 1] = t.y; d[4 * k + 2] = t.z; d[4 * k + 3] = t.w;
    }
  }
}

template <class Op>
__global__ void __launch_bounds__(Op::kWarps * 32, Op::kMinCtas)
walk_staged_kernel(Op op, const PlanHeader* __restrict__ hdr, const int32_t* __restrict__ erow,
                   const int32_t* __restrict__ other, const int32_t* __restrict__ eid, long long E, int tile,
                   long long n_rows, int32_t* __restrict__ rows_next, const int32_t* __restrict__ tile_start) {
  constexpr int U = Op::kBatch;
  constexpr int DEPTH = Op::kDepth;
  constexpr int EB = Op::kEdgeBytes;
  constexpr bool kOut = Op::kRowOut;
  constexpr bool kShared = SharesEntries<Op>::value;
  static_assert((U & (U - 1)) == 0 && DEPTH % U == 0 && DEPTH + U <= kWinBlock,
                "batch: a power of two; ring: whole batches, look-ahead within one block");
  extern __shared__ uint4 gk_smem[];
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  const long long t = (long long)blockIdx.x * Op::kWarps + w;
  // uniform tiles, or a plan's row-aligned ones (see walk_kernel): up to 2 * tile - 1 positions then, which the
  // rolling metadata window does not mind
  if (t * tile >= E) return;
  const long long j0 = tile_start ? (long long)__ldg(tile_start + t) : t * tile;
  const long long j1 = tile_start ? (long long)__ldg(tile_start + t + 1) : (j0 + tile < E ? j0 + tile : E);
  const int nt = (int)(j1 - j0);

  if constexpr (kOut) {
    if (t == 0 && hdr->cover_hi <= hdr->cover_lo) {  // no covered position at all
      op.zero_rows(0, n_rows, lane);
      if (rows_next && lane == 0) { rows_next[0] = -1; rows_next[1] = -1; }
      return;
    }
  }

  unsigned char* mine = reinterpret_cast<unsigned char*>(gk_smem) + (size_t)w * staged_warp_bytes<Op>();
  int* w_row = reinterpret_cast<int*>(mine);
  int* w_oth = w_row + kWin;
  int* w_eid = w_oth + kWin;  // present only when Op::kUsesEid
  unsigned char* w_rem = reinterpret_cast<unsigned char*>(w_oth + (Op::kUsesEid ? 2 : 1) * kWin);
  unsigned char* ring = mine + staged_meta_bytes<Op>();
  // ring bytes of slots that do not exist (rows narrower than the lanes) are never copied to: they read as zero
  for (int off = lane * 16; off < DEPTH * EB; off += 32 * 16) *reinterpret_cast<uint4*>(ring + off) = uint4{0, 0, 0, 0};

  // Metadata window.  Block b (positions 32 b .. 32 b + 31 of the tile) occupies window entries
  // (b & 1) * 32 + lane.  w_rem = number of consecutive positions from this one on that have the same node,
  // never past the block's end: a batch never crosses a block.  Positions past the tile get node -2, and every
  // position without a node points at node 0 / edge 0, so that the ring can be refilled without looking at the
  // node.  One block is always held in registers ahead of the window.
  const int before = j0 > 0 ? __ldg(erow + j0 - 1) : -1;
  int nr, no, ne;
  auto fetch_block = [&](int b) {
    const int i = b * kWinBlock + lane;
    const bool inb = i < nt;
    nr = inb ? __ldg(erow + j0 + i) : -2;
    no = (inb && other) ? __ldg(other + j0 + i) : 0;
    ne = (Op::kUsesEid && inb) ? (eid ? __ldg(eid + j0 + i) : (int)(j0 + i)) : 0;
  };
  auto publish_block = [&](int b) {
    const int s = (b & 1) * kWinBlock + lane;
    const int down = __shfl_down_sync(kFull, nr, 1);
    const unsigned ends = __ballot_sync(kFull, lane == 31 || nr != down);  // bit l: a run ends at lane l
    if constexpr (NodeRows<Op>::value) {
      const int up = __shfl_up_sync(kFull, nr, 1);
      if (nr >= 0 && (lane == 0 || nr != up)) op.prefetch_rows_l2(nr);  // a node starts (or goes on) here
    }
    w_row[s] = nr;
    w_oth[s] = nr >= 0 ? no : 0;
    if constexpr (Op::kUsesEid) w_eid[s] = nr >= 0 ? ne : 0;
    w_rem[s] = (unsigned char)__ffs(ends >> lane);
  };
  fetch_block(0);
  publish_block(0);
  fetch_block(1);
  publish_block(1);
  fetch_block(2);
  __syncwarp();

  typename Op::State st;
  op.setup(st, lane);
  if constexpr (WantsTileBase<Op>::value) st.tile_base = (int)j0;
  if constexpr (ScratchBytes<Op>::value != 0) st.scratch = ring + (size_t)DEPTH * EB;
  const int first = w_row[0];
  const bool head_open = before >= 0 && before == first;
  bool first_seg = true;
  int cur = -1;
  int last_valid = before;
  int head_row = -1;

  // The ring is NG groups of U entries.  Group g of the tile (positions g U .. g U + U - 1) always occupies ring
  // group g mod NG, so every entry of a batch sits at a compile-time offset from the group's base, and one
  // cp.async commit group per refill maps commit groups one to one onto ring groups: waiting for all but the
  // last NG - 1 commit groups is waiting for exactly the group about to be folded.  Copies are issued whether
  // or not a position carries an edge.
  constexpr int NG = DEPTH / U;
  constexpr int kGroupBytes = U * EB;
  auto refill = [&](int pos0, unsigned char* grp) {
    const int wi = pos0 & (kWin - 1);
    int oth[U], eds[U];
    load_meta<U>(oth, w_oth + wi);
    if constexpr (Op::kUsesEid) load_meta<U>(eds, w_eid + wi);
#pragma unroll
    for (int u = 0; u < U; ++u) op.stage(st, grp + u * EB, oth[u], Op::kUsesEid ? eds[u] : 0, lane);
    cp_async_commit();
  };
#pragma unroll
  for (int g = 0; g < NG; ++g) refill(g * U, ring + g * kGroupBytes);

  // a segment of node r starts at position `pos` (r < 0: positions without a node)
  auto enter = [&](int r, int pos) {
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
      const int nx = pos + w_rem[pos & (kWin - 1)];
      if (nx < nt) {
        const int rn = w_row[nx & (kWin - 1)];
        if (rn >= 0 && rn != r) op.prefetch_node(st, rn, lane);
      }
    }
    cur = r;
  };

  int blk = 0;
  unsigned char* grp = ring;  // ring group of the batch being folded
  for (int i = 0; i < nt; i += U) {
    if (i >= (blk + 1) * kWinBlock) {
      // the walk enters block blk + 1: block blk's window entries are free for block blk + 2
      __syncwarp();
      ++blk;
      publish_block(blk + 1);
      fetch_block(blk + 2);
      __syncwarp();
    }
    const int wi = i & (kWin - 1);
    int rows[U];
    load_meta<U>(rows, w_row + wi);
    bool uniform = rows[0] == cur;
#pragma unroll
    for (int u = 1; u < U; ++u) uniform = uniform && rows[u] == rows[0];
    cp_async_wait<NG - 1>();
    if constexpr (kShared) __syncwarp();  // every lane's copies of these entries have landed
    if (uniform) {  // the common case: a whole group of the current node's edges
      if (cur >= 0) {
        if constexpr (WantsTileBase<Op>::value) st.batch_pos = i;
        op.template consume_batch<true>(st, grp, U, Op::kUsesEid ? w_eid + wi : nullptr, lane);
      }
    } else {
      // run by run: the group holds a node boundary, the tile's end or positions without a node
      int u = 0;
      while (u < U && i + u < nt) {
        const int r = w_row[wi + u];
        int run = w_rem[wi + u];
        run = run < U - u ? run : U - u;
        if (r != cur) enter(r, i + u);  // adjacent runs never share a node
        if (r >= 0) {
          if constexpr (WantsTileBase<Op>::value) st.batch_pos = i + u;
          if (run == U) op.template consume_batch<true>(st, grp, U, Op::kUsesEid ? w_eid + wi : nullptr, lane);
          else op.template consume_batch<false>(st, grp + u * EB, run, Op::kUsesEid ? w_eid + wi + u : nullptr, lane);
        }
        u += run;
      }
    }
    if constexpr (kShared) __syncwarp();  // all lanes have read the entries about to be refilled
    refill(i + DEPTH, grp);
    grp = (grp == ring + (NG - 1) * kGroupBytes) ? ring : grp + kGroupBytes;
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

// Ring geometry shared by the staged ops: entries of `kOperands` feature rows (32*R slots of 16 bytes each) plus
// `kMoreBytes`; the ring holds NG groups of U entries (U = batch).  What a warp may use: one SM's shared memory
// (228 KB, of which every resident block costs 1 KB of its own) over `min_ctas` blocks of kWarpsPerCta warps,
// less the metadata window and `extra` bytes of scratch.
constexpr int ring_budget(int min_ctas, bool uses_eid, int extra) {
  return (228 * 1024 - min_ctas * 1024) / min_ctas / kWarpsPerCta - (kWin * (uses_eid ? 13 : 9) + 15) / 16 * 16 - extra;
}
// Batch: the largest power of two <= umax of which the ring holds at least two groups (so that one group is in
// flight while another is folded); 1 when even that does not fit twice.
constexpr int pick_batch(int edge_bytes, int budget, int umax) {
  for (int u = umax; u > 1; u >>= 1)
    if (2 * u * edge_bytes <= budget) return u;
  return 1;
}
// Groups: as many as fit, at most 4, the look-ahead (NG + 1) * U staying within one metadata block.
constexpr int pick_groups(int edge_bytes, int budget, int u) {
  int ng = budget / (u * edge_bytes);
  const int cap = (kWinBlock - u) / u;
  ng = ng > 4 ? 4 : ng;
  ng = ng > cap ? cap : ng;
  return ng < 1 ? 1 : ng;
}

template <typename T, int R, int kOperands, bool kEid, int kCtasNarrow = GK_CTAS_NARROW, int kExtra = 0,
          int kMoreBytes = 0, int kForceBatch = 0>
struct RingShape {
  using A = typename AccOf<T>::type;
  static constexpr int kRowBytes = 32 * R * 16;
  static constexpr int kEdgeBytes = kOperands * kRowBytes + kMoreBytes;
  // 4-byte elements: 16 bytes of accumulator per slot, 64 registers are enough; 2-byte elements
  // (8 accumulators per slot) and doubles need the 80 registers of 3 resident blocks
  static constexpr int kMinCtas = R == 1 ? (sizeof(T) == 4 ? kCtasNarrow : (kCtasNarrow < 3 ? kCtasNarrow : 3))
                                         : (R == 2 ? 2 : 1);
  static constexpr int kBudget = ring_budget(kMinCtas, kEid, kExtra);
  static constexpr int kBatch = kForceBatch ? kForceBatch : pick_batch(kEdgeBytes, kBudget, R == 1 ? 4 : (R == 2 ? 2 : 1));
  static constexpr int kGroups = pick_groups(kEdgeBytes, kBudget, kBatch);
  static constexpr int kDepth = kGroups * kBatch;
};

// Sum of per-register partial dot products over the lanes of one head, lanes-per-head known at
// compile time (LPH = 1, 2, 4, 8, 16 or 32; LPH = 0: read it from `lph`, any power of two).
template <int LPH, typename A, int R>
__device__ __forceinline__ void reduce_heads_ct(A (&p)[R], int lph) {
  if constexpr (LPH == 0) {
    reduce_heads<A, R>(p, lph);
  } else {
#pragma unroll
    for (int o = 1; o < LPH; o <<= 1)
#pragma unroll
      for (int i = 0; i < R; ++i) p[i] += __shfl_xor_sync(kFull, p[i], o);
  }
}

// Sums U (2 or 4) per-lane partials over the LPH lanes of a head so that lane l ends up holding the total of
// value (l & (U - 1)): exchange steps in which a lane keeps half of its values and hands the other half to its
// partner, then butterfly steps over the remaining lane bits.  For four values log2(LPH) + 1 shuffles instead of
// 4 * log2(LPH); every sum is formed in the order of an ascending butterfly (lane distance 1, 2, 4, ...).
template <int LPH, int U, typename A>
__device__ __forceinline__ A reduce_transposed(const A (&s)[U], int lane) {
  static_assert((U == 2 || U == 4) && LPH >= U && (LPH & (LPH - 1)) == 0, "2 or 4 values, lanes per head a power of two");
  const bool b0 = (lane & 1) != 0;
  A keep;
  if constexpr (U == 4) {
    const bool b1 = (lane & 2) != 0;
    A keep0 = b0 ? s[1] : s[0];
    A keep1 = b0 ? s[3] : s[2];
    const A send0 = b0 ? s[0] : s[1];
    const A send1 = b0 ? s[2] : s[3];
    keep0 += __shfl_xor_sync(kFull, send0, 1);
    keep1 += __shfl_xor_sync(kFull, send1, 1);
    keep = b1 ? keep1 : keep0;
    const A send = b1 ? keep0 : keep1;
    keep += __shfl_xor_sync(kFull, send, 2);
  } else {
    keep = b0 ? s[1] : s[0];
    const A send = b0 ? s[0] : s[1];
    keep += __shfl_xor_sync(kFull, send, 1);
  }
#pragma unroll
  for (int o = U; o < LPH; o <<= 1) keep += __shfl_xor_sync(kFull, keep, o);
  return keep;
}
// Batch size, scratch and lane roles of the ops that reduce with reduce_transposed: rows of one or two 16-byte
// slots per lane (a lane's two slots belong to two heads, 32 / LPH apart), 2 to 32 lanes per head.  Lane l of a head's group owns edge l & (U - 1) of the batch; the first U
// lanes of each group publish their edge's scalar in the warp's scratch, U consecutive values per head.
constexpr int kFastBatch = GK_FAST_BATCH;
constexpr int kFastScratch = 128;  // U values of kAccBytes for each of the 32 R / LPH heads of a row of 32 R slots
template <int R, int LPH, int kAccBytes = 4> struct FastShape {
  static constexpr bool value = (R == 1 || R == 2) && LPH >= kFastBatch &&
                                (LPH == 2 || LPH == 4 || LPH == 8 || LPH == 16 || LPH == 32) &&
                                (32 * R / (LPH ? LPH : 1)) * kFastBatch * kAccBytes <= kFastScratch;
};
template <int U, typename A>
__device__ __forceinline__ void lds_batch(A (&d)[U], const A* p) {
  if constexpr (sizeof(A) * U == 16) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    memcpy(d, &t, 16);
  } else if constexpr (sizeof(A) * U == 8) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    memcpy(d, &t, 8);
  } else {
    const uint4 t0 = reinterpret_cast<const uint4*>(p)[0], t1 = reinterpret_cast<const uint4*>(p)[1];
    memcpy(d, &t0, 16);
    memcpy(reinterpret_cast<unsigned char*>(d) + 16, &t1, 16);
  }
}

#define GK_RING_SLOT(u) (ring + (u) * kEdgeBytes)
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
  // weights: one 4- or 8-byte word per lane and register (2-byte elements travel as the aligned 4-byte word
  // that contains them, except the last element of a tensor with an odd element count, which is read alone)
  using WWord = typename std::conditional<sizeof(T) == 8, double, uint32_t>::type;
  using Ring = RingShape<T, R, 1, true, GK_CTAS_NARROW, 0, 32 * R * (int)sizeof(WWord)>;
  static constexpr int kEdgeBytes = Ring::kEdgeBytes, kDepth = Ring::kDepth, kBatch = Ring::kBatch,
                       kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr bool kUsesEid = true;
  static constexpr bool kSharedEntry = true;  // in the packed modes lanes read weights that other lanes copied
  // How an edge's H weights reach the ring entry (set by the host):
  //   kWeightsPerLane  every lane copies the word of its own head (any H, any element size);
  //   kWeightsWords    lane j < H copies weight j, lanes read the weight of their head (4- and 8-byte
  //                    elements, H <= 32 * R; 2-byte elements with an even H on a 4-byte aligned tensor: lane j
  //                    copies the word that holds weights 2 j and 2 j + 1);
  //   kWeightsPieces   the H weights travel as 16-byte pieces copied by the first lanes (the weight
  //                    row is a whole number of aligned 16-byte pieces).
  // One scattered copy per edge instead of one per lane is what the packed modes buy.
  //   kWeightsHalfWords  2-byte elements otherwise (odd H, or a tensor that is only 2-byte aligned): the first lanes
  //                    copy the aligned 4-byte words that cover the edge's H weights (H / 2 + 1 at most); the row
  //                    starts in the lower or the upper half of the first word, which the readers work out from
  //                    the edge id.
  enum { kWeightsPerLane = 0, kWeightsWords = 1, kWeightsPieces = 2, kWeightsHalfWords = 3 };
  int wmode = kWeightsPerLane;
  // 2-byte elements, per-lane and half-word modes: the two elements whose aligned 4-byte word would reach outside the tensor
  // (the first one when the tensor starts in the upper half of a word, the last one when it ends in the lower
  // half); they are copied alone.  Null when the tensor's ends are word-aligned.
  const T* w_first_alone = nullptr;
  const T* w_last_alone = nullptr;
  __host__ void set_weight_bounds(long long n_elems) {
    if (sizeof(T) != 2 || n_elems <= 0) return;
    const uintptr_t lo = reinterpret_cast<uintptr_t>(this->w), hi = lo + 2 * (uintptr_t)(n_elems - 1);
    w_first_alone = (lo & 2) ? this->w : nullptr;
    w_last_alone = (hi & 2) ? nullptr : this->w + (n_elems - 1);
  }
  __device__ __forceinline__ int mode() const { return kMode >= 0 ? kMode : wmode; }

  __host__ static int pick_wmode(const void* w, int H, int feat0, int HD, int block_elems) {
    const bool whole = feat0 == 0 && HD <= block_elems && H <= 32 * R;  // one feature block sees every head
    if (!whole) return kWeightsPerLane;
    if ((H * sizeof(T)) % 16 == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0) return kWeightsPieces;
    if (sizeof(T) >= 4) return kWeightsWords;
    // 2-byte elements: an even number of heads on a 4-byte aligned tensor is a row of whole aligned words
    return (H % 2 == 0 && (reinterpret_cast<uintptr_t>(w) & 3) == 0) ? kWeightsWords : kWeightsHalfWords;
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
      if (st.sm.ok[i]) cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.xb[i], kEdgeFeat ? e : c, rowb));
      const int j = lane + 32 * i;
      if (mode() == kWeightsPieces) {
        if (j * 16 < wbytes) cp_async16(entry + Ring::kRowBytes + j * 16, wrow + j * 16);
      } else if (mode() == kWeightsWords) {
        if constexpr (sizeof(T) >= 4) {
          if (j < this->H)
            cp_async_small<sizeof(T)>(entry + Ring::kRowBytes + j * sizeof(T), wrow + j * sizeof(T));
        } else {
          if (j * 4 < wbytes) cp_async_small<4>(entry + Ring::kRowBytes + j * 4, wrow + j * 4);  // two weights per word
        }
      } else if (sizeof(T) == 2 && mode() == kWeightsHalfWords) {
        const uintptr_t first = reinterpret_cast<uintptr_t>(wrow);               // the row's first weight
        const uintptr_t a = (first & ~uintptr_t(3)) + 4 * (uintptr_t)j;          // lane j's word
        if (a < first + (uintptr_t)wbytes) {
          WWord* wdst = reinterpret_cast<WWord*>(entry + Ring::kRowBytes) + j;
          // the two words that reach outside the tensor: only their inner half is read
          if (a + 2 == reinterpret_cast<uintptr_t>(w_first_alone))
            reinterpret_cast<uint16_t*>(wdst)[1] = __ldg(reinterpret_cast<const uint16_t*>(a + 2));
          else if (a == reinterpret_cast<uintptr_t>(w_last_alone))
            reinterpret_cast<uint16_t*>(wdst)[0] = __ldg(reinterpret_cast<const uint16_t*>(a));
          else
            cp_async_small<4>(wdst, reinterpret_cast<const void*>(a));
        }
      } else {
        const T* wsrc = this->w + (long long)e * this->H + st.sm.head[i];
        WWord* wdst = reinterpret_cast<WWord*>(entry + Ring::kRowBytes) + lane + 32 * i;
        if constexpr (sizeof(T) == 2) {
          if (wsrc == w_first_alone || wsrc == w_last_alone) {
            const bool up = (reinterpret_cast<uintptr_t>(wsrc) & 2) != 0;
            reinterpret_cast<uint16_t*>(wdst)[up ? 1 : 0] = __ldg(reinterpret_cast<const uint16_t*>(wsrc));
          } else {
            cp_async_small<4>(wdst, reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(wsrc) & ~uintptr_t(3)));
          }
        } else {
          cp_async_small<sizeof(T)>(wdst, wsrc);
        }
      }
    }
  }
  __device__ __forceinline__ void prefetch_node(State&, int, int) const {}
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int cnt,
                                                const int* eids, int lane) const {
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_SLOT(u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        A xv[V];
        lds_acc<T, V>(xv, entry + (lane + 32 * i) * 16);
        A wv;
        if (sizeof(T) == 2 && mode() == kWeightsHalfWords) {
          // the row starts in the upper half of its first word when its first weight's address is odd in elements
          const uintptr_t first = reinterpret_cast<uintptr_t>(this->w) + 2 * (uintptr_t)((long long)eids[u] * this->H);
          wv = to_acc<T>(reinterpret_cast<const T*>(entry + Ring::kRowBytes)[st.sm.head[i] + (int)((first >> 1) & 1)]);
        } else if (mode() != kWeightsPerLane) {
          wv = to_acc<T>(reinterpret_cast<const T*>(entry + Ring::kRowBytes)[st.sm.head[i]]);
        } else if constexpr (sizeof(T) == 2) {
          const WWord word = reinterpret_cast<const WWord*>(entry + Ring::kRowBytes)[lane + 32 * i];
          const bool hi = (reinterpret_cast<uintptr_t>(this->w + (long long)eids[u] * this->H + st.sm.head[i]) & 2) != 0;
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
  // batches of 2 for one-slot rows: measured against 4 (the most the ring would hold) and 1 on R-MAT 21 and Zipf 50M,
  // 5.15 / 6.13 / 5.70 ms and 3.66 / 4.03 / 3.96 ms per step's two launches
  using Ring = RingShape<T, R, 1, true, GK_CTAS_NARROW, 0, 0, R == 1 ? 2 : 0>;
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
    if constexpr (kPrefetch) {
  #pragma unroll
      for (int i = 0; i < R; ++i) load_acc<T, V>(st.an[i], this->a + (long long)node * this->HD + st.sm.feat[i]);
      st.next_node = node;
    }
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
      if (st.sm.ok[i]) cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.bb[i], kEdgeFeat ? e : c, rowb));
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int cnt,
                                                const int* eids, int lane) const {
    A p[kBatch][R];
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_SLOT(u);
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
// kBias: a third row per entry, the edge's row of `rel` laid out slot by slot like the key row (every head's lanes
// copy the same D elements: they come out of L1 / L2), added to the key as it is read back.
template <typename T, int V, int R, int LPH, bool kBias = false>
struct AttnFwdStaged : AttnFwdOp<T, V, R, kBias> {
  using Base = AttnFwdOp<T, V, R, kBias>;
  using A = typename Base::A;
  struct State : Base::State {
    A qn[R][V]; int next_node; const unsigned char* kb[R]; const unsigned char* vb[R]; const unsigned char* rb[R];
    unsigned char* scratch;
  };
  // the next node\'s resident rows are fetched ahead only while they fit 16 bytes per lane: wider rows need
  // the registers for the node being processed
  static constexpr bool kPrefetch = R * V * (int)sizeof(A) <= 16;
  using CarryIn = typename Base::CarryIn;
  static constexpr bool kFast = FastShape<R, LPH, (int)sizeof(A)>::value;
  using Ring = RingShape<T, R, kBias ? 3 : 2, kBias, GK_CTAS_NARROW, kFastScratch, 0, kFast ? kFastBatch : 0>;
  static constexpr int kEdgeBytes = Ring::kEdgeBytes, kDepth = Ring::kDepth, kBatch = Ring::kBatch,
                       kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr int kScratchBytes = kFast ? kFastScratch : 0;
  static constexpr bool kUsesEid = kBias;   // the edge term is indexed by edge id (the position, without an eid array)

  __device__ __forceinline__ void setup(State& st, int lane) const {
    Base::setup(st, lane);
    st.next_node = -1;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.kb[i] = reinterpret_cast<const unsigned char*>(this->k + st.sm.feat[i]);
      st.vb[i] = reinterpret_cast<const unsigned char*>(this->v + st.sm.feat[i]);
      st.rb[i] = kBias ? reinterpret_cast<const unsigned char*>(this->rel + st.sm.efeat[i]) : nullptr;
    }
  }
  // the key slot of a ring entry, with the edge term added when there is one
  __device__ __forceinline__ void load_key(A (&kv)[V], const unsigned char* entry, int slot) const {
    lds_acc<T, V>(kv, entry + slot * 16);
    if constexpr (kBias) {
      A rv[V];
      lds_acc<T, V>(rv, entry + 2 * Ring::kRowBytes + slot * 16);
#pragma unroll
      for (int e = 0; e < V; ++e) kv[e] += rv[e];
    }
  }
  __device__ __forceinline__ void prefetch_node(State& st, int node, int) const {
    if constexpr (kPrefetch) {
  #pragma unroll
      for (int i = 0; i < R; ++i) load_acc<T, V>(st.qn[i], this->q + (long long)node * this->HD + st.sm.feat[i]);
      st.next_node = node;
    }
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
  __device__ __forceinline__ void stage(const State& st, unsigned char* entry, int c, int edge, int lane) const {
    const unsigned rowb = (unsigned)this->HD * (unsigned)sizeof(T);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (!st.sm.ok[i]) continue;
      cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.kb[i], c, rowb));
      cp_async16(entry + Ring::kRowBytes + (lane + 32 * i) * 16, row_ptr(st.vb[i], c, rowb));
      if constexpr (kBias)
        cp_async16(entry + 2 * Ring::kRowBytes + (lane + 32 * i) * 16,
                   row_ptr(st.rb[i], edge, (unsigned)this->D * (unsigned)sizeof(T)));
    }
  }
  // Batch of U = 2 or 4 with one 16-byte slot per lane: the U partial dot products of a lane are reduced
  // "transposed" (lane l of the head ends up with the score of edge l & (U - 1)), the scores travel to the head's
  // other lanes through the warp's scratch, and every lane then forms the U probabilities itself.
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_fast(State& st, const unsigned char* ring, int cnt, int lane) const {
    constexpr int U = kFastBatch;
    A s[R][U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int i = 0; i < R; ++i) {
        s[i][u] = A(0);
        if (kFullBatch || u < cnt) {  // a partial batch may end at the ring's last entry: nothing is read past it
          A kv[V];
          load_key(kv, GK_RING_SLOT(u), lane + 32 * i);
          s[i][u] = st.q[i][0] * kv[0];
#pragma unroll
          for (int e = 1; e < V; ++e) s[i][u] += st.q[i][e] * kv[e];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
      A mine = reduce_transposed<LPH, U, A>(s[i], lane);
      if (!kFullBatch && (lane & (U - 1)) >= cnt) mine = neg_inf<A>();  // positions past the batch: probability 0
      A* sc = reinterpret_cast<A*>(st.scratch) + ((lane + 32 * i) / LPH) * U;
      if ((lane & (LPH - 1)) < U) sc[lane & (U - 1)] = mine;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < R; ++i) {
      A sv[U];
      lds_batch<U, A>(sv, reinterpret_cast<const A*>(st.scratch) + ((lane + 32 * i) / LPH) * U);
      A mn = st.m[i];
#pragma unroll
      for (int u = 0; u < U; ++u) mn = sv[u] > mn ? sv[u] : mn;
      const A corr = gk_exp2(st.m[i] - mn);  // m = -inf at a node's first batch: 2^-inf = 0
      A p[U];
      A psum = A(0);
#pragma unroll
      for (int u = 0; u < U; ++u) { p[u] = gk_exp2(sv[u] - mn); psum += p[u]; }
      st.m[i] = mn;
      st.l[i] = st.l[i] * corr + psum;
#pragma unroll
      for (int e = 0; e < V; ++e) st.acc[i][e] *= corr;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (kFullBatch || u < cnt) {
          A vv[V];
          lds_acc<T, V>(vv, GK_RING_SLOT(u) + Ring::kRowBytes + (lane + 32 * i) * 16);
#pragma unroll
          for (int e = 0; e < V; ++e) st.acc[i][e] += p[u] * vv[e];
        }
      }
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int cnt, const int*,
                                                int lane) const {
    if constexpr (kFast) consume_fast<kFullBatch>(st, ring, cnt, lane);
    else consume_slow<kFullBatch>(st, ring, cnt, lane);
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_slow(State& st, const unsigned char* ring, int cnt, int lane) const {
    A s[kBatch][R];
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_SLOT(u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        A kv[V];
        load_key(kv, entry, lane + 32 * i);
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
      const unsigned char* entry = GK_RING_SLOT(u) + Ring::kRowBytes;
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
template <typename T, int V, int R, int LPH, bool kBias = false>
struct AttnBwdDstStaged : AttnBwdDstOp<T, V, R, kBias> {
  using Base = AttnBwdDstOp<T, V, R, kBias>;
  using A = typename Base::A;
  struct State : Base::State {
    A qn[R][V]; A gn[R][V]; A on[R][V]; A lsen[R]; int next_node; int tile_base; int batch_pos;
    const unsigned char* kb[R]; const unsigned char* vb[R]; const unsigned char* rb[R];
    unsigned char* pdw[R];  // where this lane writes its head's (p, ds) of edge 0, or null: not a writer
    unsigned char* scratch;
  };
  static constexpr bool kTileBase = true;
  EdgePair<A>* __restrict__ pd = nullptr;  // (n_edges, Hp) out when not null: (p, ds) of every edge, by position
  // the next node\'s resident rows are fetched ahead only while they fit 16 bytes per lane: wider rows need
  // the registers for the node being processed
  static constexpr bool kPrefetch = R * V * (int)sizeof(A) <= 16;
  static constexpr bool kFast = FastShape<R, LPH, (int)sizeof(A)>::value;
  using Ring = RingShape<T, R, kBias ? 3 : 2, kBias, GK_CTAS_DST, kFastScratch, 0, kFast ? kFastBatch : 0>;
  static constexpr int kEdgeBytes = Ring::kEdgeBytes, kDepth = Ring::kDepth, kBatch = Ring::kBatch,
                       kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr int kScratchBytes = kFast ? kFastScratch : 0;
  static constexpr bool kUsesEid = kBias;   // the edge term (see AttnFwdStaged) is indexed by edge id
  static constexpr bool kNodeRows = true;

  // the key slot of a ring entry, with the edge term added when there is one (dq sums ds * (k + rel))
  __device__ __forceinline__ void load_key(A (&kv)[V], const unsigned char* entry, int slot) const {
    lds_acc<T, V>(kv, entry + slot * 16);
    if constexpr (kBias) {
      A rv[V];
      lds_acc<T, V>(rv, entry + 2 * Ring::kRowBytes + slot * 16);
#pragma unroll
      for (int e = 0; e < V; ++e) kv[e] += rv[e];
    }
  }

  __device__ __forceinline__ void prefetch_rows_l2(int node) const {
    const unsigned rowb = (unsigned)this->HD * (unsigned)sizeof(T);
    const long long at = (long long)node * this->HD;
    prefetch_row_l2(this->q + at, rowb);
    prefetch_row_l2(this->dout + at, rowb);
    prefetch_row_l2(this->o + at, rowb);
    prefetch_l2(this->lse + (long long)node * this->H);
  }
  __device__ __forceinline__ void setup(State& st, int lane) const {
    Base::setup(st, lane);
    st.next_node = -1;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.kb[i] = reinterpret_cast<const unsigned char*>(this->k + st.sm.feat[i]);
      st.vb[i] = reinterpret_cast<const unsigned char*>(this->v + st.sm.feat[i]);
      st.rb[i] = kBias ? reinterpret_cast<const unsigned char*>(this->rel + st.sm.efeat[i]) : nullptr;
      // the slow path writes a head's pair from the lane that holds the head's first slot; the fast path from
      // the first U lanes of the head's group, lane j writing edge j of the batch
      const bool writer = kFast ? (lane & (LPH - 1)) < kFastBatch : st.sm.efeat[i] == 0;
      st.pdw[i] = (pd && st.sm.ok[i] && writer)
                      ? reinterpret_cast<unsigned char*>(pd + st.sm.head[i]) +
                            (kFast ? (size_t)(lane & (kFastBatch - 1)) * (size_t)this->Hp * sizeof(EdgePair<A>) : (size_t)0)
                      : nullptr;
    }
  }
  // Batch of U = 2 or 4, one 16-byte slot per lane: q.k and dO.v of the U edges are reduced transposed, so lane l
  // of a head holds both sums of edge l & (U - 1) and forms that edge's p and ds alone (one ex2 per lane and
  // batch); the first U lanes of the head store the pairs (consecutive positions, consecutive heads: whole
  // 32-byte sectors) and publish ds in the warp's scratch for the accumulation of dq.
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_fast(State& st, const unsigned char* ring, int cnt, int lane) const {
    constexpr int U = kFastBatch;
    A s[R][U], dp[R][U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int i = 0; i < R; ++i) {
        s[i][u] = A(0);
        dp[i][u] = A(0);
        if (kFullBatch || u < cnt) {  // a partial batch may end at the ring's last entry: nothing is read past it
          const unsigned char* entry = GK_RING_SLOT(u);
          A kv[V], vv[V];
          load_key(kv, entry, lane + 32 * i);
          lds_acc<T, V>(vv, entry + Ring::kRowBytes + (lane + 32 * i) * 16);
          s[i][u] = st.q[i][0] * kv[0];
          dp[i][u] = st.g[i][0] * vv[0];
#pragma unroll
          for (int e = 1; e < V; ++e) { s[i][u] += st.q[i][e] * kv[e]; dp[i][u] += st.g[i][e] * vv[e]; }
        }
      }
    }
    const bool live = kFullBatch || (lane & (U - 1)) < cnt;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const A s_mine = reduce_transposed<LPH, U, A>(s[i], lane);
      const A dp_mine = reduce_transposed<LPH, U, A>(dp[i], lane);
      const A p = gk_exp2(s_mine - st.lse[i]);
      A ds = p * (dp_mine - st.delta[i]) * this->scale;
      if (!live) ds = A(0);
      if (st.pdw[i] && live) {
        const unsigned pairb = (unsigned)this->Hp * (unsigned)sizeof(EdgePair<A>);
        *reinterpret_cast<EdgePair<A>*>(st.pdw[i] + (unsigned long long)(unsigned)(st.tile_base + st.batch_pos) * pairb) =
            EdgePair<A>{p, ds};
      }
      A* sc = reinterpret_cast<A*>(st.scratch) + ((lane + 32 * i) / LPH) * U;
      if ((lane & (LPH - 1)) < U) sc[lane & (U - 1)] = ds;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < R; ++i) {
      A dsv[U];
      lds_batch<U, A>(dsv, reinterpret_cast<const A*>(st.scratch) + ((lane + 32 * i) / LPH) * U);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (kFullBatch || u < cnt) {
          A kv[V];
          load_key(kv, GK_RING_SLOT(u), lane + 32 * i);
#pragma unroll
          for (int e = 0; e < V; ++e) st.acc[i][e] += dsv[u] * kv[e];
        }
      }
    }
  }
  __device__ __forceinline__ void prefetch_node(State& st, int node, int) const {
    if constexpr (kPrefetch) {
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
      // the fast path sums dO.v in the ascending order: delta the same way, so that a node with a single edge
      // gets dp - delta = 0 exactly
      if constexpr (kFast) {
#pragma unroll
        for (int i = 0; i < R; ++i) dl[i] = reduce_ascending<LPH, A>(dl[i]);
      } else {
        reduce_heads_ct<LPH, A, R>(dl, this->lph);
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
        st.delta[i] = dl[i];
        if (st.sm.ok[i] && st.sm.efeat[i] == 0)
          this->stat[(long long)node * this->Hp + st.sm.head[i]] = StatPair<A>{st.lsen[i], dl[i]};
      }
      return;
    }
    Base::template begin_ordered<(kFast ? LPH : 0)>(st, node, lane);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      st.lse[i] *= A(kLog2e);
#pragma unroll
      for (int e = 0; e < V; ++e) st.q[i][e] *= c;
    }
  }
  __device__ __forceinline__ void stage(const State& st, unsigned char* entry, int c, int edge, int lane) const {
    const unsigned rowb = (unsigned)this->HD * (unsigned)sizeof(T);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      if (!st.sm.ok[i]) continue;
      cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.kb[i], c, rowb));
      cp_async16(entry + Ring::kRowBytes + (lane + 32 * i) * 16, row_ptr(st.vb[i], c, rowb));
      if constexpr (kBias)
        cp_async16(entry + 2 * Ring::kRowBytes + (lane + 32 * i) * 16,
                   row_ptr(st.rb[i], edge, (unsigned)this->D * (unsigned)sizeof(T)));
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int cnt, const int*,
                                                int lane) const {
    if constexpr (kFast) consume_fast<kFullBatch>(st, ring, cnt, lane);
    else consume_slow<kFullBatch>(st, ring, cnt, lane);
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_slow(State& st, const unsigned char* ring, int cnt, int lane) const {
    const unsigned pairb = (unsigned)this->Hp * (unsigned)sizeof(EdgePair<A>);
    A s[kBatch][R], dp[kBatch][R];
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_SLOT(u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        A kv[V], vv[V];
        load_key(kv, entry, lane + 32 * i);
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
      const unsigned char* entry = GK_RING_SLOT(u);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const A p = gk_exp2(s[u][i] - st.lse[i]);
        const A ds = p * (dp[u][i] - st.delta[i]) * this->scale;
        if (st.pdw[i])
          *reinterpret_cast<EdgePair<A>*>(st.pdw[i] + (unsigned long long)(unsigned)(st.tile_base + st.batch_pos + u) * pairb) =
              EdgePair<A>{p, ds};
        A kv[V];
        load_key(kv, entry, lane + 32 * i);
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
  // (lse, delta) pairs of the most heads this instantiation can see: 32 * R / LPH (every head when the
  // lanes per head are only known at run time), at least one 16-byte piece
  static constexpr int kMaxHeads = LPH ? (32 * R / LPH > 2 ? 32 * R / LPH : 2) : 32 * R;
  static constexpr int kPairBytes = (kMaxHeads * (int)sizeof(StatPair<A>) + 15) / 16 * 16;
  using Ring = RingShape<T, R, 2, false, 3, 0, kPairBytes, R == 1 ? 2 : 0>;
  static constexpr int kEdgeBytes = Ring::kEdgeBytes, kDepth = Ring::kDepth, kBatch = Ring::kBatch,
                       kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
  static constexpr bool kUsesEid = false;
  static constexpr bool kSharedEntry = true;  // lanes read pair bytes that other lanes copied

  __device__ __forceinline__ void setup(State& st, int lane) const { Base::setup(st, lane); st.next_node = -1; }
  __device__ __forceinline__ void prefetch_node(State& st, int node, int) const {
    if constexpr (kPrefetch) {
  #pragma unroll
      for (int i = 0; i < R; ++i) {
        const long long off = (long long)node * this->HD + st.sm.feat[i];
        load_acc<T, V>(st.kn[i], this->k + off);
        load_acc<T, V>(st.vn[i], this->v + off);
      }
      st.next_node = node;
    }
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
      if (st.sm.ok[i]) {
        cp_async16(entry + (lane + 32 * i) * 16, this->q + (long long)c * this->HD + st.sm.feat[i]);
        cp_async16(entry + Ring::kRowBytes + (lane + 32 * i) * 16,
                   this->dout + (long long)c * this->HD + st.sm.feat[i]);
      }
      const int piece = lane + 32 * i;
      if (piece < pieces) cp_async16(entry + 2 * Ring::kRowBytes + piece * 16, pairs + piece * 16);
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int cnt, const int*,
                                                int lane) const {
    A s[kBatch][R], dp[kBatch][R];
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_SLOT(u);
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
      const unsigned char* entry = GK_RING_SLOT(u);
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
  static constexpr int kMaxHeads = LPH ? (32 * R / LPH > 2 ? 32 * R / LPH : 2) : 32 * R;
  static constexpr int kPairBytes = (kMaxHeads * (int)sizeof(EdgePair<A>) + 15) / 16 * 16;
  using Ring = RingShape<T, R, 2, true, GK_CTAS_SRC, 0, kPairBytes>;
  static constexpr int kEdgeBytes = Ring::kEdgeBytes, kDepth = Ring::kDepth, kBatch = Ring::kBatch,
                       kMinCtas = Ring::kMinCtas, kWarps = kWarpsPerCta;
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
      if (st.sm.ok[i]) {
        cp_async16(entry + (lane + 32 * i) * 16, row_ptr(st.qb[i], c, rowb));
        cp_async16(entry + Ring::kRowBytes + (lane + 32 * i) * 16, row_ptr(st.gb[i], c, rowb));
      }
      const int piece = lane + 32 * i;
      if (piece < pieces) cp_async16(entry + 2 * Ring::kRowBytes + piece * 16, pairs + piece * 16);
    }
  }
  template <bool kFullBatch>
  __device__ __forceinline__ void consume_batch(State& st, const unsigned char* ring, int cnt, const int*,
                                                int lane) const {
    GK_BATCH_LOOP(u) {
      const unsigned char* entry = GK_RING_SLOT(u);
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
