// Host side of the C ABI: argument checks, workspace carving, kernel selection and the
// launch sequences.  Everything here enqueues on the caller's stream and never synchronises.
#pragma once
#include <atomic>
#include <cstdio>
#include <mutex>
#include <type_traits>
#include <utility>
#include <vector>

#include "../../include/graphop_b200.h"
#include "gk_common.cuh"
#include "gk_ops.cuh"
#include "gk_softmax.cuh"
#include "gk_staged.cuh"

namespace gk {

inline thread_local int g_last_cuda_error = 0;

#define GK_CUDA(expr)                                   \
  do {                                                  \
    cudaError_t err__ = (expr);                         \
    if (err__ != cudaSuccess) {                         \
      gk::g_last_cuda_error = (int)err__;                 \
      return GRAPHOP_ERR_CUDA;                          \
    }                                                   \
  } while (0)
#define GK_LAUNCH_CHECK() GK_CUDA(cudaGetLastError())

// Every kernel launch of the library goes through GK_LAUNCHED(name), which checks the launch.  The benchmark's
// instrumented twin of the library (compiled with -DGK_BENCH_HOOKS, see csrc/bench/) also counts the launch and,
// while a profile is open, records a CUDA event behind the kernel on the caller's stream, so that the time
// between two consecutive events is the device time of the later kernel.  The product library has none of it.
#ifdef GK_BENCH_HOOKS
struct Profiler {
  std::mutex lock;   // autograd runs the backward ops on another host thread
  bool enabled = false;
  long long launches = 0;
  std::vector<std::pair<const char*, cudaEvent_t>> marks;
};
inline Profiler& profiler() {
  static Profiler p;
  return p;
}
inline void mark(const char* name, cudaStream_t st) {
  Profiler& p = profiler();
  std::lock_guard<std::mutex> hold(p.lock);
  ++p.launches;
  if (p.enabled) {
    cudaEvent_t e;
    if (cudaEventCreate(&e) == cudaSuccess) {
      cudaEventRecord(e, st);
      p.marks.emplace_back(name, e);
    }
  }
}
#define GK_LAUNCHED(name)  \
  do {                     \
    GK_LAUNCH_CHECK();     \
    gk::mark(name, st);    \
  } while (0)
#else
#define GK_LAUNCHED(name) GK_LAUNCH_CHECK()
#endif
#define GK_TRY(expr)                    \
  do {                                  \
    int rc__ = (expr);                  \
    if (rc__ != GRAPHOP_OK) return rc__; \
  } while (0)

constexpr size_t kAlign = 256;
inline size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// Bump allocator over the caller's workspace.  With base == nullptr it only measures.
struct Arena {
  char* base;
  size_t cap, used = 0;
  bool overflow = false;
  Arena(void* b, size_t c) : base((char*)b), cap(c) {}
  void* take(size_t bytes) {
    const size_t at = used;
    used += align_up(bytes ? bytes : 1);
    if (!base) return nullptr;
    if (used > cap) { overflow = true; return nullptr; }
    return base + at;
  }
};

// ---------------------------------------------------------------------------------------
// tiling
// ---------------------------------------------------------------------------------------
constexpr int kCarryTile = 32;  // wider tiles on the short upper levels save a launch but run slower: a warp
                                // walks its slots one after the other (ER-small 0.27 -> 0.40 ms with 256)
constexpr int kMaxLevels = 12;

// Positions per warp at level 0: small graphs get small tiles so that every SM has work,
// large graphs get 256 so that carries stay a fraction of a percent of the traffic.
inline int pick_tile(long long n_edges) {
  long long t = 32;
  while (t < GK_TILE && n_edges / t > 16384) t <<= 1;
  return (int)t;
}

struct Levels {
  int n = 0;
  long long len[kMaxLevels];
  int tile[kMaxLevels];
  long long ntiles[kMaxLevels];
};
inline Levels make_levels(long long n_edges, int tile0) {
  Levels lv;
  long long len = n_edges;
  int tile = tile0;
  for (;;) {
    const long long nt = (len + tile - 1) / tile;
    lv.len[lv.n] = len; lv.tile[lv.n] = tile; lv.ntiles[lv.n] = nt;
    ++lv.n;
    if (nt <= 1 || lv.n == kMaxLevels) break;
    len = 2 * nt;
    tile = kCarryTile;
  }
  return lv;
}

inline unsigned grid_for_warps(long long warps, int warps_per_cta) {
  long long g = (warps + warps_per_cta - 1) / warps_per_cta;
  return (unsigned)(g < 1 ? 1 : g);
}

// ---------------------------------------------------------------------------------------
// graph preparation: erow[] and 32-bit index arrays
// ---------------------------------------------------------------------------------------
struct GraphView {
  const PlanHeader* hdr;
  const int32_t* erow;
  const int32_t* other;  // may be null (ops without a second endpoint)
  const int32_t* eid;    // may be null: identity
  long long E;
  // from a plan: boundaries of the level-0 tiles moved up to row starts (for tiles of `start_tile` positions), and
  // whether no row crosses a boundary any more (then there is nothing for the carry levels to do)
  const int32_t* tile_start = nullptr;
  int start_tile = 0;
  bool no_carry = false;
  const int32_t* starts_for(int tile) const { return tile == start_tile ? tile_start : nullptr; }
};

template <typename I>
inline int prepare_graph(Arena& ar, const I* row, const I* indptr, const I* eid, const I* indices, long long C,
                         long long E, cudaStream_t st, GraphView* g) {
  auto* hdr = (PlanHeader*)ar.take(sizeof(PlanHeader));
  auto* erow = (int32_t*)ar.take((size_t)E * 4);
  int32_t* other32 = nullptr;
  int32_t* eid32 = nullptr;
  if (sizeof(I) == 8) {
    if (indices) other32 = (int32_t*)ar.take((size_t)E * 4);
    if (eid) eid32 = (int32_t*)ar.take((size_t)E * 4);
  }
  if (!ar.base) return GRAPHOP_OK;
  if (ar.overflow) return GRAPHOP_ERR_WORKSPACE;
  const long long warps = (E + kExpandTile - 1) / kExpandTile;
  expand_rows_kernel<I><<<grid_for_warps(warps, kWarpsPerCta), kWarpsPerCta * 32, 0, st>>>(row, indptr, C, E, erow, hdr);
  GK_LAUNCHED("expand_rows");
  g->hdr = hdr;
  g->erow = erow;
  g->E = E;
  if (sizeof(I) == 8) {
    const unsigned grid = (unsigned)((E + 1023) / 1024 < 4096 ? (E + 1023) / 1024 : 4096);
    if (indices) {
      narrow_index_kernel<I><<<grid ? grid : 1, 256, 0, st>>>(indices, other32, E);
      GK_LAUNCHED("narrow_index");
    }
    if (eid) {
      narrow_index_kernel<I><<<grid ? grid : 1, 256, 0, st>>>(eid, eid32, E);
      GK_LAUNCHED("narrow_index");
    }
    g->other = other32;
    g->eid = eid32;
  } else {
    g->other = (const int32_t*)indices;
    g->eid = (const int32_t*)eid;
  }
  return GRAPHOP_OK;
}

// Where an op's GraphView comes from: expanded on the spot from the caller's chunk table (into the workspace), or
// taken from a plan that graphop_plan_build_* made once for the graph.
template <typename I>
struct FromChunks {
  const I* row; const I* indptr; const I* eid; const I* indices; long long C, E;
  bool valid(bool need_indices) const { return row && indptr && (!need_indices || indices); }
  int operator()(Arena& ar, cudaStream_t st, GraphView* g) const {
    return prepare_graph<I>(ar, row, indptr, eid, indices, C, E, st, g);
  }
};
struct FromPlan {
  const graphop_plan_t* p;
  bool valid(bool need_indices) const { return p && p->erow && p->header && (!need_indices || p->other); }
  int operator()(Arena&, cudaStream_t, GraphView* g) const {
    g->hdr = (const PlanHeader*)p->header;
    g->erow = p->erow;
    g->other = p->other;
    g->eid = p->eid;
    g->E = p->n_edges;
    if ((p->flags & GRAPHOP_PLAN_ROW_TILES) && p->tile_start) {
      g->tile_start = p->tile_start;
      g->start_tile = p->tile;
      g->no_carry = (p->flags & GRAPHOP_PLAN_NO_CARRY) != 0;
    }
    return GRAPHOP_OK;
  }
};

inline int zero_uncovered(const GraphView& g, void* out, size_t bytes, cudaStream_t st) {
  const long long words = (long long)(bytes / 4);
  if (words == 0) return GRAPHOP_OK;
  const unsigned grid = (unsigned)((words + 1023) / 1024 < 2048 ? (words + 1023) / 1024 : 2048);
  zero_uncovered_kernel<uint32_t><<<grid, 256, 0, st>>>(g.hdr, g.E, (uint32_t*)out, words);
  GK_LAUNCHED("zero_uncovered");
  return GRAPHOP_OK;
}

// ---------------------------------------------------------------------------------------
// vector shape selection
// ---------------------------------------------------------------------------------------
template <typename T> struct VecMax { static constexpr int value = 16 / (int)sizeof(T); };

inline bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
inline bool is_pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }

struct VecShape { int V, R, S; };
// V elements per slot and R slots per lane for an H*D row; R = 0: does not fit 8 slots per lane.
template <typename T>
inline VecShape pick_shape(int HD, int D, bool all_aligned) {
  VecShape s;
  constexpr int VM = VecMax<T>::value;
  s.V = (all_aligned && D % VM == 0) ? VM : 1;
  s.S = HD / s.V;
  if (s.V == 1) s.R = s.S <= 256 ? 8 : 0;
  else s.R = s.S <= 32 ? 1 : s.S <= 64 ? 2 : s.S <= 128 ? 4 : s.S <= 256 ? 8 : 0;
  return s;
}

// Calls f(integral_constant<int,V>, integral_constant<int,R>) for the instantiated pairs.
template <typename T, class F>
inline int dispatch_shape(const VecShape& s, F&& f) {
  constexpr int VM = VecMax<T>::value;
  using std::integral_constant;
  if (s.V == 1 && s.R == 8) return f(integral_constant<int, 1>{}, integral_constant<int, 8>{});
  if (s.V == VM) {
    switch (s.R) {
      case 1: return f(integral_constant<int, VM>{}, integral_constant<int, 1>{});
      case 2: return f(integral_constant<int, VM>{}, integral_constant<int, 2>{});
      case 4: return f(integral_constant<int, VM>{}, integral_constant<int, 4>{});
      case 8: return f(integral_constant<int, VM>{}, integral_constant<int, 8>{});
    }
  }
  return GRAPHOP_ERR_UNSUPPORTED;
}

// Calls f(integral_constant<int, LPH>) with the compile-time lanes-per-head the staged dot-product
// ops are specialised for (2 to 32), or 0 for "read it at run time".
template <class F>
inline int dispatch_lph(int lph, F&& f) {
  using std::integral_constant;
  switch (lph) {
    case 2: return f(integral_constant<int, 2>{});
    case 4: return f(integral_constant<int, 4>{});
    case 8: return f(integral_constant<int, 8>{});
    case 16: return f(integral_constant<int, 16>{});
    case 32: return f(integral_constant<int, 32>{});
    default: return f(integral_constant<int, 0>{});
  }
}

// ---------------------------------------------------------------------------------------
// level-0 + carry-level launch sequence of a row-producing op
// ---------------------------------------------------------------------------------------
template <class Op>
inline size_t staged_smem_bytes() {
  return (size_t)Op::kWarps * staged_warp_bytes<Op>();
}

// Launches the staged level-0 walker; raises the kernel's dynamic shared memory limit once per device.
template <class Op>
inline int launch_staged(const Op& op, const GraphView& g, int tile, long long n_rows, int32_t* rows_next,
                         cudaStream_t st) {
  // one flag per device and kernel; several host threads may get here at once (autograd's backward thread):
  // setting the attribute twice is harmless, the flag only saves the call
  static std::atomic<bool> configured[64];
  int dev = 0;
  GK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    GK_CUDA(cudaFuncSetAttribute(walk_staged_kernel<Op>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)staged_smem_bytes<Op>()));
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  const long long nt = (g.E + tile - 1) / tile;
  walk_staged_kernel<Op><<<grid_for_warps(nt, Op::kWarps), Op::kWarps * 32, staged_smem_bytes<Op>(), st>>>(
      op, g.hdr, g.erow, g.other, g.eid, g.E, tile, n_rows, rows_next, g.starts_for(tile));
  GK_LAUNCHED(Op::kName);
  return GRAPHOP_OK;
}

template <class X> struct TypeTag { using type = X; };
template <class Op, class = void> struct IsStaged : std::false_type {};
template <class Op> struct IsStaged<Op, std::void_t<decltype(Op::kEdgeBytes)>> : std::true_type {};

// `make_op(carry_out, carry_in)` returns the op bound to one level's carry buffers; `make_op0`
// does the same for level 0 when that level runs a different (staged) op that writes the same
// carry format.
template <class MakeOp, class MakeOp0>
inline int run_row_levels(Arena& ar, const GraphView& g, int tile0, long long n_rows, size_t carry_elem_bytes,
                          long long carry_stride, cudaStream_t st, MakeOp&& make_op, MakeOp0&& make_op0) {
  Levels lv = make_levels(g.E, tile0);
  if (g.no_carry && g.starts_for(tile0)) lv.n = 1;   // row-aligned tiles that no row crosses: level 0 stores every row
  void* carry[kMaxLevels];
  int32_t* rows[kMaxLevels + 1];
  rows[0] = nullptr;
  for (int k = 0; k < lv.n; ++k) {
    const bool last = k == lv.n - 1;
    carry[k] = last ? nullptr : ar.take((size_t)(2 * lv.ntiles[k]) * carry_stride * carry_elem_bytes);
    rows[k + 1] = last ? nullptr : (int32_t*)ar.take((size_t)(2 * lv.ntiles[k]) * 4);
  }
  if (!ar.base) return GRAPHOP_OK;
  if (ar.overflow) return GRAPHOP_ERR_WORKSPACE;
  {
    auto op = make_op0(carry[0], nullptr);
    using Op = decltype(op);
    if constexpr (IsStaged<Op>::value) {
      GK_TRY(launch_staged(op, g, lv.tile[0], n_rows, rows[1], st));
    } else {
      walk_kernel<Op, false><<<grid_for_warps(lv.ntiles[0], kWarpsPerCta), kWarpsPerCta * 32, 0, st>>>(
          op, g.hdr, g.erow, g.other, g.eid, g.E, lv.tile[0], n_rows, rows[1], g.starts_for(lv.tile[0]));
      GK_LAUNCHED(Op::kName);
    }
  }
  for (int k = 1; k < lv.n; ++k) {
    auto op = make_op(carry[k], carry[k - 1]);
    using Op = decltype(op);
    walk_kernel<Op, true><<<grid_for_warps(lv.ntiles[k], kWarpsPerCta), kWarpsPerCta * 32, 0, st>>>(
        op, g.hdr, rows[k], nullptr, nullptr, lv.len[k], lv.tile[k], n_rows, rows[k + 1], nullptr);
    GK_LAUNCHED("carry_level");
  }
  return GRAPHOP_OK;
}
template <class MakeOp>
inline int run_row_levels(Arena& ar, const GraphView& g, int tile0, long long n_rows, size_t carry_elem_bytes,
                          long long carry_stride, cudaStream_t st, MakeOp&& make_op) {
  return run_row_levels(ar, g, tile0, n_rows, carry_elem_bytes, carry_stride, st, make_op, make_op);
}

// out[node] = sum_k w[eid[k]] * feat(k): picks the vector shape, splits very wide rows into
// feature blocks of 256 slots (each block is an independent aggregation).
template <typename T, bool kEdgeFeat>
inline int run_aggregate(Arena& ar, const GraphView& g, const T* w, const T* x, T* y, long long n_rows, int H, int D,
                         cudaStream_t st) {
  using A = typename AccOf<T>::type;
  const int HD = H * D;
  const bool al = aligned16(x) && aligned16(y);
  VecShape s = pick_shape<T>(HD, D, al);
  const int tile0 = pick_tile(g.E);
  const int block_elems = 256 * s.V;  // widest register-resident block
  for (int feat0 = 0; feat0 < HD; feat0 += block_elems) {
    const int elems = HD - feat0 < block_elems ? HD - feat0 : block_elems;
    VecShape b = s;
    b.S = elems / s.V;
    if (s.V == 1) b.R = 8;
    else b.R = b.S <= 32 ? 1 : b.S <= 64 ? 2 : b.S <= 128 ? 4 : 8;
    const size_t mark = ar.used;
    GK_TRY((dispatch_shape<T>(b, [&](auto Vc, auto Rc) -> int {
      constexpr int V = decltype(Vc)::value, R = decltype(Rc)::value;
      using OpT = typename std::conditional<(V > 1 || sizeof(T) == 16), AggregateStaged<T, V, R, kEdgeFeat>,
                                            AggregateOp<T, V, R, kEdgeFeat>>::type;
      int wm = 0;
      if constexpr (IsStaged<OpT>::value) wm = OpT::pick_wmode(w, H, feat0, HD, block_elems);
      auto run = [&](auto op_type) -> int {
        using OpM = typename decltype(op_type)::type;
        return run_row_levels(ar, g, tile0, n_rows, sizeof(A), HD, st, [&](void* cout, void* cin) {
          OpM op;
          op.w = w; op.x = x; op.y = y; op.carry = (A*)cout; op.carry_in = (const A*)cin;
          op.H = H; op.D = D; op.HD = HD; op.S = b.S; op.feat0 = feat0;
          if constexpr (IsStaged<OpM>::value) { op.wmode = wm; op.set_weight_bounds((long long)g.E * H); }
          return op;
        });
      };
      if constexpr (IsStaged<OpT>::value) {
        // the packed modes get their own instantiations; the per-lane mode keeps the run-time test
        using Pieces = AggregateStaged<T, V, R, kEdgeFeat, OpT::kWeightsPieces>;
        using Words = AggregateStaged<T, V, R, kEdgeFeat, OpT::kWeightsWords>;
        if (wm == OpT::kWeightsPieces) return run(TypeTag<Pieces>{});
        if (wm == OpT::kWeightsWords) return run(TypeTag<Words>{});
        if constexpr (sizeof(T) == 2) {
          using Half = AggregateStaged<T, V, R, kEdgeFeat, OpT::kWeightsHalfWords>;
          if (wm == OpT::kWeightsHalfWords) return run(TypeTag<Half>{});
        }
      }
      return run(TypeTag<OpT>{});
    })));
    if (feat0 + block_elems < HD) ar.used = mark;  // blocks run back to back on one stream: reuse the scratch
  }
  return GRAPHOP_OK;
}

// y[eid[k], h] = a[node(k), h, :] . feat(k)[h, :]
template <typename T, bool kEdgeFeat>
inline int run_edge_dot(const GraphView& g, const T* a, const T* b, T* y, int H, int D, cudaStream_t st) {
  const int HD = H * D;
  const bool al = aligned16(a) && aligned16(b);
  const VecShape s = pick_shape<T>(HD, D, al);
  const int tile0 = pick_tile(g.E);
  const long long nt = (g.E + tile0 - 1) / tile0;
  const unsigned grid = grid_for_warps(nt, kWarpsPerCta);
  const int lph = D / s.V;
  if (s.R == 0 || !is_pow2(lph)) {
    EdgeDotAnyOp<T, kEdgeFeat> op;
    op.a = a; op.b = b; op.y = y; op.H = H; op.D = D; op.HD = HD;
    walk_kernel<decltype(op), false><<<grid, kWarpsPerCta * 32, 0, st>>>(op, g.hdr, g.erow, g.other, g.eid, g.E, tile0, 0,
                                                                        nullptr, nullptr);
    GK_LAUNCHED("edge_dot_any");
    return GRAPHOP_OK;
  }
  return dispatch_shape<T>(s, [&](auto Vc, auto Rc) -> int {
    constexpr int V = decltype(Vc)::value, R = decltype(Rc)::value;
    if constexpr (V > 1) {
      return dispatch_lph(lph, [&](auto Lc) -> int {
        EdgeDotStaged<T, V, R, kEdgeFeat, decltype(Lc)::value> op;
        op.a = a; op.b = b; op.y = y; op.H = H; op.D = D; op.HD = HD; op.S = s.S; op.lph = lph;
        return launch_staged(op, g, tile0, 0, nullptr, st);
      });
    } else {
      EdgeDotOp<T, V, R, kEdgeFeat> op;
      op.a = a; op.b = b; op.y = y; op.H = H; op.D = D; op.HD = HD; op.S = s.S; op.lph = lph;
      walk_kernel<decltype(op), false><<<grid, kWarpsPerCta * 32, 0, st>>>(op, g.hdr, g.erow, g.other, g.eid, g.E,
                                                                          tile0, 0, nullptr, nullptr);
      GK_LAUNCHED("edge_dot");
      return (int)GRAPHOP_OK;
    }
  });
}

// dB[eid[k], :] = sum_h dy[eid[k], h] * A[node(k), h, :]
template <typename T>
inline int run_edge_mix(const GraphView& g, const T* dy, const T* a, T* db, int H, int D, cudaStream_t st) {
  constexpr int VM = VecMax<T>::value;
  const bool vec = aligned16(a) && aligned16(db) && D % VM == 0;
  const long long total = g.E * (vec ? D / VM : D);
  const unsigned grid = (unsigned)((total + 255) / 256 < (1 << 20) ? (total + 255) / 256 : (1 << 20));
  const int ds = vec ? D / VM : D;
  int shift = -1;
  if (is_pow2(ds)) for (shift = 0; (1 << shift) < ds; ++shift) {}
  const unsigned blocks = grid ? grid : 1;
#define GK_MIX(VV, HH) \
  edge_mix_heads_kernel<T, VV, HH><<<blocks, 256, 0, st>>>(g.erow, g.eid, dy, a, db, g.E, H, D, shift)
  if (vec) {
    if (H == 1) GK_MIX(VM, 1); else if (H == 2) GK_MIX(VM, 2); else if (H == 4) GK_MIX(VM, 4);
    else if (H == 8) GK_MIX(VM, 8); else GK_MIX(VM, 0);
  } else {
    GK_MIX(1, 0);
  }
#undef GK_MIX
  GK_LAUNCHED("edge_mix_heads");
  return GRAPHOP_OK;
}

// ---------------------------------------------------------------------------------------
// softmax
// ---------------------------------------------------------------------------------------
template <typename T, int H, bool kBackward>
inline int run_softmax_heads(Arena& ar, const GraphView& g, const T* in0, const T* in1, T* out, long long n_nodes,
                             int hs, int h0, cudaStream_t st) {
  using A = typename AccOf<T>::type;
  constexpr int kTile = SoftmaxSteps<H>::value * 32;
  constexpr int kW = kBackward ? H : 2 * H;
  const long long nt0 = (g.E + kTile - 1) / kTile;
  // level 0 is the lane-per-edge kernel; levels >= 1 are generic carry levels over 2*nt0 slots
  Levels lv = make_levels(2 * nt0, kCarryTile);
  A* carry0 = (A*)ar.take((size_t)(2 * nt0) * kW * sizeof(A));
  int32_t* rows1 = (int32_t*)ar.take((size_t)(2 * nt0) * 4);
  A* stats = (A*)ar.take((size_t)n_nodes * kW * sizeof(A));
  void* carry[kMaxLevels];
  int32_t* rows[kMaxLevels + 1];
  for (int k = 0; k < lv.n; ++k) {
    const bool last = k == lv.n - 1;
    carry[k] = last ? nullptr : ar.take((size_t)(2 * lv.ntiles[k]) * kW * sizeof(A));
    rows[k + 1] = last ? nullptr : (int32_t*)ar.take((size_t)(2 * lv.ntiles[k]) * 4);
  }
  if (!ar.base) return GRAPHOP_OK;
  if (ar.overflow) return GRAPHOP_ERR_WORKSPACE;
  const unsigned grid0 = grid_for_warps(nt0, kSoftmaxWarps);
  softmax_tile_kernel<T, H, kBackward><<<grid0, kSoftmaxWarps * 32, 0, st>>>(g.erow, g.eid, in0, in1, out, carry0, rows1,
                                                                            g.E, hs, h0);
  GK_LAUNCHED(kBackward ? "softmax_bwd_tile" : "softmax_fwd_tile");
  rows[0] = rows1;
  for (int k = 0; k < lv.n; ++k) {
    SegStatOp<A, !kBackward> op;
    op.stats = stats; op.carry = (A*)carry[k]; op.carry_in = k ? (const A*)carry[k - 1] : carry0; op.H = H;
    op.n_nodes = n_nodes;
    walk_kernel<decltype(op), true><<<grid_for_warps(lv.ntiles[k], kWarpsPerCta), kWarpsPerCta * 32, 0, st>>>(
        op, g.hdr, rows[k], nullptr, nullptr, lv.len[k], lv.tile[k], n_nodes, rows[k + 1], nullptr);
    GK_LAUNCHED("carry_level");
  }
  softmax_finish_kernel<T, H, kBackward><<<grid0, kSoftmaxWarps * 32, 0, st>>>(g.erow, g.eid, in0, in1, out, stats,
                                                                              n_nodes, g.E, hs, h0);
  GK_LAUNCHED(kBackward ? "softmax_bwd_finish" : "softmax_fwd_finish");
  return GRAPHOP_OK;
}

template <typename T, bool kBackward>
inline int run_softmax(Arena& ar, const GraphView& g, const T* in0, const T* in1, T* out, long long n_nodes, int H,
                       cudaStream_t st) {
  const size_t hb = (size_t)H * sizeof(T);
  const bool vec_ok = ((uintptr_t)in0 % (hb < 16 ? hb : 16)) == 0 && ((uintptr_t)out % (hb < 16 ? hb : 16)) == 0 &&
                      (!kBackward || ((uintptr_t)in1 % (hb < 16 ? hb : 16)) == 0);
  if (vec_ok && H == 1) return run_softmax_heads<T, 1, kBackward>(ar, g, in0, in1, out, n_nodes, 1, 0, st);
  if (vec_ok && H == 2) return run_softmax_heads<T, 2, kBackward>(ar, g, in0, in1, out, n_nodes, 2, 0, st);
  if (vec_ok && H == 4) return run_softmax_heads<T, 4, kBackward>(ar, g, in0, in1, out, n_nodes, 4, 0, st);
  if (vec_ok && H == 8) return run_softmax_heads<T, 8, kBackward>(ar, g, in0, in1, out, n_nodes, 8, 0, st);
  // any other head count: one head at a time through the H = 1 kernels, scratch reused
  const size_t mark = ar.used;
  for (int h = 0; h < H; ++h) {
    ar.used = mark;
    GK_TRY((run_softmax_heads<T, 1, kBackward>(ar, g, in0, in1, out, n_nodes, H, h, st)));
    if (!ar.base) break;
  }
  return GRAPHOP_OK;
}

// ---------------------------------------------------------------------------------------
// argument checks shared by the entry points
// ---------------------------------------------------------------------------------------
inline int check_sizes(long long C, long long E, long long n0, long long n1, int H, int D) {
  if (C < 0 || E < 0 || n0 < 0 || n1 < 0 || H < 1 || D < 1) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (E >= (1LL << 31) || n0 >= (1LL << 31) || n1 >= (1LL << 31)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if ((long long)H * D >= (1LL << 24)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  return GRAPHOP_OK;
}
inline int check_ws(const void* ws) {
  if (!ws || ((uintptr_t)ws & (kAlign - 1))) return GRAPHOP_ERR_WORKSPACE;
  return GRAPHOP_OK;
}

// ---------------------------------------------------------------------------------------
// the ten operations
// ---------------------------------------------------------------------------------------
template <typename T, class GS>
inline int maskedmm_forward(const GS& gs, const T* A_, const T* B_, T* y, long long C, long long E, long long n_dst,
                            long long n_src, int H, int D, void* ws, size_t wsb, cudaStream_t st) {
  GK_TRY(check_sizes(C, E, n_dst, n_src, H, D));
  if (E == 0) return GRAPHOP_OK;
  if (!gs.valid(true) || !A_ || !B_ || !y) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  GraphView g;
  GK_TRY(gs(ar, st, &g));
  GK_TRY(zero_uncovered(g, y, (size_t)E * H * sizeof(T), st));
  return run_edge_dot<T, false>(g, A_, B_, y, H, D, st);
}

template <typename T, class GS>
inline int maskedmm_backward(const GS& gs_r, const GS& gs_c, long long Cr, long long Cc, const T* A_, const T* B_,
                             const T* dy, T* dA, T* dB, long long E, long long n_dst, long long n_src, int H, int D,
                             void* ws, size_t wsb, cudaStream_t st) {
  GK_TRY(check_sizes(Cr, E, n_dst, n_src, H, D));
  if (Cc < 0) return GRAPHOP_ERR_INVALID_ARGUMENT;
  const size_t HD = (size_t)H * D;
  if (E == 0) {
    if (n_dst) GK_CUDA(cudaMemsetAsync(dA, 0, (size_t)n_dst * HD * sizeof(T), st));
    if (n_src) GK_CUDA(cudaMemsetAsync(dB, 0, (size_t)n_src * HD * sizeof(T), st));
    return GRAPHOP_OK;
  }
  if (!gs_r.valid(true) || !gs_c.valid(true) || !A_ || !B_ || !dy || !dA || !dB) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  {
    GraphView g;
    GK_TRY(gs_r(ar, st, &g));
    GK_TRY((run_aggregate<T, false>(ar, g, dy, B_, dA, n_dst, H, D, st)));
  }
  ar.used = 0;  // the second pass runs after the first on the same stream: reuse the scratch
  GraphView g;
  GK_TRY(gs_c(ar, st, &g));
  return run_aggregate<T, false>(ar, g, dy, A_, dB, n_src, H, D, st);
}

template <typename T, class GS>
inline int node_mul_edge_forward(const GS& gs, const T* A_, const T* B_, T* y, long long C, long long E,
                                 long long n_dst, int H, int D, void* ws, size_t wsb, cudaStream_t st) {
  GK_TRY(check_sizes(C, E, n_dst, 0, H, D));
  if (E == 0) return GRAPHOP_OK;
  if (!gs.valid(false) || !A_ || !B_ || !y) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  GraphView g;
  GK_TRY(gs(ar, st, &g));
  GK_TRY(zero_uncovered(g, y, (size_t)E * H * sizeof(T), st));
  return run_edge_dot<T, true>(g, A_, B_, y, H, D, st);
}

template <typename T, class GS>
inline int node_mul_edge_backward(const GS& gs, const T* A_, const T* B_, const T* dy, T* dA, T* dB, long long C,
                                  long long E, long long n_dst, int H, int D, void* ws, size_t wsb, cudaStream_t st) {
  GK_TRY(check_sizes(C, E, n_dst, 0, H, D));
  if (E == 0) {
    if (n_dst) GK_CUDA(cudaMemsetAsync(dA, 0, (size_t)n_dst * H * D * sizeof(T), st));
    return GRAPHOP_OK;
  }
  if (!gs.valid(false) || !A_ || !B_ || !dy || !dA || !dB) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  GraphView g;
  GK_TRY(gs(ar, st, &g));
  GK_TRY((run_aggregate<T, true>(ar, g, dy, B_, dA, n_dst, H, D, st)));
  if (!ar.base) return GRAPHOP_OK;
  GK_TRY(zero_uncovered(g, dB, (size_t)E * D * sizeof(T), st));
  return run_edge_mix<T>(g, dy, A_, dB, H, D, st);
}

template <typename T, bool kBackward, class GS>
inline int sparse_softmax(const GS& gs, const T* in0, const T* in1, T* out, long long C, long long E,
                          long long n_nodes, int H, void* ws, size_t wsb, cudaStream_t st) {
  GK_TRY(check_sizes(C, E, n_nodes, 0, H, 1));
  if (E == 0) return GRAPHOP_OK;
  if (!gs.valid(false) || !in0 || !out || (kBackward && !in1)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  GraphView g;
  GK_TRY(gs(ar, st, &g));
  GK_TRY(zero_uncovered(g, out, (size_t)E * H * sizeof(T), st));
  return run_softmax<T, kBackward>(ar, g, in0, in1, out, n_nodes, H, st);
}

template <typename T, class GS>
inline int spmm_forward(const GS& gs, const T* edata, const T* x, T* y, long long C, long long E, long long n_dst,
                        long long n_src, int H, int D, void* ws, size_t wsb, cudaStream_t st) {
  GK_TRY(check_sizes(C, E, n_dst, n_src, H, D));
  if (n_dst == 0) return GRAPHOP_OK;
  if (E == 0) {
    GK_CUDA(cudaMemsetAsync(y, 0, (size_t)n_dst * H * D * sizeof(T), st));
    return GRAPHOP_OK;
  }
  if (!gs.valid(true) || !edata || !x || !y) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  GraphView g;
  GK_TRY(gs(ar, st, &g));
  return run_aggregate<T, false>(ar, g, edata, x, y, n_dst, H, D, st);
}

template <typename T, class GS>
inline int spmm_backward(const GS& gs_r, const GS& gs_c, long long C, long long Ct, const T* edata, const T* dy,
                         const T* x, T* dedata, T* dx, long long E, long long n_dst, long long n_src, int H, int D,
                         void* ws, size_t wsb, cudaStream_t st) {
  GK_TRY(check_sizes(C, E, n_dst, n_src, H, D));
  if (Ct < 0) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if (E == 0) {
    if (n_src) GK_CUDA(cudaMemsetAsync(dx, 0, (size_t)n_src * H * D * sizeof(T), st));
    return GRAPHOP_OK;
  }
  if (!gs_r.valid(true) || !gs_c.valid(true) || !edata || !dy || !x || !dedata || !dx) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  {
    GraphView g;
    GK_TRY(gs_r(ar, st, &g));
    if (ar.base) {
      GK_TRY(zero_uncovered(g, dedata, (size_t)E * H * sizeof(T), st));
      GK_TRY((run_edge_dot<T, false>(g, dy, x, dedata, H, D, st)));
    }
  }
  ar.used = 0;
  GraphView g;
  GK_TRY(gs_c(ar, st, &g));
  return run_aggregate<T, false>(ar, g, edata, dy, dx, n_src, H, D, st);
}

template <typename A>
__global__ void fill_kernel(A* __restrict__ out, A value, long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = value;
}
template <typename A> inline A neg_inf_host();
template <> inline float neg_inf_host<float>() { return -INFINITY; }
template <> inline double neg_inf_host<double>() { return -(double)INFINITY; }

template <typename T>
inline bool attention_shape_ok(int H, int D, bool al, VecShape* s) {
  *s = pick_shape<T>(H * D, D, al);
  return s->V == VecMax<T>::value && s->R != 0 && is_pow2(D / s->V);
}

template <typename T, class GS>
inline int attention_forward(const GS& gs, long long C, const T* q, const T* k, const T* v, double scale, T* o,
                             void* lse, long long E, long long n_dst, long long n_src, int H, int D, void* ws,
                             size_t wsb, cudaStream_t st) {
  using A = typename AccOf<T>::type;
  GK_TRY(check_sizes(C, E, n_dst, n_src, H, D));
  VecShape s;
  if (!attention_shape_ok<T>(H, D, aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o), &s))
    return GRAPHOP_ERR_UNSUPPORTED;
  if (n_dst == 0) return GRAPHOP_OK;
  if (!q || !k || !v || !o || !lse) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  GraphView g;
  const int HD = H * D;
  if (E == 0) {
    // no edge anywhere: o = 0 and lse = -inf for every node
    GK_CUDA(cudaMemsetAsync(o, 0, (size_t)n_dst * HD * sizeof(T), st));
    const long long cells = n_dst * H;
    const unsigned grid = (unsigned)((cells + 255) / 256 < 4096 ? (cells + 255) / 256 : 4096);
    fill_kernel<A><<<grid ? grid : 1, 256, 0, st>>>((A*)lse, neg_inf_host<A>(), cells);
    GK_LAUNCHED("fill");
    return GRAPHOP_OK;
  }
  if (!gs.valid(true)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(gs(ar, st, &g));
  const int tile0 = pick_tile(E);
  return dispatch_shape<T>(s, [&](auto Vc, auto Rc) -> int {
    constexpr int V = decltype(Vc)::value, R = decltype(Rc)::value;
    const long long cstride = HD + 2 * s.S;
    if constexpr (V == 1) return (int)GRAPHOP_ERR_UNSUPPORTED;
    else return dispatch_lph(D / V, [&](auto Lc) -> int {
      constexpr int LPH = decltype(Lc)::value;
      auto generic = [&](void* cout, void* cin) {
        AttnFwdStaged<T, V, R, LPH> op;
        op.q = q; op.k = k; op.v = v; op.o = o; op.lse = (A*)lse; op.carry = (A*)cout; op.carry_in = (const A*)cin;
        op.scale = (A)scale; op.H = H; op.D = D; op.HD = HD; op.S = s.S; op.lph = D / V; op.cstride = cstride;
        return op;
      };
      return run_row_levels(ar, g, tile0, n_dst, sizeof(A), cstride, st, generic);
    });
  });
}

// Defined in gk_banded.cuh for bfloat16: the tensor-core kernel for dense-band graphs.  Returns
// GRAPHOP_ERR_UNSUPPORTED when the shape is not one it takes (the caller then runs the walker).
template <typename T>
int banded_attention_forward(const graphop_plan_t* plan, const T* q, const T* k, const T* v, double scale, T* o,
                             void* lse, long long n_dst, long long n_src, int H, int D, cudaStream_t st);
template <typename T>
inline int banded_attention_forward(const graphop_plan_t*, const T*, const T*, const T*, double, T*, void*, long long,
                                    long long, int, int, cudaStream_t) {
  return GRAPHOP_ERR_UNSUPPORTED;
}

template <typename T>
int banded_attention_backward(const graphop_plan_t* plan_r, const graphop_plan_t* plan_t, const T* q, const T* k,
                              const T* v, const T* o, const void* lse, const T* d_o, double scale, T* dq, T* dk, T* dv,
                              long long n_dst, long long n_src, int H, int D, void* ws, size_t wsb, cudaStream_t st);
template <typename T>
inline int banded_attention_backward(const graphop_plan_t*, const graphop_plan_t*, const T*, const T*, const T*,
                                     const T*, const void*, const T*, double, T*, T*, T*, long long, long long, int, int,
                                     void*, size_t, cudaStream_t) {
  return GRAPHOP_ERR_UNSUPPORTED;
}

template <typename T>
inline int attention_forward_planned(const graphop_plan_t* plan, const T* q, const T* k, const T* v, double scale,
                                     T* o, void* lse, long long n_dst, long long n_src, int H, int D, void* ws,
                                     size_t wsb, cudaStream_t st) {
  if (!plan) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if ((plan->flags & GRAPHOP_PLAN_DENSE_BAND) && q && k && v && o && lse) {
    const int rc = banded_attention_forward<T>(plan, q, k, v, scale, o, lse, n_dst, n_src, H, D, st);
    if (rc != GRAPHOP_ERR_UNSUPPORTED) return rc;
  }
  return attention_forward<T>(FromPlan{plan}, plan->n_chunks, q, k, v, scale, o, lse, plan->n_edges, n_dst, n_src, H,
                              D, ws, wsb, st);
}

// has_eid_t: the transposed source carries edge ids (the positions of its edges in the row CSR)
template <typename T, class GS>
inline int attention_backward(const GS& gs_r, const GS& gs_c, bool has_eid_t, long long C, long long Ct, const T* q,
                              const T* k, const T* v, const T* o, const void* lse, const T* dout, double scale, T* dq,
                              T* dk, T* dv, long long E, long long n_dst, long long n_src, int H, int D, void* ws,
                              size_t wsb, cudaStream_t st) {
  using A = typename AccOf<T>::type;
  GK_TRY(check_sizes(C, E, n_dst, n_src, H, D));
  if (Ct < 0) return GRAPHOP_ERR_INVALID_ARGUMENT;
  VecShape s;
  const bool al = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) && aligned16(dout) && aligned16(dq) &&
                  aligned16(dk) && aligned16(dv);
  if (!attention_shape_ok<T>(H, D, al, &s)) return GRAPHOP_ERR_UNSUPPORTED;
  if (E == 0) {  // no edge: every gradient is zero
    if ((n_dst && !dq) || (n_src && (!dk || !dv))) return GRAPHOP_ERR_INVALID_ARGUMENT;
    const size_t rowb = (size_t)H * D * sizeof(T);
    if (n_dst) GK_CUDA(cudaMemsetAsync(dq, 0, (size_t)n_dst * rowb, st));
    if (n_src) GK_CUDA(cudaMemsetAsync(dk, 0, (size_t)n_src * rowb, st));
    if (n_src) GK_CUDA(cudaMemsetAsync(dv, 0, (size_t)n_src * rowb, st));
    return GRAPHOP_OK;
  }
  if (!gs_r.valid(true) || !gs_c.valid(true) || !q || !k || !v || !o || !lse || !dout || !dq || !dk || !dv)
    return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  const int HD = H * D;
  const int tile0 = pick_tile(E);
  const int Hp = stat_heads(H, (int)sizeof(A));
  StatPair<A>* stat = (StatPair<A>*)ar.take((size_t)n_dst * Hp * sizeof(StatPair<A>));  // survives both passes
  // with the transposed CSR's edge ids the destination pass leaves (p, ds) of every edge for the source pass
  EdgePair<A>* pd = has_eid_t ? (EdgePair<A>*)ar.take((size_t)E * Hp * sizeof(EdgePair<A>)) : nullptr;
  const size_t mark = ar.used;
  {
    GraphView g;
    GK_TRY(gs_r(ar, st, &g));
    GK_TRY((dispatch_shape<T>(s, [&](auto Vc, auto Rc) -> int {
      constexpr int V = decltype(Vc)::value, R = decltype(Rc)::value;
      if constexpr (V == 1) return (int)GRAPHOP_ERR_UNSUPPORTED;
      else return dispatch_lph(D / V, [&](auto Lc) -> int {
        constexpr int LPH = decltype(Lc)::value;
        auto generic = [&](void* cout, void* cin) {
          AttnBwdDstStaged<T, V, R, LPH> op;
          op.q = q; op.k = k; op.v = v; op.o = o; op.dout = dout; op.lse = (const A*)lse; op.stat = stat;
          op.pd = pd; op.dq = dq; op.carry = (A*)cout; op.carry_in = (const A*)cin; op.scale = (A)scale;
          op.H = H; op.Hp = Hp; op.D = D; op.HD = HD; op.S = s.S; op.lph = D / V;
          return op;
        };
        return run_row_levels(ar, g, tile0, n_dst, sizeof(A), HD, st, generic);
      });
    })));
  }
  ar.used = mark;
  GraphView g;
  GK_TRY(gs_c(ar, st, &g));
  return dispatch_shape<T>(s, [&](auto Vc, auto Rc) -> int {
    constexpr int V = decltype(Vc)::value, R = decltype(Rc)::value;
    if constexpr (V == 1) return (int)GRAPHOP_ERR_UNSUPPORTED;
    else return dispatch_lph(D / V, [&](auto Lc) -> int {
      constexpr int LPH = decltype(Lc)::value;
      if (pd) {
        auto weighted = [&](void* cout, void* cin) {
          AttnBwdSrcPairsStaged<T, V, R, LPH> op;
          op.q = q; op.k = k; op.v = v; op.dout = dout; op.stat = stat; op.pd = pd; op.dk = dk;
          op.dv = dv; op.carry = (A*)cout; op.carry_in = (const A*)cin; op.scale = (A)scale;
          op.H = H; op.Hp = Hp; op.D = D; op.HD = HD; op.S = s.S; op.lph = D / V;
          return op;
        };
        return run_row_levels(ar, g, tile0, n_src, sizeof(A), 2 * HD, st, weighted);
      }
      auto generic = [&](void* cout, void* cin) {
        AttnBwdSrcStaged<T, V, R, LPH> op;
        op.q = q; op.k = k; op.v = v; op.dout = dout; op.stat = stat; op.dk = dk;
        op.dv = dv; op.carry = (A*)cout; op.carry_in = (const A*)cin; op.scale = (A)scale;
        op.H = H; op.Hp = Hp; op.D = D; op.HD = HD; op.S = s.S; op.lph = D / V;
        return op;
      };
      return run_row_levels(ar, g, tile0, n_src, sizeof(A), 2 * HD, st, generic);
    });
  });
}

// ---------------------------------------------------------------------------------------
// Attention with an edge term in the scores: s_k = scale * q[n] . (k[other[k]] + rel[k]), rel an (n_edges, D)
// tensor indexed by row-CSR position and shared by the heads.  It is the reference's node_mul_edge
// (graphop_kernel.cu:16-34, "designed for relative positional encoding") added to maskedmm's scores before
// the softmax, computed in the fused pass instead of as two more (n_edges, H) tensors.
// ---------------------------------------------------------------------------------------
template <typename T, class GS>
inline int attention_bias_forward(const GS& gs, long long C, const T* q, const T* k, const T* v, const T* rel,
                                  double scale, T* o, void* lse, long long E, long long n_dst, long long n_src, int H,
                                  int D, void* ws, size_t wsb, cudaStream_t st) {
  using A = typename AccOf<T>::type;
  GK_TRY(check_sizes(C, E, n_dst, n_src, H, D));
  VecShape s;
  if (!attention_shape_ok<T>(H, D, aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) && aligned16(rel), &s))
    return GRAPHOP_ERR_UNSUPPORTED;
  if (E == 0 || n_dst == 0)   // no edge: the edge term has nothing to add
    return attention_forward<T>(gs, C, q, k, v, scale, o, lse, E, n_dst, n_src, H, D, ws, wsb, st);
  if (!q || !k || !v || !rel || !o || !lse || !gs.valid(true)) return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  GraphView g;
  GK_TRY(gs(ar, st, &g));
  const int HD = H * D, tile0 = pick_tile(E);
  return dispatch_shape<T>(s, [&](auto Vc, auto Rc) -> int {
    constexpr int V = decltype(Vc)::value, R = decltype(Rc)::value;
    const long long cstride = HD + 2 * s.S;
    if constexpr (V == 1) return (int)GRAPHOP_ERR_UNSUPPORTED;
    else return dispatch_lph(D / V, [&](auto Lc) -> int {
      constexpr int LPH = decltype(Lc)::value;
      return run_row_levels(ar, g, tile0, n_dst, sizeof(A), cstride, st, [&](void* cout, void* cin) {
        AttnFwdStaged<T, V, R, LPH, true> op;
        op.q = q; op.k = k; op.v = v; op.rel = rel; op.o = o; op.lse = (A*)lse; op.carry = (A*)cout;
        op.carry_in = (const A*)cin; op.scale = (A)scale; op.H = H; op.D = D; op.HD = HD; op.S = s.S; op.lph = D / V;
        op.cstride = cstride;
        return op;
      });
    });
  });
}

// Gradients of the above.  The transposed CSR must carry eid_t (for each of its positions the row-CSR position of
// the same edge): the destination pass leaves (p, ds) of every edge in the workspace, the source pass aggregates
// them into dk and dv, and d_rel[j] = sum_h ds[j, h] q[node(j), h] comes from the same pairs.
template <typename T, class GS>
inline int attention_bias_backward(const GS& gs_r, const GS& gs_c, bool has_eid_t, long long C, long long Ct,
                                   const T* q, const T* k, const T* v, const T* rel, const T* o, const void* lse,
                                   const T* dout, double scale, T* dq, T* dk, T* dv, T* d_rel, long long E,
                                   long long n_dst, long long n_src, int H, int D, void* ws, size_t wsb,
                                   cudaStream_t st) {
  using A = typename AccOf<T>::type;
  GK_TRY(check_sizes(C, E, n_dst, n_src, H, D));
  if (Ct < 0) return GRAPHOP_ERR_INVALID_ARGUMENT;
  VecShape s;
  const bool al = aligned16(q) && aligned16(k) && aligned16(v) && aligned16(o) && aligned16(dout) && aligned16(dq) &&
                  aligned16(dk) && aligned16(dv) && aligned16(rel);
  if (!attention_shape_ok<T>(H, D, al, &s)) return GRAPHOP_ERR_UNSUPPORTED;
  if (E == 0)
    return attention_backward<T>(gs_r, gs_c, has_eid_t, C, Ct, q, k, v, o, lse, dout, scale, dq, dk, dv, E, n_dst,
                                 n_src, H, D, ws, wsb, st);
  if (!has_eid_t || !gs_r.valid(true) || !gs_c.valid(true) || !q || !k || !v || !rel || !o || !lse || !dout || !dq ||
      !dk || !dv || !d_rel)
    return GRAPHOP_ERR_INVALID_ARGUMENT;
  GK_TRY(check_ws(ws));
  Arena ar(ws, wsb);
  const int HD = H * D, tile0 = pick_tile(E), Hp = stat_heads(H, (int)sizeof(A));
  StatPair<A>* stat = (StatPair<A>*)ar.take((size_t)n_dst * Hp * sizeof(StatPair<A>));
  EdgePair<A>* pd = (EdgePair<A>*)ar.take((size_t)E * Hp * sizeof(EdgePair<A>));
  const size_t mark = ar.used;
  {
    GraphView g;
    GK_TRY(gs_r(ar, st, &g));
    GK_TRY((dispatch_shape<T>(s, [&](auto Vc, auto Rc) -> int {
      constexpr int V = decltype(Vc)::value, R = decltype(Rc)::value;
      if constexpr (V == 1) return (int)GRAPHOP_ERR_UNSUPPORTED;
      else return dispatch_lph(D / V, [&](auto Lc) -> int {
        constexpr int LPH = decltype(Lc)::value;
        return run_row_levels(ar, g, tile0, n_dst, sizeof(A), HD, st, [&](void* cout, void* cin) {
          AttnBwdDstStaged<T, V, R, LPH, true> op;
          op.q = q; op.k = k; op.v = v; op.rel = rel; op.o = o; op.dout = dout; op.lse = (const A*)lse;
          op.stat = stat; op.pd = pd; op.dq = dq; op.carry = (A*)cout; op.carry_in = (const A*)cin;
          op.scale = (A)scale; op.H = H; op.Hp = Hp; op.D = D; op.HD = HD; op.S = s.S; op.lph = D / V;
          return op;
        });
      });
    })));
    {
      constexpr int VM = VecMax<T>::value;
      const bool vec = aligned16(d_rel) && D % VM == 0;   // q is 16-byte aligned (checked above)
      const int slots = vec ? D / VM : D;
      int shift = -1;
      if (is_pow2(slots)) for (shift = 0; (1 << shift) < slots; ++shift) {}
      const long long total = E * slots;
      const unsigned grid = (unsigned)((total + 255) / 256 < (1 << 20) ? (total + 255) / 256 : (1 << 20));
      if (vec) bias_grad_kernel<T, VM><<<grid ? grid : 1, 256, 0, st>>>(g.erow, pd, q, d_rel, E, H, Hp, D, shift);
      else bias_grad_kernel<T, 1><<<grid ? grid : 1, 256, 0, st>>>(g.erow, pd, q, d_rel, E, H, Hp, D, shift);
    }
    GK_LAUNCHED("attention_bias_grad");
  }
  ar.used = mark;
  GraphView g;
  GK_TRY(gs_c(ar, st, &g));
  return dispatch_shape<T>(s, [&](auto Vc, auto Rc) -> int {
    constexpr int V = decltype(Vc)::value, R = decltype(Rc)::value;
    if constexpr (V == 1) return (int)GRAPHOP_ERR_UNSUPPORTED;
    else return dispatch_lph(D / V, [&](auto Lc) -> int {
      constexpr int LPH = decltype(Lc)::value;
      return run_row_levels(ar, g, tile0, n_src, sizeof(A), 2 * HD, st, [&](void* cout, void* cin) {
        AttnBwdSrcPairsStaged<T, V, R, LPH> op;
        op.q = q; op.k = k; op.v = v; op.dout = dout; op.stat = stat; op.pd = pd; op.dk = dk;
        op.dv = dv; op.carry = (A*)cout; op.carry_in = (const A*)cin; op.scale = (A)scale;
        op.H = H; op.Hp = Hp; op.D = D; op.HD = HD; op.S = s.S; op.lph = D / V;
        return op;
      });
    });
  });
}

template <typename T>
inline int attention_backward_planned(const graphop_plan_t* plan_r, const graphop_plan_t* plan_t, const T* q,
                                      const T* k, const T* v, const T* o, const void* lse, const T* dout, double scale,
                                      T* dq, T* dk, T* dv, long long n_dst, long long n_src, int H, int D, void* ws,
                                      size_t wsb, cudaStream_t st) {
  if (!plan_r || !plan_t) return GRAPHOP_ERR_INVALID_ARGUMENT;
  if ((plan_r->flags & plan_t->flags & GRAPHOP_PLAN_DENSE_BAND) && q && k && v && o && lse && dout && dq && dk && dv) {
    const int rc = banded_attention_backward<T>(plan_r, plan_t, q, k, v, o, lse, dout, scale, dq, dk, dv, n_dst, n_src,
                                                H, D, ws, wsb, st);
    if (rc != GRAPHOP_ERR_UNSUPPORTED) return rc;
  }
  return attention_backward<T>(FromPlan{plan_r}, FromPlan{plan_t}, plan_t->eid != nullptr, plan_r->n_chunks,
                               plan_t->n_chunks, q, k, v, o, lse, dout, scale, dq, dk, dv, plan_r->n_edges, n_dst,
                               n_src, H, D, ws, wsb, st);
}

}  // namespace gk
