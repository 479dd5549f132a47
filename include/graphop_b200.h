/*
 * graphop_b200: C ABI of the sparse graph-attention operator set for NVIDIA B200 (sm_100a).
 *
 * This is the boundary a host binding links against.  It replaces the host launchers of the
 * reference extension (graphop/graphop_kernel.cu:235-600, the eight *_cuda_forward /
 * *_cuda_backward functions that graphop/graphop.cpp:8-214 declares and wraps for Python)
 * with plain pointers and sizes: no torch types, no allocation, no exceptions.  Every operator
 * entry point enqueues its kernels on `stream` and returns at once with a status code; nothing
 * synchronises the device.  Two set-up / debugging calls are the exceptions and say so below:
 * graphop_check_graph_* (allocates one word with cudaMallocAsync and waits for its verdict) and
 * graphop_plan_build_* (waits once for the graph's shape flags).
 *
 * Graph arguments follow the reference contract (graphop_kernel.cu:20, 41, ...): `row` holds
 * one owner node per chunk (length n_chunks), `indptr` the n_chunks + 1 chunk boundaries as
 * CSR positions, `eid` maps a position to an edge id (the row index of every edge tensor;
 * NULL means the identity), `indices` gives the other endpoint of a position.  Chunks come
 * from partition_csr (part_csr.py:13-27) or are the plain CSR rows (row = 0..N-1).  Required
 * of the caller: indptr non-decreasing, chunks of one node consecutive, node ids
 * non-decreasing along `row` and below the node count passed with them, eid injective,
 * n_edges < 2^31 (graphop_check_graph_* verifies all of it).  Under that contract every
 * reduction is computed by exactly one owner in a fixed order: results are bit-reproducible
 * (the reference accumulates with atomics, graphop/atomic.cuh:57-96).
 *
 * Tensor layouts are those of the reference: node tensors (n, H, D) row-major, edge tensors
 * (n_edges, H) row-major; H = 1 covers the reference's 2-D / 1-D spellings.
 *
 * Naming: graphop_<op>_<elem>_<index>, elem in {f32, f64, bf16}, index in {i32, i64}.
 * f32 / f64 with i64 indices is the reference's own type set (AT_DISPATCH_FLOATING_TYPES and
 * .data<int64_t>(), graphop_kernel.cu:254-258); bf16 (fp32 accumulation) and i32 indices are
 * additions.  bf16 values are passed as uint16_t bit patterns.
 *
 * Workspace: each entry point needs scratch memory in device global memory, passed as
 * (workspace, workspace_bytes); graphop_workspace_bytes() gives a sufficient size.  The
 * workspace holds no state between calls.
 */
#ifndef GRAPHOP_B200_H_
#define GRAPHOP_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* graphop_stream_t; /* a cudaStream_t */

enum {
  GRAPHOP_OK = 0,
  GRAPHOP_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, n_edges >= 2^31, ... */
  GRAPHOP_ERR_WORKSPACE = 2,        /* workspace_bytes too small or workspace misaligned */
  GRAPHOP_ERR_UNSUPPORTED = 3,      /* shape outside what this entry point implements */
  GRAPHOP_ERR_CUDA = 4              /* a CUDA call failed; see graphop_last_cuda_error() */
};

/* Operation ids for graphop_workspace_bytes(). */
enum {
  GRAPHOP_OP_MASKEDMM_FWD = 0,
  GRAPHOP_OP_MASKEDMM_BWD = 1,
  GRAPHOP_OP_NODE_MUL_EDGE_FWD = 2,
  GRAPHOP_OP_NODE_MUL_EDGE_BWD = 3,
  GRAPHOP_OP_SOFTMAX_FWD = 4,
  GRAPHOP_OP_SOFTMAX_BWD = 5,
  GRAPHOP_OP_SPMM_FWD = 6,
  GRAPHOP_OP_SPMM_BWD = 7,
  GRAPHOP_OP_ATTENTION_FWD = 8,
  GRAPHOP_OP_ATTENTION_BWD = 9,          /* graphop_attention_backward with eid_t == NULL */
  GRAPHOP_OP_ATTENTION_BWD_PAIRS = 10     /* ... with eid_t: room for (p, ds) of every edge and head */
};

int graphop_version(void);
const char* graphop_error_string(int code);
/* cudaError_t of the most recent failed CUDA call made by this library on this thread. */
int graphop_last_cuda_error(void);

/* out[r, :] = table[idx[r], :] for r < n_rows, rows of row_bytes bytes (a multiple of 16; both tensors
 * 16-byte aligned).  Packs the rows a peer asked for before they are sent, and the rows a shard references
 * from its own block (sharded SpMM).  The reference runs on one device and has no counterpart. */
int graphop_gather_rows_i32(const int32_t* idx, int64_t n_rows, const void* table, int64_t row_bytes, void* out,
                            graphop_stream_t stream);

/* out[r, :] = tables[p][idx[r], :] for the rows r of segment p, seg[p] <= r < seg[p + 1] (`tables` and `seg` are host
 * arrays of n_tables pointers and n_tables + 1 offsets, seg[0] = 0; n_tables <= GRAPHOP_MAX_PEERS).  The tables are
 * the blocks of a row-sharded tensor on this and on peer GPUs, mapped into this process (CUDA IPC / symmetric memory):
 * one kernel on the receiving GPU pulls every needed row across NVLink once, with plain peer loads, instead of the
 * owners packing rows and a collective delivering them.  The caller orders the call after the owners' writes (and the
 * owners' next writes after it).  Rows are row_bytes bytes, a multiple of 16; tables and out 16-byte aligned. */
#define GRAPHOP_MAX_PEERS 16
int graphop_pull_rows_i32(const void* const* tables, const int64_t* seg, int n_tables, const int32_t* idx,
                          int64_t row_bytes, void* out, graphop_stream_t stream);

/* partition_csr on the device (reference: part_csr.py:13-27, a host double loop): every CSR row
 * [indptr[r], indptr[r+1]) cut into chunks of at most chunk_size positions; row[c] = the row of chunk c,
 * indptr_out[c] = its first position, indptr_out[n_chunks] = indptr[n_rows].  Outputs are int64 for either index
 * type.  Two calls, because the caller allocates the outputs: _count writes the number of chunks to the HOST
 * integer *n_chunks (synchronises `stream`) and leaves every row's first chunk in `ws`; _fill, given the same `ws`
 * untouched, writes row (n_chunks entries) and indptr_out (n_chunks + 1 entries).  n_rows < 2^31 - 1. */
size_t graphop_partition_csr_workspace_bytes(int64_t n_rows);
int graphop_partition_csr_count_i32(const int32_t* indptr, int64_t n_rows, int64_t chunk_size, void* ws,
                                    size_t ws_bytes, int64_t* n_chunks, graphop_stream_t stream);
int graphop_partition_csr_count_i64(const int64_t* indptr, int64_t n_rows, int64_t chunk_size, void* ws,
                                    size_t ws_bytes, int64_t* n_chunks, graphop_stream_t stream);
int graphop_partition_csr_fill_i32(const int32_t* indptr, int64_t n_rows, int64_t chunk_size, const void* ws,
                                   int64_t n_chunks, int64_t* row, int64_t* indptr_out, graphop_stream_t stream);
int graphop_partition_csr_fill_i64(const int64_t* indptr, int64_t n_rows, int64_t chunk_size, const void* ws,
                                   int64_t n_chunks, int64_t* row, int64_t* indptr_out, graphop_stream_t stream);

/* The transposed CSR the backward passes take (the reference's scripts build it with scipy on the host,
 * wrapper.py:96-112): edges regrouped by source with ties in row-CSR order, so within one source the destinations
 * ascend.  indptr (n_dst + 1) and indices (n_edges, source ids in [0, n_src)) are the row CSR whose edge ids are its
 * positions; outputs, in the same integer type: indptr_t (n_src + 1), indices_t (n_edges: the destination of every
 * transposed position), eid_t (n_edges: its position in the row CSR).  Deterministic; does not synchronise.
 * n_edges < 2^31 - 1. */
size_t graphop_transpose_csr_workspace_bytes(int64_t n_edges, int index_bytes);
int graphop_transpose_csr_i32(const int32_t* indptr, const int32_t* indices, int64_t n_dst, int64_t n_src,
                              int64_t n_edges, int32_t* indptr_t, int32_t* indices_t, int32_t* eid_t,
                              void* ws, size_t ws_bytes, graphop_stream_t stream);
int graphop_transpose_csr_i64(const int64_t* indptr, const int64_t* indices, int64_t n_dst, int64_t n_src,
                              int64_t n_edges, int64_t* indptr_t, int64_t* indices_t, int64_t* eid_t,
                              void* ws, size_t ws_bytes, graphop_stream_t stream);

/* Sufficient workspace for one call of `op`.  n_nodes: the largest node count among the
 * call's node tensors (for the softmax ops: an upper bound on node id + 1).  elem_bytes: 2, 4
 * or 8; index_bytes: 4 or 8. */
size_t graphop_workspace_bytes(int op, int64_t n_edges, int64_t n_nodes, int H, int D, int elem_bytes,
                               int index_bytes);

/* Checks the graph contract stated above on the device and copies the verdict back
 * (synchronises `stream`).  Returns GRAPHOP_OK, or GRAPHOP_ERR_INVALID_ARGUMENT with
 * *violations (may be NULL) set to a bit mask: 1 indptr decreases, 2 row decreases,
 * 4 an index outside [0, n_other), 8 an edge id outside [0, n_edges), 16 a position range
 * outside [0, n_edges).  `indices` and `eid` may be NULL to skip their checks. */
int graphop_check_graph_i32(const int32_t* row, const int32_t* indptr, const int32_t* eid, const int32_t* indices,
                            int64_t n_chunks, int64_t n_edges, int64_t n_nodes, int64_t n_other, int* violations,
                            graphop_stream_t stream);
int graphop_check_graph_i64(const int64_t* row, const int64_t* indptr, const int64_t* eid, const int64_t* indices,
                            int64_t n_chunks, int64_t n_edges, int64_t n_nodes, int64_t n_other, int* violations,
                            graphop_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Graph plans.  Every entry point above rebuilds, per call, what depends on the graph alone: the owner node of
 * every CSR position (from the chunk table) and, for 64-bit indices, 32-bit copies of `indices` and `eid`.  A plan
 * holds those once per graph, in memory the caller provides, and the *_planned entry points take plans in place of
 * the (row, indptr, eid, indices) arguments.  The reference does its graph preprocessing on the host in Python
 * loops before any op runs (part_csr.py:18-21, wrapper.py:93-112); a plan is the same one-time step, on the device.
 *
 * graphop_plan_build_* also looks at the graph's shape: GRAPHOP_PLAN_DENSE_BAND is set when every node's
 * neighbours are one run of consecutive ids and any 128 consecutive nodes reach at most
 * GRAPHOP_BAND_MAX_SPAN different neighbours (sliding-window attention written as a graph, the reference's
 * block-diagonal test graph of wrapper.py:79-112): graphop_attention_forward_planned_bf16 then runs such a graph on
 * the tensor cores.
 *
 * The kernels cut the position stream into tiles of equal length, one warp each, and a node whose positions cross a
 * tile boundary is finished by small follow-up launches (carry levels).  plan_build moves every boundary up to the
 * next row start where there is one inside the tile; if no node crosses a boundary then (every node at most a tile
 * long: the two flags GRAPHOP_PLAN_ROW_TILES | GRAPHOP_PLAN_NO_CARRY are set together), the planned row-reducing ops
 * use those tiles and are one launch each.  The order in which a row's terms are added then differs from the
 * chunk-table entry points' (whole rows instead of tile pieces): results agree to rounding, not to the bit; each
 * stays reproducible from run to run.  On every other graph the planned ops use the same tiles as the chunk-table
 * ones and give identical bits.
 *
 * A plan refers to the caller's `indices` / `eid` arrays when they are 32-bit (they must outlive the plan) and to
 * plan memory otherwise.  graphop_plan_build_* enqueues its kernels on `stream` and waits for them once, to read
 * the shape flags back: it is a set-up call, not a per-step one.
 * --------------------------------------------------------------------------------------------------------- */
enum {
  GRAPHOP_PLAN_DENSE_BAND = 1,
  GRAPHOP_PLAN_ROW_TILES = 2, /* tile_start holds the work tiles' boundaries, moved up to row starts, ... */
  GRAPHOP_PLAN_NO_CARRY = 4   /* ... and no node's positions cross one: row reductions finish in one launch */
};
#define GRAPHOP_BAND_MAX_SPAN 384

typedef struct graphop_plan {
  int64_t n_chunks;        /* chunks of the table the plan was built from */
  int64_t n_edges;         /* CSR positions */
  int64_t n_nodes;         /* bound on the owner node ids (rows of the per-node arrays below) */
  const void* header;      /* device: first / one-past-last position any chunk covers */
  const int32_t* erow;     /* device, n_edges: owner node of every position, -1 where no chunk covers it */
  const int32_t* other;    /* device, n_edges: the other endpoint of every position; NULL when built without */
  const int32_t* eid;      /* device, n_edges: edge id of every position; NULL: the identity */
  const int32_t* node_lo;  /* device, n_nodes: first neighbour of every node (dense-band graphs; else undefined) */
  const int32_t* node_deg; /* device, n_nodes: number of positions every node owns */
  int32_t flags;           /* GRAPHOP_PLAN_* */
  int32_t band_span;       /* most different neighbours any 128 consecutive nodes reach (dense-band graphs) */
  const int32_t* tile_start; /* device, n_tiles + 1: first position of every work tile (GRAPHOP_PLAN_ROW_TILES) */
  int32_t tile;            /* nominal positions per work tile the boundaries were made for */
  int32_t reserved;
} graphop_plan_t;

/* Bytes of device memory (256-byte aligned) a plan of these sizes needs. */
size_t graphop_plan_bytes(int64_t n_chunks, int64_t n_edges, int64_t n_nodes, int index_bytes);
/* Builds a plan in `memory`.  `indices` may be NULL for ops without a second endpoint (then no shape analysis is
 * made), `eid` NULL for the identity.  Synchronises `stream` once. */
int graphop_plan_build_i32(const int32_t* row, const int32_t* indptr, const int32_t* eid, const int32_t* indices,
                           int64_t n_chunks, int64_t n_edges, int64_t n_nodes, void* memory, size_t memory_bytes,
                           graphop_plan_t* plan, graphop_stream_t stream);
int graphop_plan_build_i64(const int64_t* row, const int64_t* indptr, const int64_t* eid, const int64_t* indices,
                           int64_t n_chunks, int64_t n_edges, int64_t n_nodes, void* memory, size_t memory_bytes,
                           graphop_plan_t* plan, graphop_stream_t stream);

/* The ten operations on plans: same results, same workspace query, argument meaning as in GRAPHOP_DECLARE below.
 * plan_r: plan of the row (destination) CSR, plan_c / plan_t: plan of the column / transposed CSR (built with
 * its `eid`: for the fused attention backward that is what lets the row pass hand (p, ds) to the transposed one). */
#define GRAPHOP_DECLARE_PLANNED(SUF, T)                                                                              \
  int graphop_maskedmm_csr_forward_planned_##SUF(const graphop_plan_t* plan, const T* A, const T* B, T* y,           \
                                                 int64_t n_dst, int64_t n_src, int H, int D, void* workspace,        \
                                                 size_t workspace_bytes, graphop_stream_t stream);                   \
  int graphop_maskedmm_csr_backward_planned_##SUF(const graphop_plan_t* plan_r, const graphop_plan_t* plan_c,        \
                                                  const T* A, const T* B, const T* dy, T* dA, T* dB, int64_t n_dst,  \
                                                  int64_t n_src, int H, int D, void* workspace,                      \
                                                  size_t workspace_bytes, graphop_stream_t stream);                  \
  int graphop_node_mul_edge_forward_planned_##SUF(const graphop_plan_t* plan, const T* A, const T* B, T* y,          \
                                                  int64_t n_dst, int H, int D, void* workspace,                      \
                                                  size_t workspace_bytes, graphop_stream_t stream);                  \
  int graphop_node_mul_edge_backward_planned_##SUF(const graphop_plan_t* plan, const T* A, const T* B, const T* dy,  \
                                                   T* dA, T* dB, int64_t n_dst, int H, int D, void* workspace,       \
                                                   size_t workspace_bytes, graphop_stream_t stream);                 \
  int graphop_sparse_softmax_forward_planned_##SUF(const graphop_plan_t* plan, const T* x, T* y, int H,              \
                                                   void* workspace, size_t workspace_bytes,                          \
                                                   graphop_stream_t stream);                                         \
  int graphop_sparse_softmax_backward_planned_##SUF(const graphop_plan_t* plan, const T* y, const T* dy, T* dx,      \
                                                    int H, void* workspace, size_t workspace_bytes,                  \
                                                    graphop_stream_t stream);                                        \
  int graphop_vector_spmm_forward_planned_##SUF(const graphop_plan_t* plan, const T* edata, const T* x, T* y,        \
                                                int64_t n_dst, int64_t n_src, int H, int D, void* workspace,         \
                                                size_t workspace_bytes, graphop_stream_t stream);                    \
  int graphop_vector_spmm_backward_planned_##SUF(const graphop_plan_t* plan_r, const graphop_plan_t* plan_t,         \
                                                 const T* edata, const T* dy, const T* x, T* dedata, T* dx,          \
                                                 int64_t n_dst, int64_t n_src, int H, int D, void* workspace,        \
                                                 size_t workspace_bytes, graphop_stream_t stream);                   \
  int graphop_attention_forward_planned_##SUF(const graphop_plan_t* plan, const T* q, const T* k, const T* v,        \
                                              double scale, T* o, void* lse, int64_t n_dst, int64_t n_src, int H,    \
                                              int D, void* workspace, size_t workspace_bytes,                        \
                                              graphop_stream_t stream);                                              \
  int graphop_attention_backward_planned_##SUF(const graphop_plan_t* plan_r, const graphop_plan_t* plan_t,           \
                                               const T* q, const T* k, const T* v, const T* o, const void* lse,      \
                                               const T* d_o, double scale, T* dq, T* dk, T* dv, int64_t n_dst,       \
                                               int64_t n_src, int H, int D, void* workspace, size_t workspace_bytes, \
                                               graphop_stream_t stream);

#define GRAPHOP_DECLARE(SUF, T, I)                                                                                   \
  /* y[eid[k], h] = sum_d A[row(k), h, d] * B[indices[k], h, d]; edge ids no chunk covers get 0.                  \
   * Replaces maskedmm_csr_cuda_forward (graphop_kernel.cu:269-304; bound at graphop.cpp:16-30, 217). */            \
  int graphop_maskedmm_csr_forward_##SUF(const I* row, const I* indptr, const I* eid, const I* indices, const T* A, \
                                         const T* B, T* y, int64_t n_chunks, int64_t n_edges, int64_t n_dst,        \
                                         int64_t n_src, int H, int D, void* workspace, size_t workspace_bytes,      \
                                         graphop_stream_t stream);                                                  \
  /* dA[n] = sum_{k in n} dy[eid_r[k]] * B[indices_r[k]] over the row CSR, dB the same over the column CSR with   \
   * A in B's place.  Replaces maskedmm_csr_cuda_backward (graphop_kernel.cu:355-409; graphop.cpp:108-131, 218). */ \
  int graphop_maskedmm_csr_backward_##SUF(const I* row, const I* indptr_r, const I* eid_r, const I* indices_r,      \
                                          int64_t n_chunks_r, const I* col, const I* indptr_c, const I* eid_c,      \
                                          const I* indices_c, int64_t n_chunks_c, const T* A, const T* B,           \
                                          const T* dy, T* dA, T* dB, int64_t n_edges, int64_t n_dst, int64_t n_src, \
                                          int H, int D, void* workspace, size_t workspace_bytes,                    \
                                          graphop_stream_t stream);                                                 \
  /* y[eid[k], h] = sum_d A[row(k), h, d] * B[eid[k], d], B an (n_edges, D) edge tensor shared by the heads.       \
   * Replaces node_mul_edge_cuda_forward (graphop_kernel.cu:235-266; graphop.cpp:39-51, 219). */                    \
  int graphop_node_mul_edge_forward_##SUF(const I* row, const I* indptr, const I* eid, const T* A, const T* B,      \
                                          T* y, int64_t n_chunks, int64_t n_edges, int64_t n_dst, int H, int D,     \
                                          void* workspace, size_t workspace_bytes, graphop_stream_t stream);        \
  /* dA[n, h, :] = sum_{k in n} dy[eid[k], h] * B[eid[k], :];  dB[eid[k], :] = sum_h dy[eid[k], h] * A[row(k), h, :]. \
   * Replaces node_mul_edge_cuda_backward (graphop_kernel.cu:306-351; graphop.cpp:141-154, 220). */                 \
  int graphop_node_mul_edge_backward_##SUF(const I* row, const I* indptr, const I* eid, const T* A, const T* B,     \
                                           const T* dy, T* dA, T* dB, int64_t n_chunks, int64_t n_edges,            \
                                           int64_t n_dst, int H, int D, void* workspace, size_t workspace_bytes,    \
                                           graphop_stream_t stream);                                                \
  /* Per (node, head): y = exp(x - max) / sum exp(x - max) over the node's edges; uncovered edge ids get 0.        \
   * n_nodes bounds node id + 1 (the reference sizes its scratch by n_edges, graphop_kernel.cu:420-427).            \
   * Replaces sparse_softmax_cuda_forward (graphop_kernel.cu:411-463; graphop.cpp:59-69, 221). */                   \
  int graphop_sparse_softmax_forward_##SUF(const I* row, const I* indptr, const I* eid, const T* x, T* y,           \
                                           int64_t n_chunks, int64_t n_edges, int64_t n_nodes, int H,               \
                                           void* workspace, size_t workspace_bytes, graphop_stream_t stream);       \
  /* dx = y * (dy - sum_node dy * y).                                                                              \
   * Replaces sparse_softmax_cuda_backward (graphop_kernel.cu:465-507; graphop.cpp:163-175, 222). */                \
  int graphop_sparse_softmax_backward_##SUF(const I* row, const I* indptr, const I* eid, const T* y, const T* dy,   \
                                            T* dx, int64_t n_chunks, int64_t n_edges, int64_t n_nodes, int H,       \
                                            void* workspace, size_t workspace_bytes, graphop_stream_t stream);      \
  /* y[n, h, :] = sum_{k in n} edata[eid[k], h] * x[indices[k], h, :]; nodes without edges get 0.  y has n_dst     \
   * rows (the reference forces n_dst = n_src by y = zeros_like(x), graphop_kernel.cu:527).                         \
   * Replaces vector_spmm_cuda_forward (graphop_kernel.cu:509-542; graphop.cpp:79-93, 223). */                      \
  int graphop_vector_spmm_forward_##SUF(const I* row, const I* indptr, const I* eid, const I* indices,              \
                                        const T* edata, const T* x, T* y, int64_t n_chunks, int64_t n_edges,        \
                                        int64_t n_dst, int64_t n_src, int H, int D, void* workspace,                \
                                        size_t workspace_bytes, graphop_stream_t stream);                           \
  /* dedata[eid[k], h] = sum_d dy[row(k), h, d] * x[indices[k], h, d];                                             \
   * dx[c, h, :] = sum_{k in c} edata[eid_t[k], h] * dy[indices_t[k], h, :] over the transposed CSR, all of its    \
   * chunks (the reference's launch drops some, graphop_kernel.cu:566, 588).                                        \
   * Replaces vector_spmm_cuda_backward (graphop_kernel.cu:544-600; graphop.cpp:190-214, 224). */                   \
  int graphop_vector_spmm_backward_##SUF(const I* row, const I* indptr, const I* eid, const I* indices,             \
                                         int64_t n_chunks, const I* col, const I* indptr_t, const I* eid_t,         \
                                         const I* indices_t, int64_t n_chunks_t, const T* edata, const T* dy,       \
                                         const T* x, T* dedata, T* dx, int64_t n_edges, int64_t n_dst,              \
                                         int64_t n_src, int H, int D, void* workspace, size_t workspace_bytes,      \
                                         graphop_stream_t stream);                                                  \
  /* Fused chain maskedmm -> *scale -> sparse_softmax -> vector_spmm without the (n_edges, H) intermediates:       \
   * o[n] = sum_k softmax_k(scale * q[n].k[indices[k]]) v[indices[k]], lse[n, h] = log sum_k exp(score) kept for   \
   * the backward (float for f32 / bf16, double for f64); nodes without edges get o = 0, lse = -inf.  No reference \
   * counterpart as one call; it composes graphop_kernel.cu:269-304, 411-463 and 509-542.                           \
   * GRAPHOP_ERR_UNSUPPORTED unless D * sizeof(T) is a power-of-two multiple of 16 bytes and H * D * sizeof(T)      \
   * <= 4096 bytes. */                                                                                              \
  int graphop_attention_forward_##SUF(const I* row, const I* indptr, const I* indices, int64_t n_chunks, const T* q, \
                                      const T* k, const T* v, double scale, T* o, void* lse, int64_t n_edges,       \
                                      int64_t n_dst, int64_t n_src, int H, int D, void* workspace,                  \
                                      size_t workspace_bytes, graphop_stream_t stream);                             \
  /* Gradients of the fused chain: dq over the row CSR, dk and dv over the transposed CSR, probabilities            \
   * recomputed from q, k and lse.  Composes graphop_kernel.cu:544-600, 465-507 and 355-409.  eid_t (may be NULL):  \
   * for every position of the transposed CSR the position of the same edge in the row CSR (the eid_t the           \
   * reference's callers build, wrapper.py:129-141, when the row CSR's edge ids are its positions).  With it the    \
   * row pass leaves (p, ds) of every edge in the workspace and the transposed pass only aggregates; without it     \
   * the transposed pass recomputes both from q, k, lse and delta. */                                               \
  int graphop_attention_backward_##SUF(const I* row, const I* indptr, const I* indices, int64_t n_chunks,           \
                                       const I* col, const I* indptr_t, const I* eid_t, const I* indices_t,         \
                                       int64_t n_chunks_t,                                                          \
                                       const T* q, const T* k, const T* v, const T* o, const void* lse,             \
                                       const T* d_o, double scale, T* dq, T* dk, T* dv, int64_t n_edges,            \
                                       int64_t n_dst, int64_t n_src, int H, int D, void* workspace,                 \
                                       size_t workspace_bytes, graphop_stream_t stream);                            \
  /* The fused chain with an edge term in the scores: s_k = scale * q[n] . (k[indices[k]] + rel[k]), rel an         \
   * (n_edges, D) tensor indexed by row-CSR position and shared by the heads.  This is the layer the reference      \
   * builds from maskedmm + node_mul_edge ("designed for relative positional encoding", graphop_kernel.cu:16-34,     \
   * 40-55) -> softmax -> vector_spmm, without the two (n_edges, H) score tensors.  Workspace:                      \
   * GRAPHOP_OP_ATTENTION_FWD.  Same shape limits as graphop_attention_forward. */                                   \
  int graphop_attention_bias_forward_##SUF(const I* row, const I* indptr, const I* indices, int64_t n_chunks,       \
                                           const T* q, const T* k, const T* v, const T* rel, double scale, T* o,    \
                                           void* lse, int64_t n_edges, int64_t n_dst, int64_t n_src, int H, int D,  \
                                           void* workspace, size_t workspace_bytes, graphop_stream_t stream);       \
  /* Its gradients: dq = sum ds (k + rel), dk, dv as in graphop_attention_backward, and                             \
   * d_rel[k, :] = sum_h ds[k, h] q[n, h, :] (node_mul_edge's dB, graphop_kernel.cu:79-93).  eid_t is required      \
   * here (for every position of the transposed CSR the row-CSR position of the same edge): the row pass leaves     \
   * (p, ds) of every edge in the workspace for the other two.  Workspace: GRAPHOP_OP_ATTENTION_BWD_PAIRS. */       \
  int graphop_attention_bias_backward_##SUF(const I* row, const I* indptr, const I* indices, int64_t n_chunks,      \
                                            const I* col, const I* indptr_t, const I* eid_t, const I* indices_t,    \
                                            int64_t n_chunks_t, const T* q, const T* k, const T* v, const T* rel,   \
                                            const T* o, const void* lse, const T* d_o, double scale, T* dq, T* dk,  \
                                            T* dv, T* d_rel, int64_t n_edges, int64_t n_dst, int64_t n_src, int H,  \
                                            int D, void* workspace, size_t workspace_bytes,                         \
                                            graphop_stream_t stream);

/* Scratch-free variant of graphop_vector_spmm_forward_f32_i32 for callers that cannot allocate
 * device memory (a plugin living inside another program's memory plan, a loop that must not take
 * the allocator's lock).  It has no counterpart in the reference.  Same arguments minus the
 * workspace: the scratch is a fixed array of GRAPHOP_STATIC_SCRATCH_BYTES inside the library, held
 * by every GPU that loads it.  Returns GRAPHOP_ERR_UNSUPPORTED, launching nothing, when
 * graphop_workspace_bytes(GRAPHOP_OP_SPMM_FWD, ...) for the sizes exceeds that.  Calls no cudaMalloc
 * / cudaFree or any allocating routine.  The first call on each device resolves the array's device
 * address (make it before any stream capture); where the CUDA runtime loads modules lazily that
 * lookup is also what loads this library's module on the device and so places the array in its
 * memory - the one moment this entry point can fail for lack of device memory.  Make one small
 * call at start-up; every later call touches no allocator.  All calls on a GPU share the array: calls that
 * overlap on the device race; stale contents are harmless, every scratch word is rewritten. */
#define GRAPHOP_STATIC_SCRATCH_BYTES (32u << 20)
size_t graphop_static_scratch_bytes(void);
int graphop_vector_spmm_forward_f32_i32_static(const int32_t* row, const int32_t* indptr, const int32_t* eid,
                                               const int32_t* indices, const float* edata, const float* x, float* y,
                                               int64_t n_chunks, int64_t n_edges, int64_t n_dst, int64_t n_src,
                                               int H, int D, graphop_stream_t stream);

GRAPHOP_DECLARE(f32_i32, float, int32_t)
GRAPHOP_DECLARE(f32_i64, float, int64_t)
GRAPHOP_DECLARE(f64_i32, double, int32_t)
GRAPHOP_DECLARE(f64_i64, double, int64_t)
GRAPHOP_DECLARE(bf16_i32, uint16_t, int32_t)
GRAPHOP_DECLARE(bf16_i64, uint16_t, int64_t)
GRAPHOP_DECLARE_PLANNED(f32, float)
GRAPHOP_DECLARE_PLANNED(f64, double)
GRAPHOP_DECLARE_PLANNED(bf16, uint16_t)

#ifdef __cplusplus
}
#endif
#endif /* GRAPHOP_B200_H_ */
