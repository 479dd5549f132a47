/*
 * Benchmark hooks of graphop_b200.  Not part of the operator surface: these symbols exist only in
 * libgraphop_b200_bench.so, the instrumented twin of the library that bench.py loads beside the product library
 * to attribute a step's time to its kernels.  The twin is built from the same sources with -DGK_BENCH_HOOKS and
 * exports the f32 operator entry points (and the bf16 fused attention) under their usual names, so the same
 * calls can be replayed through it.  The reference has no counterpart; it times whole calls with time.time()
 * (wrapper.py:154-160).
 */
#ifndef GRAPHOP_B200_BENCH_H_
#define GRAPHOP_B200_BENCH_H_

#include <stddef.h>
#include <stdint.h>

#include "../../../include/graphop_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Number of kernels the instrumented library has launched in this process so far. */
long long graphop_bench_launch_count(void);

/* Between graphop_bench_profile_begin(stream) and graphop_bench_profile_end() every kernel the instrumented
 * library launches is followed by a CUDA event on its stream (all calls must use that one stream).
 * graphop_bench_profile_end() waits for the last event and returns the number n of kernels timed (-1 on a CUDA
 * error): ms[i] is the device time of the i-th kernel and `names` receives the n kernel names, one per line. */
int graphop_bench_profile_begin(graphop_stream_t stream);
int graphop_bench_profile_end(char* names, size_t names_bytes, float* ms, int max_entries);

/* Gather ceiling.  For every position k < n_edges a warp reads the row_bytes-byte row table0[indices[k]] (and
 * table1[indices[k]] when table1 is not NULL) and nothing else: no arithmetic beyond a checksum that is never
 * stored, no shared memory, every lane 16 bytes of each row, four edges of loads in flight per warp at 64 warps
 * per SM.  The time of this launch is what gathering one row per edge from these tables through this index
 * stream costs on the GPU at hand, whatever is then done with the rows.  row_bytes: a multiple of 16, at most
 * 512; tables 16-byte aligned; sink: 4 writable bytes (written only if a warp's checksum hits one particular
 * value). */
int graphop_bench_gather_probe_i32(const int32_t* indices, int64_t n_edges, const void* table0, const void* table1,
                                   int row_bytes, void* sink, graphop_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GRAPHOP_B200_BENCH_H_ */
