/* A consumer of the C ABI with no Python and no torch in the process: device memory from the CUDA runtime, one
 * vector_spmm forward through the workspace entry point and one through the static-scratch entry point, on a graph
 * small enough to check by hand.  Built and run by tests/test_c_consumer_gpu.py. */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdio.h>
#include <string.h>

#include "graphop_b200.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
  printf("cuda error %s at line %d\n", cudaGetErrorString(e_), __LINE__); return 10; } } while (0)

static void* to_device(const void* host, size_t bytes) {
  void* d = NULL;
  if (cudaMalloc(&d, bytes ? bytes : 16) != cudaSuccess) return NULL;
  if (host && bytes && cudaMemcpy(d, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return NULL;
  return d;
}

int main(void) {
  /* 3 destinations, 3 sources; node 0 <- {0, 2}, node 1 <- {1}, node 2 has no edge.  The un-chunked form of the
   * chunk table: one chunk per node. */
  const int32_t row[3] = {0, 1, 2}, indptr[4] = {0, 2, 3, 3}, eid[3] = {0, 1, 2}, indices[3] = {0, 2, 1};
  const float edata[3] = {0.5f, 2.0f, -1.0f};
  const float x[12] = {1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12};
  const float want[12] = {18.5f, 21.0f, 23.5f, 26.0f, -5, -6, -7, -8, 0, 0, 0, 0};
  float got[12], got_static[12];
  int i, rc;

  int32_t* d_row = (int32_t*)to_device(row, sizeof row);
  int32_t* d_ptr = (int32_t*)to_device(indptr, sizeof indptr);
  int32_t* d_eid = (int32_t*)to_device(eid, sizeof eid);
  int32_t* d_idx = (int32_t*)to_device(indices, sizeof indices);
  float* d_w = (float*)to_device(edata, sizeof edata);
  float* d_x = (float*)to_device(x, sizeof x);
  float* d_y = (float*)to_device(NULL, sizeof got);
  size_t ws_bytes = graphop_workspace_bytes(GRAPHOP_OP_SPMM_FWD, 3, 3, 1, 4, 4, 4);
  void* d_ws = to_device(NULL, ws_bytes);
  if (!d_row || !d_ptr || !d_eid || !d_idx || !d_w || !d_x || !d_y || !d_ws || ws_bytes == 0) {
    printf("allocation failed: %s (workspace %lu bytes)\n", cudaGetErrorString(cudaGetLastError()), (unsigned long)ws_bytes);
    return 11;
  }

  CHECK_CUDA(cudaMemset(d_y, 0xff, sizeof got));   /* NaN pattern: every element must be written */
  rc = graphop_vector_spmm_forward_f32_i32(d_row, d_ptr, d_eid, d_idx, d_w, d_x, d_y, 3, 3, 3, 3, 1, 4, d_ws, ws_bytes,
                                           NULL);
  if (rc != GRAPHOP_OK) { printf("workspace entry: %s\n", graphop_error_string(rc)); return 12; }
  CHECK_CUDA(cudaDeviceSynchronize());
  CHECK_CUDA(cudaMemcpy(got, d_y, sizeof got, cudaMemcpyDeviceToHost));

  CHECK_CUDA(cudaMemset(d_y, 0xff, sizeof got));
  rc = graphop_vector_spmm_forward_f32_i32_static(d_row, d_ptr, d_eid, d_idx, d_w, d_x, d_y, 3, 3, 3, 3, 1, 4, NULL);
  if (rc != GRAPHOP_OK) { printf("static entry: %s\n", graphop_error_string(rc)); return 13; }
  CHECK_CUDA(cudaDeviceSynchronize());
  CHECK_CUDA(cudaMemcpy(got_static, d_y, sizeof got, cudaMemcpyDeviceToHost));

  for (i = 0; i < 12; ++i) {
    if (!(fabsf(got[i] - want[i]) <= 1e-6f * (1.0f + fabsf(want[i])))) { printf("y[%d] = %g, want %g\n", i, got[i], want[i]); return 14; }
  }
  if (memcmp(got, got_static, sizeof got) != 0) { printf("the two entry points differ\n"); return 15; }

  /* a too small workspace is refused, nothing is launched */
  rc = graphop_vector_spmm_forward_f32_i32(d_row, d_ptr, d_eid, d_idx, d_w, d_x, d_y, 3, 3, 3, 3, 1, 4, d_ws, 16, NULL);
  if (rc != GRAPHOP_ERR_WORKSPACE) { printf("small workspace: got %d\n", rc); return 16; }

  cudaFree(d_row); cudaFree(d_ptr); cudaFree(d_eid); cudaFree(d_idx); cudaFree(d_w); cudaFree(d_x); cudaFree(d_y);
  cudaFree(d_ws);
  printf("ok\n");
  return 0;
}
