// graphop_vector_spmm_forward_f32_i32_static: the float32 / int32 vector SpMM for callers that
// must not allocate device memory.
//
// Who that is: code that runs inside someone else's memory plan, where a cudaMalloc (or a
// caching-allocator call that may turn into one) is either forbidden or arrives at a bad time.
// Examples are a plugin hosted by an inference server that hands the plugin its tensors and
// nothing else, a real-time loop that may not take the driver's allocation lock, and a process
// whose whole memory pool has already been carved up.  All other entry points ask such a caller
// for a workspace; this one brings its own.
//
// The scratch lives in a file-scope __device__ array of kStaticScratchBytes.  Every GPU on which
// this library's module gets loaded holds that array from load until the process exits, which is
// why the size is modest and fixed.  Problem sizes whose workspace would not fit are refused with
// GRAPHOP_ERR_UNSUPPORTED; nothing is launched in that case.
//
// The array's name is a host-side handle here, not a device address, so the address the kernels
// receive comes from cudaGetSymbolAddress.  That lookup happens on the first call made with a
// given device current, and is remembered per device.  Make that first call outside any stream
// capture: it is an ordinary synchronous runtime query.  If this library's module has not been
// loaded on that device yet (lazy loading), the lookup loads it, and loading it is what places the
// 32 MiB array in that device's memory: so the first call on a device is the one call that can
// fail for lack of device memory, and "allocation-free" is a property of every call after it.
// Call it once with a tiny problem at start-up to have that behind you.
//
// All calls on one GPU share the one array.  The kernels write every scratch word before they
// read it (the owner table, the per-tile carry slots and the slot directory are produced afresh
// by each call), so stale contents from an earlier call never matter and nothing has to be
// cleared.  Two calls that run concurrently on the same GPU (different streams, or different
// host threads) would overwrite each other's scratch: run them one after the other.
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/graphop_b200.h"
#include "gk_host.cuh"

namespace {

constexpr size_t kStaticScratchBytes = (size_t)GRAPHOP_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_address[kMaxDevices];   // zero-initialised; two threads may both resolve, to the same value

// Device address of the array on the current device, resolved once per device.  A failing runtime call
// leaves its code where graphop_last_cuda_error() finds it, like every other entry point's.
int scratch_for_current_device(void** out) {
  int dev = -1;
  GK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return GRAPHOP_ERR_UNSUPPORTED;
  void* p = g_scratch_address[dev].load(std::memory_order_acquire);
  if (!p) {
    GK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    if (!p) return GRAPHOP_ERR_CUDA;
    g_scratch_address[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return GRAPHOP_OK;
}

}  // namespace

extern "C" size_t graphop_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int graphop_vector_spmm_forward_f32_i32_static(const int32_t* row, const int32_t* indptr,
                                                          const int32_t* eid, const int32_t* indices,
                                                          const float* edata, const float* x, float* y,
                                                          int64_t n_chunks, int64_t n_edges, int64_t n_dst,
                                                          int64_t n_src, int H, int D, graphop_stream_t stream) {
  if (n_edges < 0 || n_dst < 0 || n_src < 0 || H < 1 || D < 1) return GRAPHOP_ERR_INVALID_ARGUMENT;
  const size_t need = graphop_workspace_bytes(GRAPHOP_OP_SPMM_FWD, n_edges, n_dst > n_src ? n_dst : n_src, H, D, 4, 4);
  if (need == 0 || need > kStaticScratchBytes) return GRAPHOP_ERR_UNSUPPORTED;
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != GRAPHOP_OK) return rc;
  return graphop_vector_spmm_forward_f32_i32(row, indptr, eid, indices, edata, x, y, n_chunks, n_edges, n_dst, n_src,
                                             H, D, scratch, kStaticScratchBytes, stream);
}
