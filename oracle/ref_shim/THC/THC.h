// Stand-in for the THC umbrella header that torch stopped shipping.  TEST INFRASTRUCTURE ONLY:
// it lets the reference extension (graphop/graphop_kernel.cu, which includes <THC/THC.h>) compile
// unmodified, from where it lies, against the torch in this image, so that its outputs can be
// used as golden vectors.  Two things the reference relies on changed in torch since it was
// written: THCudaCheck is gone, and AT_DISPATCH_FLOATING_TYPES no longer accepts the deprecated
// `tensor.type()` object.  Both are mapped onto today's equivalents here; no reference source
// line is touched or copied.
#pragma once
#include <ATen/Dispatch.h>
#include <c10/cuda/CUDAException.h>

#define THCudaCheck(expr) C10_CUDA_CHECK(expr)

namespace graphop_ref_shim {
inline at::ScalarType scalar_type_of(at::ScalarType t) { return t; }
inline at::ScalarType scalar_type_of(const at::DeprecatedTypeProperties& t) { return t.scalarType(); }
}  // namespace graphop_ref_shim

#undef AT_DISPATCH_FLOATING_TYPES
#define AT_DISPATCH_FLOATING_TYPES(TYPE, NAME, ...) \
  AT_DISPATCH_SWITCH(graphop_ref_shim::scalar_type_of(TYPE), NAME, AT_DISPATCH_CASE_FLOATING_TYPES(__VA_ARGS__))
