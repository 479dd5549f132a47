// C ABI entry points, float32 element type.
#include "graphop_capi_impl.cuh"
GRAPHOP_DEFINE(f32_i32, float, float, int32_t)
GRAPHOP_DEFINE(f32_i64, float, float, int64_t)
