// C ABI entry points, float64 element type.
#include "graphop_capi_impl.cuh"
GRAPHOP_DEFINE(f64_i32, double, double, int32_t)
GRAPHOP_DEFINE(f64_i64, double, double, int64_t)
