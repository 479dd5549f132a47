// C ABI entry points of the eight reference ops, f64 element type.
#include "graphop_capi_impl.cuh"
GRAPHOP_DEFINE_OPS(f64_i32, double, double, int32_t)
GRAPHOP_DEFINE_OPS(f64_i64, double, double, int64_t)
GRAPHOP_DEFINE_PLANNED_OPS(f64, double, double)
