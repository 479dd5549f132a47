// C ABI entry points of the fused attention pair and of its variant with an edge term in the scores, f64 element type.
#include "graphop_capi_impl.cuh"
GRAPHOP_DEFINE_ATTENTION(f64_i32, double, double, int32_t)
GRAPHOP_DEFINE_ATTENTION(f64_i64, double, double, int64_t)
GRAPHOP_DEFINE_ATTENTION_BIAS(f64_i32, double, double, int32_t)
GRAPHOP_DEFINE_ATTENTION_BIAS(f64_i64, double, double, int64_t)
GRAPHOP_DEFINE_PLANNED_ATTENTION(f64, double, double)
