// C ABI entry points of the fused attention pair and of its variant with an edge term in the scores, f32 element type.
#include "graphop_capi_impl.cuh"
GRAPHOP_DEFINE_ATTENTION(f32_i32, float, float, int32_t)
GRAPHOP_DEFINE_ATTENTION(f32_i64, float, float, int64_t)
GRAPHOP_DEFINE_ATTENTION_BIAS(f32_i32, float, float, int32_t)
GRAPHOP_DEFINE_ATTENTION_BIAS(f32_i64, float, float, int64_t)
GRAPHOP_DEFINE_PLANNED_ATTENTION(f32, float, float)
