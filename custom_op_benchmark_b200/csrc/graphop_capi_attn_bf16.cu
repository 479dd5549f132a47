// C ABI entry points of the fused attention pair and of its variant with an edge term in the scores, bf16 element type.
#include "gk_banded.cuh"
#include "graphop_capi_impl.cuh"
GRAPHOP_DEFINE_ATTENTION(bf16_i32, uint16_t, __nv_bfloat16, int32_t)
GRAPHOP_DEFINE_ATTENTION(bf16_i64, uint16_t, __nv_bfloat16, int64_t)
GRAPHOP_DEFINE_ATTENTION_BIAS(bf16_i32, uint16_t, __nv_bfloat16, int32_t)
GRAPHOP_DEFINE_ATTENTION_BIAS(bf16_i64, uint16_t, __nv_bfloat16, int64_t)
GRAPHOP_DEFINE_PLANNED_ATTENTION(bf16, uint16_t, __nv_bfloat16)
