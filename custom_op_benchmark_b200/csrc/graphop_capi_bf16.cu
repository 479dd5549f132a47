// C ABI entry points, bfloat16 element type (fp32 accumulation).
#include "graphop_capi_impl.cuh"
GRAPHOP_DEFINE(bf16_i32, uint16_t, __nv_bfloat16, int32_t)
GRAPHOP_DEFINE(bf16_i64, uint16_t, __nv_bfloat16, int64_t)
