// C ABI entry points of the eight reference ops, bf16 element type.
#include "graphop_capi_impl.cuh"
GRAPHOP_DEFINE_OPS(bf16_i32, uint16_t, __nv_bfloat16, int32_t)
GRAPHOP_DEFINE_OPS(bf16_i64, uint16_t, __nv_bfloat16, int64_t)
GRAPHOP_DEFINE_PLANNED_OPS(bf16, uint16_t, __nv_bfloat16)
