// Reducing collective kernels for one group of element types (see coll_reduce_part.inl).
#define AMEM_PART_FN launch_reduce_part_bf16
#define AMEM_PART_TYPES(ALL, SUM) ALL(kBF16, kBF16, __nv_bfloat16, __nv_bfloat16) SUM(kF32, kBF16, float, __nv_bfloat16) SUM(kBF16, kF32, __nv_bfloat16, float)
#include "coll_reduce_part.inl"
