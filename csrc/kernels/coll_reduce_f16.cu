// Reducing collective kernels for one group of element types (see coll_reduce_part.inl).
#define AMEM_PART_FN launch_reduce_part_f16
#define AMEM_PART_TYPES(ALL, SUM) ALL(kF16, kF16, __half, __half) SUM(kF32, kF16, float, __half) SUM(kF16, kF32, __half, float)
#include "coll_reduce_part.inl"
