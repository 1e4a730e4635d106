// Reducing collective kernels for one group of element types (see coll_reduce_part.inl).
#define AMEM_PART_FN launch_reduce_part_f32
#define AMEM_PART_TYPES(ALL, SUM) ALL(kF32, kF32, float, float)
#include "coll_reduce_part.inl"
