// Reducing collective kernels for one group of element types (see coll_reduce_part.inl).
#define AMEM_PART_FN launch_reduce_part_f64
#define AMEM_PART_TYPES(ALL, SUM) ALL(kF64, kF64, double, double)
#include "coll_reduce_part.inl"
