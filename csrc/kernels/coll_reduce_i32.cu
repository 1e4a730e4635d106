// Reducing collective kernels for one group of element types (see coll_reduce_part.inl).
#define AMEM_PART_FN launch_reduce_part_i32
#define AMEM_PART_TYPES(ALL, SUM) ALL(kI32, kI32, int, int) ALL(kU32, kU32, unsigned, unsigned)
#include "coll_reduce_part.inl"
