// Reducing collective kernels for one group of element types (see coll_reduce_part.inl).
#define AMEM_PART_FN launch_reduce_part_i8
#define AMEM_PART_TYPES(ALL, SUM) ALL(kI8, kI8, signed char, signed char) ALL(kU8, kU8, unsigned char, unsigned char)
#include "coll_reduce_part.inl"
