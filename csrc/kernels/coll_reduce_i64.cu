// Reducing collective kernels for one group of element types (see coll_reduce_part.inl).
#define AMEM_PART_FN launch_reduce_part_i64
#define AMEM_PART_TYPES(ALL, SUM) ALL(kI64, kI64, long long, long long) ALL(kU64, kU64, unsigned long long, unsigned long long)
#include "coll_reduce_part.inl"
