// Body of one coll_reduce_*.cu file.  The including file defines
//   AMEM_PART_FN                 name of the launcher it provides
//   AMEM_PART_TYPES(ALL, SUM)    its element types: ALL(code_in, code_out, TI, TO) for every
//                                operator, SUM(code_in, code_out, TI, TO) for the fused-cast sums
#include "coll_kernels.cuh"

namespace amem {

Status AMEM_PART_FN(const CollArgs& a, const LaunchPlan& plan, cudaStream_t stream, const CollArgs* dev_all, int nranks, bool* handled) {
  *handled = false;
  Status st = kSuccess;
  bool ok = true;
  const dim3 block(plan.threads);
  size_t chunk = plan.chunk_elems;
#define AMEM_LAUNCH(TI, TO, OP)                                                                                         \
  do {                                                                                                                  \
    *handled = true;                                                                                                    \
    if (dev_all) {                                                                                                      \
      dim3 grid(plan.blocks, nranks);                                                                                   \
      void* params[] = {(void*)&dev_all, (void*)&chunk};                                                                \
      st = coop_launch(dev::coll_kernel_emu<TI, TO, OP, true>, grid, block, params, stream, "collective(emu)");         \
    } else {                                                                                                            \
      dev::coll_kernel<TI, TO, OP, true><<<dim3(plan.blocks), block, 0, stream>>>(a, chunk);                            \
    }                                                                                                                   \
  } while (0)
#define AMEM_PART_ALL(DI, DO, TI, TO) \
  if (!*handled && a.dtype == (DI) && a.out_dtype == (DO)) { AMEM_DISPATCH_OP(TI, TO, a.redop, AMEM_LAUNCH) }
#define AMEM_PART_SUM(DI, DO, TI, TO) \
  if (!*handled && a.dtype == (DI) && a.out_dtype == (DO) && (a.redop == kSum || a.redop == kAvg)) { AMEM_LAUNCH(TI, TO, ::amem::kSum); }
  AMEM_PART_TYPES(AMEM_PART_ALL, AMEM_PART_SUM)
#undef AMEM_PART_ALL
#undef AMEM_PART_SUM
#undef AMEM_LAUNCH
  if (!ok) *handled = false;  // the type is ours but the operator is unknown
  return st;
}

}  // namespace amem
