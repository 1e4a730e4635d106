// Device bodies of the collectives and the kernel templates built on them, shared by the
// translation units that instantiate them (collectives.cu: copy kernels, NVLS, send/recv;
// coll_reduce_*.cu: the reducing kernels, one file per group of element types so that they
// compile side by side).
#pragma once
#include <cooperative_groups.h>

#include "../core/log.h"
#include "../core/status.h"
#include "coll_device.cuh"
#include "dispatch.h"
#include "launch.h"

namespace amem {
namespace dev {
#define AMEM_FN __device__ __forceinline__
#define AMEM_BODY __device__ __noinline__
#include "coll_bodies.inl"
#undef AMEM_FN
#undef AMEM_BODY

template <typename TI, typename TO, int OP, bool RED>
__global__ void __launch_bounds__(512) coll_kernel(const __grid_constant__ CollArgs a, size_t chunk_elems) {
  __shared__ int s_abort;
  run_body<TI, TO, OP, RED>(a, blockIdx.x, gridDim.x, &s_abort, chunk_elems);
}

template <typename TI, typename TO, int OP, bool RED>
__global__ void __launch_bounds__(512) coll_kernel_emu(const CollArgs* __restrict__ all, size_t chunk_elems) {
  __shared__ int s_abort;
  run_body<TI, TO, OP, RED>(all[blockIdx.y], blockIdx.x, gridDim.x, &s_abort, chunk_elems);
}
}  // namespace dev

template <typename K>
static Status coop_launch(K kernel, dim3 grid, dim3 block, void** params, cudaStream_t stream, const char* what) {
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)kernel, grid, block, params, 0, stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(kCudaError, "%s cooperative launch (%u x %u blocks) failed: %s", what, grid.x, grid.y, cudaGetErrorString(e));
  }
  return kSuccess;
}

// Reducing kernels of one group of element types (defined in coll_reduce_*.cu).  `dev_all`
// non-null selects the emulation kernel over `nranks` ranks.  *handled tells whether the
// group covers (a.dtype, a.out_dtype, a.redop).
#define AMEM_DECLARE_REDUCE_PART(name) \
  Status name(const CollArgs& a, const LaunchPlan& plan, cudaStream_t stream, const CollArgs* dev_all, int nranks, bool* handled)
AMEM_DECLARE_REDUCE_PART(launch_reduce_part_i8);
AMEM_DECLARE_REDUCE_PART(launch_reduce_part_i32);
AMEM_DECLARE_REDUCE_PART(launch_reduce_part_i64);
AMEM_DECLARE_REDUCE_PART(launch_reduce_part_f16);
AMEM_DECLARE_REDUCE_PART(launch_reduce_part_f32);
AMEM_DECLARE_REDUCE_PART(launch_reduce_part_f64);
AMEM_DECLARE_REDUCE_PART(launch_reduce_part_bf16);

}  // namespace amem
