// MoE dispatch / combine kernels (sm_100a).  See moe.h for the scheme.  Three launches make a
// dispatch -- count (per-segment expert histograms), plan (scan + exchange of the histograms
// between ranks + row offsets), scatter (rows written into the owners' buffers over NVLink) --
// and one launch makes a combine.  Peers are reached with plain 16-byte loads and stores; all
// cross-rank waits go through the bounded block barrier of coll_device.cuh.
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include "../core/log.h"
#include "coll_device.cuh"
#include "moe.h"

namespace amem {
namespace moek {

constexpr int kThreads = 256;

struct Launch {
  int segments;
  int combine_ctas;
};

// ---- K1: histogram of expert ids per contiguous segment of (token, choice) pairs
__device__ void count_body(const MoeArgs& a, int seg, int segments) {
  __shared__ int hist[kMoeMaxExperts];
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int P = a.T * a.k;
  const int per = (P + segments - 1) / segments;
  const int lo = min(P, seg * per), hi = min(P, lo + per);
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    int e = a.topk_idx[i];
    if (e >= 0 && e < a.E) atomicAdd(&hist[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < a.E; e += blockDim.x) a.seg_hist[seg * a.E + e] = hist[e];
}

// ---- K2: one CTA per rank.  Scan the segment histograms, all-gather the per-expert totals
// through the control blocks, derive where my rows start in every owner's buffer.
__device__ void plan_body(const MoeArgs& a, int segments, int* s_abort) {
  __shared__ int cnt[kMaxRanks][kMoeMaxExperts];
  const int n = a.coll.nranks, r = a.coll.rank, E = a.E, El = a.E / n;
  dev::Proto p;
  dev::proto_begin(p, a.coll, 0, 1, s_abort);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int s = 0; s < segments; ++s) {
      a.seg_base[s * E + e] = run;
      run += a.seg_hist[s * E + e];
    }
    cnt[r][e] = run;
  }
  // peers may still read the totals of the previous dispatch: they signal this barrier only
  // after they have left it
  dev::block_barrier(p);
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int q = 0; q < n; ++q) a.coll.ctrl[q]->xchg[r][e] = (uint32_t)cnt[r][e];
  dev::block_barrier(p);
  for (int i = threadIdx.x; i < n * E; i += blockDim.x) {
    int s = i / E, e = i % E;
    cnt[s][e] = (int)dev::ld_volatile(&a.coll.ctrl[r]->xchg[s][e]);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int owner = e / El, first = owner * El;
    int off = 0;
    for (int e2 = first; e2 < e; ++e2)
      for (int s = 0; s < n; ++s) off += cnt[s][e2];
    for (int s = 0; s < r; ++s) off += cnt[s][e];
    a.send_off[e] = off;
  }
  if (threadIdx.x == 0) {
    // rows land expert after expert, so the ones beyond the capacity are exactly the tail of
    // this sequence: clamping the running total gives the counts of the rows actually stored
    const int cap = a.capacity_rows;
    int run = 0;
    for (int el = 0; el < El; ++el) {
      int c = 0;
      for (int s = 0; s < n; ++s) c += cnt[s][r * El + el];
      const int lo = min(run, cap), hi = min(run + c, cap);
      a.expert_counts[el] = hi - lo;
      a.expert_offsets[el] = lo;
      run += c;
    }
    a.expert_offsets[El] = min(run, cap);
    if (a.dropped_rows) *a.dropped_rows = max(0, run - cap);
  }
  dev::proto_end(p);
}

// ---- K3: every pair's row goes to its final place in the owner's receive buffer
__device__ void scatter_body(const MoeArgs& a, int seg, int segments, int* s_abort) {
  __shared__ int run[kMoeMaxExperts];
  __shared__ int c_pos[kThreads];
  __shared__ int c_exp[kThreads];
  const int n = a.coll.nranks, E = a.E, El = a.E / n;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, nwarps = blockDim.x / 32;
  dev::Proto p;
  dev::proto_begin(p, a.coll, seg, segments, s_abort);
  for (int e = threadIdx.x; e < E; e += blockDim.x) run[e] = a.send_off[e] + a.seg_base[seg * E + e];
  __syncthreads();
  const int P = a.T * a.k;
  const int per = (P + segments - 1) / segments;
  const int lo = min(P, seg * per), hi = min(P, lo + per);
  const size_t row_bytes = (size_t)a.d * 2;
  for (int base = lo; base < hi; base += blockDim.x) {
    const int i = base + threadIdx.x;
    int e = -1;
    if (i < hi) {
      e = a.topk_idx[i];
      if (e < 0 || e >= E) e = -1;
    }
    int pos = -1;
    // warps take turns so that rows keep token order inside (source, expert)
    for (int w = 0; w < nwarps; ++w) {
      if (warp == w) {
        unsigned valid = __ballot_sync(0xffffffffu, e >= 0);
        if (e >= 0) {
          unsigned same = __match_any_sync(valid, e);
          int before = __popc(same & ((1u << lane) - 1u));
          int start = run[e];
          __syncwarp(valid);
          if (before == 0) run[e] = start + __popc(same);
          pos = start + before;
        }
      }
      __syncthreads();
    }
    if (pos >= a.capacity_rows) pos = -1;  // no room at the owner: not sent (the plan kernel counted it)
    if (i < hi) a.send_pos[i] = pos;
    c_pos[threadIdx.x] = pos;
    c_exp[threadIdx.x] = e;
    __syncthreads();
    const int in_chunk = min((int)blockDim.x, hi - base);
    for (int j = warp; j < in_chunk; j += nwarps) {
      int pj = c_pos[j];
      if (pj < 0) continue;
      int owner = c_exp[j] / El;
      const uint4* src = (const uint4*)((const char*)a.x + (size_t)((base + j) / a.k) * row_bytes);
      uint4* dst = (uint4*)(a.recv[owner] + (size_t)pj * row_bytes);
      const int nvec = (int)(row_bytes / 16);
      int v = lane;
      for (; v + 96 < nvec; v += 128) {
        uint4 t0 = src[v], t1 = src[v + 32], t2 = src[v + 64], t3 = src[v + 96];
        dst[v] = t0;
        dst[v + 32] = t1;
        dst[v + 64] = t2;
        dst[v + 96] = t3;
      }
      for (; v < nvec; v += 32) dst[v] = src[v];
    }
    __syncthreads();
  }
  // my rows are out; when this barrier passes on every block of a rank, every rank's rows for
  // it have landed (all ranks run the same number of blocks)
  dev::block_barrier(p);
  dev::proto_end(p);
}

// ---- combine: out[t] = sum_j w[t,j] * y_owner(t,j)[row(t,j)]
__device__ void combine_body(const MoeArgs& a, int cta, int nctas, int* s_abort) {
  const int n = a.coll.nranks, El = a.E / n;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, nwarps = blockDim.x / 32;
  dev::Proto p;
  dev::proto_begin(p, a.coll, cta, nctas, s_abort);
  dev::block_barrier(p);  // the expert outputs of every rank are complete
  const int nvec = a.d / 8;
  __nv_bfloat16* out = (__nv_bfloat16*)a.out;
  for (int t = cta * nwarps + warp; t < a.T; t += nctas * nwarps) {
    for (int cv = lane; cv < nvec; cv += 32) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      for (int j0 = 0; j0 < a.k; j0 += 8) {
        uint4 raw[8];
        float w[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          int j = j0 + jj;
          w[jj] = 0.f;
          raw[jj] = make_uint4(0, 0, 0, 0);
          if (j < a.k) {
            int pos = a.send_pos[t * a.k + j];
            if (pos >= 0) {
              int owner = a.topk_idx[t * a.k + j] / El;
              w[jj] = a.topk_w[t * a.k + j];
              raw[jj] = *(const uint4*)(a.ybuf[owner] + ((size_t)pos * a.d + (size_t)cv * 8) * 2);
            }
          }
        }
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const __nv_bfloat16* h = (const __nv_bfloat16*)&raw[jj];
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = fmaf(w[jj], __bfloat162float(h[q]), acc[q]);
        }
      }
      alignas(16) __nv_bfloat16 res[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) res[q] = __float2bfloat16_rn(acc[q]);
      *(uint4*)(out + (size_t)t * a.d + (size_t)cv * 8) = *(const uint4*)res;
    }
  }
  // nobody may overwrite its expert outputs while a peer still reads them
  dev::block_barrier(p);
  dev::proto_end(p);
}

// ---- kernels: one rank per launch, and all ranks of an emulated communicator per launch
__global__ void __launch_bounds__(kThreads) count_kernel(const __grid_constant__ MoeArgs a) { count_body(a, blockIdx.x, gridDim.x); }
__global__ void __launch_bounds__(kThreads) plan_kernel(const __grid_constant__ MoeArgs a, int segments) {
  __shared__ int s_abort;
  plan_body(a, segments, &s_abort);
}
__global__ void __launch_bounds__(kThreads) scatter_kernel(const __grid_constant__ MoeArgs a) {
  __shared__ int s_abort;
  scatter_body(a, blockIdx.x, gridDim.x, &s_abort);
}
__global__ void __launch_bounds__(kThreads) combine_kernel(const __grid_constant__ MoeArgs a) {
  __shared__ int s_abort;
  combine_body(a, blockIdx.x, gridDim.x, &s_abort);
}
__global__ void __launch_bounds__(kThreads) count_kernel_emu(const MoeArgs* __restrict__ all) { count_body(all[blockIdx.y], blockIdx.x, gridDim.x); }
__global__ void __launch_bounds__(kThreads) plan_kernel_emu(const MoeArgs* __restrict__ all, int segments) {
  __shared__ int s_abort;
  plan_body(all[blockIdx.y], segments, &s_abort);
}
__global__ void __launch_bounds__(kThreads) scatter_kernel_emu(const MoeArgs* __restrict__ all) {
  __shared__ int s_abort;
  scatter_body(all[blockIdx.y], blockIdx.x, gridDim.x, &s_abort);
}
__global__ void __launch_bounds__(kThreads) combine_kernel_emu(const MoeArgs* __restrict__ all) {
  __shared__ int s_abort;
  combine_body(all[blockIdx.y], blockIdx.x, gridDim.x, &s_abort);
}

}  // namespace moek

static Status launched(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kCudaError, "%s launch failed: %s", what, cudaGetErrorString(e));
  return kSuccess;
}

Status launch_moe_dispatch(const MoeArgs& a, cudaStream_t stream) {
  moek::count_kernel<<<kMoeSegments, moek::kThreads, 0, stream>>>(a);
  AMEM_TRY(launched("moe count"));
  moek::plan_kernel<<<1, moek::kThreads, 0, stream>>>(a, kMoeSegments);
  AMEM_TRY(launched("moe plan"));
  moek::scatter_kernel<<<kMoeSegments, moek::kThreads, 0, stream>>>(a);
  return launched("moe scatter");
}

Status launch_moe_combine(const MoeArgs& a, cudaStream_t stream) {
  moek::combine_kernel<<<2 * kMoeSegments, moek::kThreads, 0, stream>>>(a);
  return launched("moe combine");
}

template <typename K>
static Status coop(K kernel, dim3 grid, void** params, cudaStream_t stream, const char* what) {
  cudaError_t e = cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3(moek::kThreads), params, 0, stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(kCudaError, "%s cooperative launch failed: %s", what, cudaGetErrorString(e));
  }
  return kSuccess;
}

Status launch_moe_dispatch_emu(const MoeArgs*, const MoeArgs* dev_all, int nranks, cudaStream_t stream) {
  const int segs = 8;
  moek::count_kernel_emu<<<dim3(segs, nranks), moek::kThreads, 0, stream>>>(dev_all);
  AMEM_TRY(launched("moe count(emu)"));
  int segments = segs;
  void* p2[] = {(void*)&dev_all, (void*)&segments};
  AMEM_TRY(coop(moek::plan_kernel_emu, dim3(1, nranks), p2, stream, "moe plan(emu)"));
  void* p3[] = {(void*)&dev_all};
  return coop(moek::scatter_kernel_emu, dim3(segs, nranks), p3, stream, "moe scatter(emu)");
}

Status launch_moe_combine_emu(const MoeArgs*, const MoeArgs* dev_all, int nranks, cudaStream_t stream) {
  void* p[] = {(void*)&dev_all};
  return coop(moek::combine_kernel_emu, dim3(8, nranks), p, stream, "moe combine(emu)");
}

}  // namespace amem
