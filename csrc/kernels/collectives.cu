// CUDA kernels of the collectives (sm_100a) and their launchers.
//
// Data moves by plain peer stores/loads through the NVSwitch (push protocol described in
// coll_args.h) or, for the NVLS all-reduce, by multimem.ld_reduce / multimem.st on the
// multicast mapping of the staging segments, which reduces inside the switch.  No TMA and
// no cluster multicast is used anywhere in this file.  Every spin is bounded (coll_device.cuh).
//
// "emu" launchers run all ranks of a communicator as ONE cooperative grid on one GPU
// (blockIdx.y = rank): kernels of different ranks wait on one another, so they must never be
// separate launches on the same device.  This is what lets the single-GPU test-suite cover
// the multi-rank protocol.
// Reference parity: see coll_bodies.inl; the NVLS variant corresponds to NCCL's NVLS algorithm, whose
// multicast handles the reference unbinds and rebinds (amem_nccl_plugin/amem_nccl.cpp:536-538,614-616).
#include "coll_kernels.cuh"

namespace amem {
namespace dev {

// ------------------------------------------------------------------ NVLS all-reduce
template <typename T> struct Multimem;
template <> struct Multimem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    v.x = __float_as_uint(__uint_as_float(v.x) * s);
    v.y = __float_as_uint(__uint_as_float(v.y) * s);
    v.z = __float_as_uint(__uint_as_float(v.z) * s);
    v.w = __float_as_uint(__uint_as_float(v.w) * s);
    return v;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint32_t scale1(uint32_t w, float s) {
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&w);
    float2 f = __bfloat1622float2(h);
    __nv_bfloat162 o = __floats2bfloat162_rn(f.x * s, f.y * s);
    return *reinterpret_cast<uint32_t*>(&o);
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    return make_uint4(scale1(v.x, s), scale1(v.y, s), scale1(v.z, s), scale1(v.w, s));
  }
};
template <> struct Multimem<__half> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ uint32_t scale1(uint32_t w, float s) {
    __half2 h = *reinterpret_cast<__half2*>(&w);
    float2 f = __half22float2(h);
    __half2 o = __floats2half2_rn(f.x * s, f.y * s);
    return *reinterpret_cast<uint32_t*>(&o);
  }
  static __device__ __forceinline__ uint4 scale(uint4 v, float s) {
    return make_uint4(scale1(v.x, s), scale1(v.y, s), scale1(v.z, s), scale1(v.w, s));
  }
};
__device__ __forceinline__ void multimem_st(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// NVLS all-reduce.  Three jobs per chunk: stage the chunk into my staging (HBM), let the switch
// add everybody's copy of my slice and broadcast the sum back into every rank's staging
// (multimem.ld_reduce + multimem.st on the multicast mapping: NVLink), copy the reduced chunk
// out (HBM).  A message of one chunk does them in turn with two barriers.  Longer messages
// run the two HBM jobs on one group of warps and the switch job on another; the groups never
// meet, they are coupled by per-block credits: "staged N" (CtrlBlock::ready) lets every rank's
// reducer start on chunk N, "reduced N" (CtrlBlock::freed) lets every rank copy chunk N out.
// Three staging regions rotate; region N % 3 is restaged only after chunk N-3 was copied out,
// which (program order of the copy group) is also after everybody's reduce of it.
template <typename T, int U>
__device__ __forceinline__ void nvls_reduce_slice(const CollArgs& a, Proto& p, char* region_mc, size_t len, size_t full, Lane lr) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(T), vi = 16 / es;
  // slices and block ranges of a FULL chunk (`full` elements), cut off at `len`: block b touches the
  // same bytes of a region in every chunk (see block_range_clip)
  size_t sl = ((full + n - 1) / n + vi - 1) / vi * vi;
  size_t b0 = (size_t)r * sl, b1 = b0 + sl;
  if (b0 > len) b0 = len;
  if (b1 > len) b1 = len;
  size_t slo, shi;
  block_range_clip(sl * es, (b1 - b0) * es, p.block, p.nblocks, &slo, &shi);
  // the staging tail beyond `len` holds stale but mapped bytes: whole vectors are safe
  size_t nvec = (shi - slo + 15) / 16;
  char* base = region_mc + b0 * es + slo;
  const size_t nt = lr.nt;
  size_t i = lr.tid;
  // U switch reductions in flight per thread: a round trip through the NVSwitch takes
  // microseconds, the link only fills with megabytes outstanding per GPU
  for (; i + (U - 1) * nt < nvec; i += U * nt) {
    uint4 v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) v[j] = Multimem<T>::ld_reduce(base + (i + j * nt) * 16);
    if (a.has_scale) {
#pragma unroll
      for (int j = 0; j < U; ++j) v[j] = Multimem<T>::scale(v[j], a.scale);
    }
#pragma unroll
    for (int j = 0; j < U; ++j) multimem_st(base + (i + j * nt) * 16, v[j]);
  }
  for (; i < nvec; i += nt) {
    uint4 v = Multimem<T>::ld_reduce(base + i * 16);
    if (a.has_scale) v = Multimem<T>::scale(v, a.scale);
    multimem_st(base + i * 16, v);
  }
}

// Copy of one chunk (`len` elements) between the user's buffer and my staging, split over the
// blocks the same way nvls_reduce_slice splits the switch job: block b moves its share of EVERY
// rank's slice.  Then block b of a reducer depends on block b of every rank and on nothing else,
// which is what the per-block barriers and credits promise.
template <typename T>
__device__ __forceinline__ void nvls_copy_sliced(char* dst, const char* src, size_t len, size_t full, const CollArgs& a, const Proto& p, Lane ln) {
  const int n = a.nranks;
  const size_t es = sizeof(T), vi = 16 / es;
  const size_t sl = ((full + n - 1) / n + vi - 1) / vi * vi;   // slice length of a full chunk, whatever this chunk's length
  int nfull = sl ? (int)(len / sl) : 0;
  if (nfull > n) nfull = n;
  size_t lo, hi;
  block_range(sl * es, p.block, p.nblocks, &lo, &hi);
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    // the full slices together: one 16-byte load per slice in flight per thread
    const size_t nvec = (hi - lo) / 16, stride = sl * es / 16, nt = ln.nt;
    const uint4* s4 = (const uint4*)(src + lo);
    uint4* d4 = (uint4*)(dst + lo);
    for (size_t i = ln.tid; i < nvec; i += nt) {
      uint4 v[kMaxRanks];
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q)
        if (q < nfull) v[q] = s4[(size_t)q * stride + i];
#pragma unroll
      for (int q = 0; q < kMaxRanks; ++q)
        if (q < nfull) d4[(size_t)q * stride + i] = v[q];
    }
  } else {
    for (int q = 0; q < nfull; ++q) copy_span(dst + (size_t)q * sl * es + lo, src + (size_t)q * sl * es + lo, hi - lo, ln);
  }
  for (int q = nfull; q < n; ++q) {  // the ragged end: at most one short slice, the rest empty
    size_t b0 = (size_t)q * sl, b1 = b0 + sl;
    if (b0 > len) b0 = len;
    if (b1 > len) b1 = len;
    block_range_clip(sl * es, (b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
    copy_span(dst + b0 * es + lo, src + b0 * es + lo, hi - lo, ln);
  }
}

template <typename T>
__device__ __forceinline__ void body_allreduce_nvls(const CollArgs& a, Proto& p, size_t chunk_elems) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(T), vi = 16 / es;
  const size_t N = a.count;
  const size_t H = 2 * quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t hoff = half_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq);
  const size_t region = (H / 3) & ~(size_t)4095;
  size_t ce = chunk_elems;
  if (ce * es > region) ce = region / es;
  ce = ce / (vi * n) * (vi * n);
  if (ce == 0) ce = vi * n;
  const uint32_t nch = (uint32_t)((N + ce - 1) / ce);
  const size_t fe = nch == 1 ? N : ce;   // slices and block ranges: of the whole message, or of a full chunk
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  auto stage_in = [&](uint32_t t, Lane ln) {
    size_t off = (size_t)t * ce, len = N - off < ce ? N - off : ce;
    nvls_copy_sliced<T>(a.stage[r] + hoff + (t % 3) * region, send + off * es, len, fe, a, p, ln);
  };
  auto stage_out = [&](uint32_t t, Lane ln) {
    size_t off = (size_t)t * ce, len = N - off < ce ? N - off : ce;
    nvls_copy_sliced<T>(recv + off * es, a.stage[r] + hoff + (t % 3) * region, len, fe, a, p, ln);
  };
  auto reduce = [&](uint32_t t, Lane ln) {
    size_t off = (size_t)t * ce, len = N - off < ce ? N - off : ce;
    nvls_reduce_slice<T, 8>(a, p, a.mc_stage + hoff + (t % 3) * region, len, fe, ln);
  };
  auto reduce_deep = [&](uint32_t t, Lane ln) {  // few warps: twice the loads in flight each
    size_t off = (size_t)t * ce, len = N - off < ce ? N - off : ce;
    nvls_reduce_slice<T, 16>(a, p, a.mc_stage + hoff + (t % 3) * region, len, fe, ln);
  };
  if (nch == 1) {
    stage_in(0, full_lane());
    block_barrier(p);
    reduce(0, full_lane());
    block_barrier(p);
    stage_out(0, full_lane());
    return;
  }
  Lane lr, lc;
  bool do_red, do_copy;
  // the switch job needs few instructions, the two HBM copies need many loads in flight
  split_lanes(true, a.nvls_split > 0 ? a.nvls_split : 4, &lr, &lc, &do_red, &do_copy);
  const uint32_t base = ld_volatile(&p.me->cseq[p.block]);
  if (do_copy) {
    for (uint32_t t = 0; t < nch + 2; ++t) {
      if (t >= 2) {
        credit_wait(p, false, base + (t - 2) + 1u, lc, true);  // every rank (mine too) has reduced chunk t-2
        stage_out(t - 2, lc);
      }
      if (t < nch) {
        stage_in(t, lc);
        credit_signal(p, true, base + t + 1u, lc, true);  // "staged t"
      }
    }
  } else {
    for (uint32_t t = 0; t < nch; ++t) {
      credit_wait(p, true, base + t + 1u, lr, true);     // every rank (mine too) has staged chunk t
      reduce_deep(t, lr);
      credit_signal(p, false, base + t + 1u, lr, true);  // "reduced t"
    }
  }
  block_sync();
  if (thread_index() == 0) p.me->cseq[p.block] = base + nch;
}

// All-reduce on registered windows through their multicast mappings: rank r asks the switch for
// the sum of everybody's slice r (multimem.ld_reduce on the input window) and has the switch write
// it into everybody's output window (multimem.st).  No staging copy on either side, so a byte
// crosses HBM once on the way out and once on the way in; one barrier before, one after.
template <typename T>
__device__ __forceinline__ void body_allreduce_window_nvls(const CollArgs& a, Proto& p) {
  const int n = a.nranks, r = a.rank;
  const size_t es = sizeof(T), vi = 16 / es;
  const size_t N = a.count;
  size_t sl = ((N + n - 1) / n + vi - 1) / vi * vi;
  size_t b0 = (size_t)r * sl, b1 = b0 + sl;
  if (b0 > N) b0 = N;
  if (b1 > N) b1 = N;
  size_t lo, hi;
  block_range((b1 - b0) * es, p.block, p.nblocks, &lo, &hi);
  block_barrier(p);
  const size_t nvec = (hi - lo) / 16;   // the launcher only takes this path for whole 16-byte vectors
  const char* src = a.mc_send + b0 * es + lo;
  char* dst = a.mc_recv + b0 * es + lo;
  const size_t nt = blockDim.x;
  size_t i = threadIdx.x;
  constexpr int U = 8;
  for (; i + (U - 1) * nt < nvec; i += U * nt) {
    uint4 v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) v[j] = Multimem<T>::ld_reduce(src + (i + j * nt) * 16);
    if (a.has_scale) {
#pragma unroll
      for (int j = 0; j < U; ++j) v[j] = Multimem<T>::scale(v[j], a.scale);
    }
#pragma unroll
    for (int j = 0; j < U; ++j) multimem_st(dst + (i + j * nt) * 16, v[j]);
  }
  for (; i < nvec; i += nt) {
    uint4 v = Multimem<T>::ld_reduce(src + i * 16);
    if (a.has_scale) v = Multimem<T>::scale(v, a.scale);
    multimem_st(dst + i * 16, v);
  }
  block_barrier(p);
}

// Reduce-scatter whose INPUT lies in a registered window with a multicast mapping: rank r asks the
// switch for the sum of everybody's slice r and stores it (scaled if asked) into its own output.
// Nothing is staged and nothing is pushed: each rank receives one slice instead of n - 1.
template <typename T>
__device__ __forceinline__ void body_reducescatter_window_nvls(const CollArgs& a, Proto& p) {
  const int r = a.rank;
  const size_t es = sizeof(T);
  const size_t R = a.count;   // elements each rank receives
  size_t lo, hi;
  block_range(R * es, p.block, p.nblocks, &lo, &hi);
  block_barrier(p);           // every rank's input is complete
  const size_t nvec = (hi - lo) / 16;
  const char* src = a.mc_send + (size_t)r * R * es + lo;
  char* dst = (char*)a.recv + lo;
  const size_t nt = blockDim.x;
  size_t i = threadIdx.x;
  constexpr int U = 8;
  for (; i + (U - 1) * nt < nvec; i += U * nt) {
    uint4 v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) v[j] = Multimem<T>::ld_reduce(src + (i + j * nt) * 16);
    if (a.has_scale) {
#pragma unroll
      for (int j = 0; j < U; ++j) v[j] = Multimem<T>::scale(v[j], a.scale);
    }
#pragma unroll
    for (int j = 0; j < U; ++j) *(uint4*)(dst + (i + j * nt) * 16) = v[j];
  }
  for (; i < nvec; i += nt) {
    uint4 v = Multimem<T>::ld_reduce(src + i * 16);
    if (a.has_scale) v = Multimem<T>::scale(v, a.scale);
    *(uint4*)(dst + i * 16) = v;
  }
  block_barrier(p);           // nobody overwrites its input while a peer's reduction still reads it
}

// All-gather whose OUTPUT lies in a registered window with a multicast mapping: ONE store per 16
// bytes, replicated by the switch into every rank's output, instead of one store per peer.
__device__ __forceinline__ void body_allgather_window_nvls(const CollArgs& a, Proto& p) {
  const int r = a.rank;
  const size_t B = a.count;   // bytes contributed by each rank (the copy collectives run on bytes)
  size_t lo, hi;
  block_range(B, p.block, p.nblocks, &lo, &hi);
  block_barrier(p);           // every rank is done with the previous contents of its output
  copy_span_mc(a.mc_recv + (size_t)r * B + lo, (const char*)a.send + lo, hi - lo, full_lane());
  block_barrier(p);           // everybody's piece has landed everywhere
}

// Reduce to a root through the switch: every rank copies its chunk into its own staging (a local
// HBM copy, nothing crosses NVLink yet), the root then asks the switch for the sum of everybody's
// copy (multimem.ld_reduce) and stores it into its output.  The root's link carries the message
// once, not n - 1 times as when every rank pushes its contribution to the root.
template <typename T>
__device__ __forceinline__ void body_reduce_nvls(const CollArgs& a, Proto& p, size_t chunk_elems) {
  const int r = a.rank;
  const size_t es = sizeof(T), vi = 16 / es;
  const size_t N = a.count;
  const size_t H = 2 * quarter_bytes(a.stage_bytes, a.p2p_slot_bytes);
  const size_t hoff = half_offset(a.stage_bytes, a.p2p_slot_bytes, p.opseq);
  size_t ce = chunk_elems;
  if (ce * es > H) ce = H / es;
  ce = ce / vi * vi;
  if (ce == 0) ce = vi;
  const char* send = (const char*)a.send;
  char* recv = (char*)a.recv;
  const size_t fe = N <= ce ? N : ce;   // what the blocks split: the whole message, or a full chunk (block_range_clip)
  for (size_t off = 0; off < N; off += ce) {
    const size_t len = N - off < ce ? N - off : ce;
    size_t lo, hi;
    block_range_clip(fe * es, len * es, p.block, p.nblocks, &lo, &hi);
    copy_span(a.stage[r] + hoff + lo, send + off * es + lo, hi - lo, full_lane());
    block_barrier(p);   // everybody's chunk is staged
    if (r == a.root) {
      // whole vectors: the staging tail beyond the chunk holds stale but mapped bytes
      const size_t nvec = (hi - lo + 15) / 16, nt = blockDim.x;
      const char* src = a.mc_stage + hoff + lo;
      char* dst = recv + off * es + lo;
      const bool dst_vec = (((uintptr_t)dst) & 15) == 0;
      for (size_t i = threadIdx.x; i < nvec; i += nt) {
        uint4 v = Multimem<T>::ld_reduce(src + i * 16);
        if (a.has_scale) v = Multimem<T>::scale(v, a.scale);
        const size_t left = (hi - lo) - i * 16;
        if (dst_vec && left >= 16) {
          *(uint4*)(dst + i * 16) = v;
        } else {
          const char* vb = (const char*)&v;
          for (size_t b = 0; b < 16 && b < left; ++b) dst[i * 16 + b] = vb[b];
        }
      }
    }
    block_barrier(p);   // the root has read the chunk: staging may be overwritten
  }
}
template <typename T>
__global__ void __launch_bounds__(512) nvls_reduce_kernel(const __grid_constant__ CollArgs a, size_t chunk_elems) {
  __shared__ int s_abort;
  Proto p;
  proto_begin(p, a, blockIdx.x, gridDim.x, &s_abort);
  body_reduce_nvls<T>(a, p, chunk_elems);
  proto_end(p);
}

template <typename T>
__global__ void __launch_bounds__(512) nvls_window_reducescatter_kernel(const __grid_constant__ CollArgs a) {
  __shared__ int s_abort;
  Proto p;
  proto_begin(p, a, blockIdx.x, gridDim.x, &s_abort);
  body_reducescatter_window_nvls<T>(a, p);
  proto_end(p);
}
__global__ void __launch_bounds__(512) nvls_window_allgather_kernel(const __grid_constant__ CollArgs a) {
  __shared__ int s_abort;
  Proto p;
  proto_begin(p, a, blockIdx.x, gridDim.x, &s_abort);
  body_allgather_window_nvls(a, p);
  proto_end(p);
}

template <typename T>
__global__ void __launch_bounds__(512) nvls_window_allreduce_kernel(const __grid_constant__ CollArgs a) {
  __shared__ int s_abort;
  Proto p;
  proto_begin(p, a, blockIdx.x, gridDim.x, &s_abort);
  body_allreduce_window_nvls<T>(a, p);
  proto_end(p);
}

// ------------------------------------------------------------------ kernels
template <typename T>
__global__ void __launch_bounds__(512) nvls_allreduce_kernel(const __grid_constant__ CollArgs a, size_t chunk_elems) {
  __shared__ int s_abort;
  Proto p;
  proto_begin(p, a, blockIdx.x, gridDim.x, &s_abort);
  body_allreduce_nvls<T>(a, p, chunk_elems);
  proto_end(p);
}

// blockIdx.x enumerates (entry, lane) pairs; lanes of an entry depend only on its byte count,
// so sender and receiver agree on them.
__device__ __forceinline__ void sendrecv_dispatch(const CollArgs& a, int* s_abort) {
  int b = blockIdx.x;
  for (int e = 0; e < a.n_p2p; ++e) {
    int lanes = p2p_lanes(a.p2p[e].bytes, a.p2p_slot_bytes, a.p2p_max_lanes);
    if (b < lanes) {
      body_sendrecv(a, e, b, lanes, s_abort);
      return;
    }
    b -= lanes;
  }
}
__global__ void __launch_bounds__(512) sendrecv_kernel(const __grid_constant__ CollArgs a) {
  __shared__ int s_abort;
  sendrecv_dispatch(a, &s_abort);
}
// Emulation: ranks may have different numbers of (entry, lane) blocks; surplus blocks exit.
__global__ void __launch_bounds__(512) sendrecv_kernel_emu(const CollArgs* __restrict__ all) {
  __shared__ int s_abort;
  sendrecv_dispatch(all[blockIdx.y], &s_abort);
}

}  // namespace dev

// ------------------------------------------------------------------ launchers
static Status check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kCudaError, "%s launch failed: %s", what, cudaGetErrorString(e));
  return kSuccess;
}

// The reducing kernels live in one translation unit per group of element types.
static Status launch_reduce(const CollArgs& a, const LaunchPlan& plan, cudaStream_t stream, const CollArgs* dev_all, int nranks, bool* ok) {
  typedef Status (*PartFn)(const CollArgs&, const LaunchPlan&, cudaStream_t, const CollArgs*, int, bool*);
  static const PartFn parts[] = {launch_reduce_part_bf16, launch_reduce_part_f32, launch_reduce_part_f16, launch_reduce_part_i32,
                                 launch_reduce_part_i64,  launch_reduce_part_i8,  launch_reduce_part_f64};
  for (PartFn fn : parts) {
    bool handled = false;
    Status st = fn(a, plan, stream, dev_all, nranks, &handled);
    if (handled) return st;
  }
  *ok = false;
  return kSuccess;
}

int sendrecv_blocks(const CollArgs& a) {
  int total = 0;
  for (int e = 0; e < a.n_p2p; ++e) total += p2p_lanes(a.p2p[e].bytes, a.p2p_slot_bytes, a.p2p_max_lanes);
  return total;
}

Status launch_collective(const CollArgs& a, const LaunchPlan& plan, cudaStream_t stream) {
  dim3 grid(plan.blocks), block(plan.threads);
  if (a.kind == kCollSendRecv) {
    int nb = sendrecv_blocks(a);
    if (nb == 0) return kSuccess;
    dev::sendrecv_kernel<<<nb, plan.threads, 0, stream>>>(a);
    return check_launch("sendrecv");
  }
  bool ok = true;
  if (a.kind == kCollAllReduce && a.algo == kAlgoNvls && a.nranks > 1) {
    if (a.dtype == kF32) dev::nvls_allreduce_kernel<float><<<grid, block, 0, stream>>>(a, plan.chunk_elems);
    else if (a.dtype == kBF16) dev::nvls_allreduce_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(a, plan.chunk_elems);
    else if (a.dtype == kF16) dev::nvls_allreduce_kernel<__half><<<grid, block, 0, stream>>>(a, plan.chunk_elems);
    else return fail(kInvalidArgument, "NVLS all-reduce supports fp32, fp16 and bf16 sums only");
    return check_launch("nvls allreduce");
  }
  if (a.kind == kCollAllReduce && a.algo == kAlgoWindow && a.nranks > 1 && a.mc_send && a.mc_recv && (a.redop == kSum || a.redop == kAvg) &&
      (a.dtype == kF32 || a.dtype == kBF16 || a.dtype == kF16) && a.dtype == a.out_dtype) {
    if (a.dtype == kF32) dev::nvls_window_allreduce_kernel<float><<<grid, block, 0, stream>>>(a);
    else if (a.dtype == kBF16) dev::nvls_window_allreduce_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(a);
    else dev::nvls_window_allreduce_kernel<__half><<<grid, block, 0, stream>>>(a);
    return check_launch("window allreduce (nvls)");
  }
  if (a.kind == kCollReduce && a.algo == kAlgoNvls && a.nranks > 2 && a.mc_stage) {
    if (a.dtype == kF32) dev::nvls_reduce_kernel<float><<<grid, block, 0, stream>>>(a, plan.chunk_elems);
    else if (a.dtype == kBF16) dev::nvls_reduce_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(a, plan.chunk_elems);
    else dev::nvls_reduce_kernel<__half><<<grid, block, 0, stream>>>(a, plan.chunk_elems);
    return check_launch("reduce (nvls)");
  }
  if (a.kind == kCollReduceScatter && a.algo == kAlgoWindow && a.nranks > 1 && a.mc_send) {
    if (a.dtype == kF32) dev::nvls_window_reducescatter_kernel<float><<<grid, block, 0, stream>>>(a);
    else if (a.dtype == kBF16) dev::nvls_window_reducescatter_kernel<__nv_bfloat16><<<grid, block, 0, stream>>>(a);
    else dev::nvls_window_reducescatter_kernel<__half><<<grid, block, 0, stream>>>(a);
    return check_launch("window reduce-scatter (nvls)");
  }
  if (a.kind == kCollAllGather && a.algo == kAlgoWindow && a.nranks > 1 && a.mc_recv) {
    dev::nvls_window_allgather_kernel<<<grid, block, 0, stream>>>(a);
    return check_launch("window all-gather (nvls)");
  }
  bool reducing = a.kind == kCollAllReduce || a.kind == kCollReduceScatter || a.kind == kCollReduce;
  if (reducing) {
    Status st = launch_reduce(a, plan, stream, nullptr, 0, &ok);
    if (st != kSuccess) return st;
  } else {
    dev::coll_kernel<unsigned char, unsigned char, kSum, false><<<grid, block, 0, stream>>>(a, plan.chunk_elems);
  }
  if (!ok) return fail(kInvalidArgument, "unsupported datatype %d -> %d with operator %d", a.dtype, a.out_dtype, a.redop);
  return check_launch("collective");
}

Status launch_collective_emu(const CollArgs* dev_all, const CollArgs& a, int nranks, const LaunchPlan& plan, cudaStream_t stream) {
  dim3 block(plan.threads);
  if (a.kind == kCollSendRecv) {
    // `plan.blocks` carries the maximum (entry, lane) count over the ranks.
    dim3 grid(plan.blocks, nranks);
    void* params[] = {(void*)&dev_all};
    return coop_launch(dev::sendrecv_kernel_emu, grid, block, params, stream, "sendrecv(emu)");
  }
  dim3 grid(plan.blocks, nranks);
  size_t chunk = plan.chunk_elems;
  void* params[] = {(void*)&dev_all, (void*)&chunk};
  bool ok = true;
  Status st = kSuccess;
  bool reducing = a.kind == kCollAllReduce || a.kind == kCollReduceScatter || a.kind == kCollReduce;
  if (reducing) {
    st = launch_reduce(a, plan, stream, dev_all, nranks, &ok);
  } else {
    st = coop_launch(dev::coll_kernel_emu<unsigned char, unsigned char, kSum, false>, grid, block, params, stream, "collective(emu)");
  }
  if (!ok) return fail(kInvalidArgument, "unsupported datatype %d -> %d with operator %d", a.dtype, a.out_dtype, a.redop);
  return st;
}


// ---- bounded-wait probe: what a kernel does when the flag it waits for never comes
namespace dev {
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns, uint32_t* status) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (!wait_flag_ge(flag, want, timeout_ns)) report_error(status, kDevBarrierTimeout, 0, 0, 0, want);
  }
}
}  // namespace dev

Status launch_wait_probe(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns, uint32_t* status, cudaStream_t stream) {
  dev::wait_probe_kernel<<<1, 32, 0, stream>>>(flag, want, timeout_ns, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kCudaError, "wait probe launch failed: %s", cudaGetErrorString(e));
  return kSuccess;
}

}  // namespace amem
