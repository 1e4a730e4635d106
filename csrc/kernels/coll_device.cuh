// Device-side building blocks of the collective kernels: system-scope flag accesses,
// the bounded block-level cross-rank barrier, 16-byte vector copy / reduce loops and the
// element-type traits.  Everything here is plain sm_100a CUDA C++ with inline PTX for the
// memory-model sensitive accesses; no library device code is used.
// Reference parity: none -- the reference's waits are on the host and several are unbounded
// (amem_nccl_plugin/amem_nccl.cpp:659-662, gmm_client_impl.cpp:108-111,182-187).
#pragma once
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "coll_args.h"

namespace amem {
namespace dev {

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_volatile(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// One flag-in-data packet: 4 bytes of payload and the operation's flag in ONE 8-byte store / load,
// so the two can never be seen apart.
__device__ __forceinline__ void ll_store(void* p, uint32_t data, uint32_t flag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(data), "r"(flag) : "memory");
}
__device__ __forceinline__ void ll_load(const void* p, uint32_t* data, uint32_t* flag) {
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(*data), "=r"(*flag) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Records the first device-side error of a launch in the host-mapped status words.
__device__ __forceinline__ void report_error(uint32_t* status, uint32_t code, int rank, int peer, int block, uint32_t epoch) {
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = (uint32_t)rank;
    status[2] = (uint32_t)peer;
    status[3] = (uint32_t)block;
    status[4] = epoch;
    __threadfence_system();
  }
}

// Spins until *flag has reached `want` (wrap-safe) or the time budget is spent.
// Returns false on timeout; the caller records the error and carries on without waiting.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
    }
    if (globaltimer_ns() - t0 > timeout_ns) return false;
  }
}

// Polls one packet until it carries `flag` or the time budget is spent (false).
__device__ __forceinline__ bool ll_wait(const void* p, uint32_t flag, uint32_t* data, unsigned long long timeout_ns) {
  uint32_t f;
  ll_load(p, data, &f);
  if (f == flag) return true;
  unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      ll_load(p, data, &f);
      if (f == flag) return true;
    }
    if (globaltimer_ns() - t0 > timeout_ns) return false;
  }
}

// Per-launch view of one rank's protocol state.
struct Proto {
  const CollArgs* a;
  CtrlBlock* me;
  uint32_t epoch;   // this block's epoch (valid in every thread)
  uint32_t opseq;
  int block;        // block index within this rank's part of the grid
  int nblocks;
  int* abort_flag;  // shared memory, one per block
};

__device__ __forceinline__ void proto_begin(Proto& p, const CollArgs& a, int block, int nblocks, int* s_abort) {
  p.a = &a;
  p.me = a.ctrl[a.rank];
  p.block = block;
  p.nblocks = nblocks;
  p.abort_flag = s_abort;
  if (threadIdx.x == 0) *s_abort = 0;
  p.epoch = ld_volatile(&p.me->epoch[block]);
  p.opseq = ld_volatile(&p.me->opseq);
  __syncthreads();
}

// All threads of the block call this.  Makes every store issued by the block so far visible
// to the peers before the flag, then waits for the same-index block of every peer.
__device__ __forceinline__ void block_barrier(Proto& p) {
  const CollArgs& a = *p.a;
  p.epoch += 1;
  __syncthreads();
  int t = threadIdx.x;
  if (t < a.nranks && t != a.rank) {
    __threadfence_system();
    st_release_sys(&a.ctrl[t]->flags[p.block][a.rank], p.epoch);
    if (*(volatile int*)p.abort_flag == 0) {
      if (!wait_flag_ge(&p.me->flags[p.block][t], p.epoch, a.timeout_ns)) {
        report_error(a.status, kDevBarrierTimeout, a.rank, t, p.block, p.epoch);
        *(volatile int*)p.abort_flag = 1;
      }
    }
  }
  __syncthreads();
}

// Stores the block's epoch back and bumps the operation counter once per launch.
__device__ __forceinline__ void proto_end(Proto& p) {
  __syncthreads();
  if (threadIdx.x == 0) {
    p.me->epoch[p.block] = p.epoch;
    __threadfence();
    uint32_t ticket = atomicAdd(&p.me->done_blocks, 1u);
    if (ticket == (uint32_t)p.nblocks - 1) {
      p.me->done_blocks = 0;
      p.me->opseq = p.opseq + 1;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------- element traits
template <typename T> struct Acc { using type = T; };
template <> struct Acc<__half> { using type = float; };
template <> struct Acc<__nv_bfloat16> { using type = float; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type to_acc(T v) { return v; }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, typename A> __device__ __forceinline__ T from_acc(A v) { return (T)v; }
template <> __device__ __forceinline__ __half from_acc<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_acc<__half, double>(double v) { return __float2half_rn((float)v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, double>(double v) { return __float2bfloat16_rn((float)v); }

template <int OP, typename A> __device__ __forceinline__ A combine(A x, A y) {
  if (OP == kSum || OP == kAvg) return x + y;
  if (OP == kProd) return x * y;
  if (OP == kMax) return x > y ? x : y;
  return x < y ? x : y;
}

template <typename A> __device__ __forceinline__ A apply_scale(A v, float s) { return (A)((double)v * (double)s); }
template <> __device__ __forceinline__ float apply_scale<float>(float v, float s) { return v * s; }

__device__ __forceinline__ void block_sync() { __syncthreads(); }
__device__ __forceinline__ int thread_index() { return threadIdx.x; }
__device__ __forceinline__ void fence_system() { __threadfence_system(); }

// ---------------------------------------------------------------- copy / reduce loops
// Range [lo, hi) in bytes is this block's share; lo is a multiple of 16.
__device__ __forceinline__ void block_range(size_t total_bytes, int block, int nblocks, size_t* lo, size_t* hi) {
  size_t nvec = (total_bytes + 15) / 16;
  size_t per = (nvec + nblocks - 1) / nblocks;
  size_t l = (size_t)block * per * 16, h = l + per * 16;
  if (l > total_bytes) l = total_bytes;
  if (h > total_bytes) h = total_bytes;
  *lo = l;
  *hi = h;
}

// The same split for a piece of `avail_bytes` of a chunked message whose full chunks have
// `full_bytes`: the ranges are those of a FULL chunk, cut off at what this chunk really has.
// Block b then touches the same staging bytes in every chunk, so the per-block barriers and
// credits (which order block b of one rank only against block b of the others) also cover a
// short last chunk; splitting `avail_bytes` itself would move the ranges and let block b of one
// rank write what block b' of another is still reading from two chunks earlier.
__device__ __forceinline__ void block_range_clip(size_t full_bytes, size_t avail_bytes, int block, int nblocks, size_t* lo, size_t* hi) {
  block_range(full_bytes, block, nblocks, lo, hi);
  if (*lo > avail_bytes) *lo = avail_bytes;
  if (*hi > avail_bytes) *hi = avail_bytes;
}

// A lane is the slice of a block's threads that executes one loop: the whole block, or the
// "push" / "drain" group of warps when a collective overlaps its two phases.
struct Lane {
  int tid, nt;
  int bar;   // named barrier of the group (0 = the whole block)
};
__device__ __forceinline__ Lane full_lane() { return Lane{(int)threadIdx.x, (int)blockDim.x, 0}; }
__device__ __forceinline__ bool lanes_split(Lane a) { return a.nt != (int)blockDim.x; }
// Barrier among the threads of one lane only.
__device__ __forceinline__ void lane_sync(Lane ln) {
  if (ln.bar == 0) __syncthreads();
  else asm volatile("bar.sync %0, %1;" ::"r"(ln.bar), "r"(ln.nt) : "memory");
}

// Splits the block's warps: the first `push_sixteenths`/16 of them push over NVLink, the rest
// drain staging into the user's buffer.  Without overlap every thread does both in turn.
__device__ __forceinline__ void split_lanes(bool overlap, int push_sixteenths, Lane* push, Lane* drain, bool* do_push, bool* do_drain) {
  if (!overlap) {
    *push = *drain = full_lane();
    *do_push = *do_drain = true;
    return;
  }
  int nwarps = blockDim.x / 32;
  int wp = nwarps * push_sixteenths / 16;
  if (wp < 1) wp = 1;
  if (wp > nwarps - 1) wp = nwarps - 1;
  int t = threadIdx.x;
  *do_push = t < wp * 32;
  *do_drain = !*do_push;
  *push = Lane{t, wp * 32, 1};
  *drain = Lane{t - wp * 32, (nwarps - wp) * 32, 2};
}

__device__ __forceinline__ void copy_span(char* dst, const char* src, size_t bytes, Lane ln) {
  if (bytes == 0) return;
  int t = ln.tid, nt = ln.nt;
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    size_t nvec = bytes / 16;
    const uint4* s = (const uint4*)src;
    uint4* d = (uint4*)dst;
    size_t i = t;
    // eight independent 16-byte loads in flight per thread: with only part of the block's warps
    // on a copy (the collectives split their warps), HBM latency needs that much to be covered
    for (; i + 7 * (size_t)nt < nvec; i += 8 * (size_t)nt) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = s[i + (size_t)j * nt];
#pragma unroll
      for (int j = 0; j < 8; ++j) d[i + (size_t)j * nt] = v[j];
    }
    for (; i < nvec; i += nt) d[i] = s[i];
    for (size_t b = nvec * 16 + t; b < bytes; b += nt) dst[b] = src[b];
  } else {
    for (size_t b = t; b < bytes; b += nt) dst[b] = src[b];
  }
}

// Copy into the multicast mapping: ONE store per 16 bytes that the NVSwitch replicates into
// every rank's memory (multimem.st), instead of one store per peer.  16-byte aligned spans only.
__device__ __forceinline__ bool mc_copy_ok(const char* dst_mc, const char* src, size_t bytes) {
  return dst_mc != nullptr && ((((uintptr_t)dst_mc | (uintptr_t)src) & 15) == 0) && (bytes % 16 == 0);
}
__device__ __forceinline__ void copy_span_mc(char* dst_mc, const char* src, size_t bytes, Lane ln) {
  const uint4* s = (const uint4*)src;
  size_t nvec = bytes / 16, nt = ln.nt, i = ln.tid;
  for (; i + 7 * nt < nvec; i += 8 * nt) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = s[i + j * nt];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst_mc + (i + j * nt) * 16), "r"(v[j].x), "r"(v[j].y), "r"(v[j].z), "r"(v[j].w) : "memory");
  }
  for (; i < nvec; i += nt) {
    uint4 v = s[i];
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst_mc + i * 16), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
}

// out[i] = cast(scale * OP_r(slot_r[i]))  for i in [0, n); reduction order is rank 0..nslots-1,
// accumulated in Acc<TI> (fp32 for 16-bit floats) and rounded once.
template <typename TI, typename TO, int OP>
__device__ __forceinline__ void reduce_span(TO* out, const TI* const* slots, int nslots, size_t n, float scale, bool has_scale, Lane ln) {
  using A = typename Acc<TI>::type;
  constexpr int VI = 16 / sizeof(TI);
  int t = ln.tid, nt = ln.nt;
  bool aligned = (((uintptr_t)out) % (VI * sizeof(TO)) == 0);
  for (int r = 0; r < nslots; ++r) aligned = aligned && (((uintptr_t)slots[r] & 15) == 0);
  size_t nvec = aligned ? n / VI : 0;
  // The slot pointers sit in the caller's local memory and the stores to `out` could alias them as
  // far as the compiler knows: copy them into registers once instead of re-reading them per vector.
  const uint4* sp[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) sp[r] = r < nslots ? (const uint4*)slots[r] : nullptr;
  auto one = [&](size_t i, const uint4* raw, auto nmax) {  // nmax: length of raw[], a compile-time constant
    constexpr int NM = decltype(nmax)::value;
    A acc[VI];
    {
      const TI* e = (const TI*)&raw[0];
#pragma unroll
      for (int k = 0; k < VI; ++k) acc[k] = to_acc<TI>(e[k]);
    }
#pragma unroll
    for (int r = 1; r < NM; ++r) {
      if (r < nslots) {
        const TI* e = (const TI*)&raw[r];
#pragma unroll
        for (int k = 0; k < VI; ++k) acc[k] = combine<OP, A>(acc[k], to_acc<TI>(e[k]));
      }
    }
    alignas(16) TO res[VI];
#pragma unroll
    for (int k = 0; k < VI; ++k) {
      A v = has_scale ? apply_scale<A>(acc[k], scale) : acc[k];
      res[k] = from_acc<TO, A>(v);
    }
    if (sizeof(TO) * VI == 16) {
      ((uint4*)out)[i] = *(const uint4*)res;
    } else if (sizeof(TO) * VI == 32) {
      ((uint4*)out)[2 * i] = ((const uint4*)res)[0];
      ((uint4*)out)[2 * i + 1] = ((const uint4*)res)[1];
    } else if (sizeof(TO) * VI == 8) {
      ((uint2*)out)[i] = *(const uint2*)res;
    } else {
#pragma unroll
      for (int k = 0; k < VI; ++k) out[i * VI + k] = res[k];
    }
  };
  size_t i = t;
  // up to four ranks: two output vectors per thread per trip, so that eight independent 16-byte
  // loads are in flight either way (with more ranks a second vector would not fit the registers)
  if (nslots <= kMaxRanks / 2) {
    for (; i + (size_t)nt < nvec; i += 2 * (size_t)nt) {
      uint4 ra[kMaxRanks / 2], rb[kMaxRanks / 2];
#pragma unroll
      for (int r = 0; r < kMaxRanks / 2; ++r) {
        if (r < nslots) {
          ra[r] = sp[r][i];
          rb[r] = sp[r][i + nt];
        }
      }
      one(i, ra, std::integral_constant<int, kMaxRanks / 2>());
      one(i + nt, rb, std::integral_constant<int, kMaxRanks / 2>());
    }
  }
  for (; i < nvec; i += nt) {
    uint4 ra[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < nslots) ra[r] = sp[r][i];
    one(i, ra, std::integral_constant<int, kMaxRanks>());
  }
  for (size_t i = nvec * VI + t; i < n; i += nt) {
    A acc = to_acc<TI>(slots[0][i]);
    for (int r = 1; r < nslots; ++r) acc = combine<OP, A>(acc, to_acc<TI>(slots[r][i]));
    if (has_scale) acc = apply_scale<A>(acc, scale);
    out[i] = from_acc<TO, A>(acc);
  }
}

}  // namespace dev
}  // namespace amem
