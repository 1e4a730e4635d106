// Host executor: runs the collective protocol of coll_bodies.inl on the calling thread for
// backends whose "device memory" is host shared memory (the mock backend).  Flags are the
// same words in the same control blocks, accessed with acquire/release atomics; a rank is a
// single block of a single thread.  Used by the CPU test-suite to exercise communicator
// set-up, the push protocol, grouped send/recv and pause/resume without a GPU.
#include <sched.h>

#include <cstring>

#include "../core/log.h"
#include "coll_args.h"
#include "dispatch.h"

namespace amem {
namespace hostx {

inline uint32_t ld_acquire_sys(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline void st_release_sys(uint32_t* p, uint32_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
inline uint32_t ld_volatile(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_RELAXED); }
inline void ll_store(void* p, uint32_t data, uint32_t flag) {
  __atomic_store_n((uint64_t*)p, (uint64_t)data | ((uint64_t)flag << 32), __ATOMIC_RELEASE);
}
inline void ll_load(const void* p, uint32_t* data, uint32_t* flag) {
  uint64_t v = __atomic_load_n((const uint64_t*)p, __ATOMIC_ACQUIRE);
  *data = (uint32_t)v;
  *flag = (uint32_t)(v >> 32);
}
inline void block_sync() {}
inline int thread_index() { return 0; }
inline void fence_system() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }

inline void report_error(uint32_t* status, uint32_t code, int rank, int peer, int block, uint32_t epoch) {
  uint32_t expect = 0;
  if (__atomic_compare_exchange_n(status, &expect, code, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) {
    status[1] = (uint32_t)rank;
    status[2] = (uint32_t)peer;
    status[3] = (uint32_t)block;
    status[4] = epoch;
  }
}

inline bool wait_flag_ge(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
  double t0 = now_ms();
  for (unsigned spins = 0;; ++spins) {
    if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
    if ((spins & 63) == 63) {
      if ((now_ms() - t0) * 1e6 > (double)timeout_ns) return false;
      sched_yield();
    }
  }
}

inline bool ll_wait(const void* p, uint32_t flag, uint32_t* data, unsigned long long timeout_ns) {
  uint32_t f;
  double t0 = now_ms();
  for (unsigned spins = 0;; ++spins) {
    ll_load(p, data, &f);
    if (f == flag) return true;
    if ((spins & 63) == 63) {
      if ((now_ms() - t0) * 1e6 > (double)timeout_ns) return false;
      sched_yield();
    }
  }
}

struct Proto {
  const CollArgs* a;
  CtrlBlock* me;
  uint32_t epoch;
  uint32_t opseq;
  int block;
  int nblocks;
  int* abort_flag;
};

inline void proto_begin(Proto& p, const CollArgs& a, int block, int nblocks, int* s_abort) {
  p.a = &a;
  p.me = a.ctrl[a.rank];
  p.block = block;
  p.nblocks = nblocks;
  p.abort_flag = s_abort;
  *s_abort = 0;
  p.epoch = ld_volatile(&p.me->epoch[block]);
  p.opseq = ld_volatile(&p.me->opseq);
}

inline void block_barrier(Proto& p) {
  const CollArgs& a = *p.a;
  p.epoch += 1;
  for (int t = 0; t < a.nranks; ++t)
    if (t != a.rank) st_release_sys(&a.ctrl[t]->flags[p.block][a.rank], p.epoch);
  for (int t = 0; t < a.nranks; ++t) {
    if (t == a.rank || *p.abort_flag) continue;
    if (!wait_flag_ge(&p.me->flags[p.block][t], p.epoch, a.timeout_ns)) {
      report_error(a.status, kDevBarrierTimeout, a.rank, t, p.block, p.epoch);
      *p.abort_flag = 1;
    }
  }
}

inline void proto_end(Proto& p) {
  p.me->epoch[p.block] = p.epoch;
  uint32_t ticket = __atomic_fetch_add(&p.me->done_blocks, 1u, __ATOMIC_ACQ_REL);
  if (ticket == (uint32_t)p.nblocks - 1) {
    p.me->done_blocks = 0;
    p.me->opseq = p.opseq + 1;
  }
}

inline void block_range(size_t total_bytes, int block, int nblocks, size_t* lo, size_t* hi) {
  size_t nvec = (total_bytes + 15) / 16;
  size_t per = (nvec + nblocks - 1) / nblocks;
  size_t l = (size_t)block * per * 16, h = l + per * 16;
  if (l > total_bytes) l = total_bytes;
  if (h > total_bytes) h = total_bytes;
  *lo = l;
  *hi = h;
}
inline void block_range_clip(size_t full_bytes, size_t avail_bytes, int block, int nblocks, size_t* lo, size_t* hi) {
  block_range(full_bytes, block, nblocks, lo, hi);
  if (*lo > avail_bytes) *lo = avail_bytes;
  if (*hi > avail_bytes) *hi = avail_bytes;
}

struct Lane {
  int tid, nt;
  int bar;
};
inline Lane full_lane() { return Lane{0, 1, 0}; }
inline bool lanes_split(Lane) { return false; }
inline void lane_sync(Lane) {}
inline void split_lanes(bool, int, Lane* push, Lane* drain, bool* do_push, bool* do_drain) {
  *push = *drain = full_lane();  // one thread plays both groups, one after the other
  *do_push = *do_drain = true;
}
inline bool mc_copy_ok(const char*, const char*, size_t) { return false; }  // no multicast on the host
inline void copy_span_mc(char*, const char*, size_t, Lane) {}
inline void copy_span(char* dst, const char* src, size_t bytes, Lane) {
  if (bytes) memmove(dst, src, bytes);
}

template <typename T> struct Acc { using type = T; };
template <> struct Acc<__half> { using type = float; };
template <> struct Acc<__nv_bfloat16> { using type = float; };
template <typename T> inline typename Acc<T>::type to_acc(T v) { return v; }
template <> inline float to_acc<__half>(__half v) { return __half2float(v); }
template <> inline float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T, typename A> inline T from_acc(A v) { return (T)v; }
template <> inline __half from_acc<__half, float>(float v) { return __float2half_rn(v); }
template <> inline __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }

template <int OP, typename A> inline A combine(A x, A y) {
  if (OP == kSum || OP == kAvg) return x + y;
  if (OP == kProd) return x * y;
  if (OP == kMax) return x > y ? x : y;
  return x < y ? x : y;
}
template <typename A> inline A apply_scale(A v, float s) { return (A)((double)v * (double)s); }
template <> inline float apply_scale<float>(float v, float s) { return v * s; }

template <typename TI, typename TO, int OP>
inline void reduce_span(TO* out, const TI* const* slots, int nslots, size_t n, float scale, bool has_scale, Lane) {
  using A = typename Acc<TI>::type;
  for (size_t i = 0; i < n; ++i) {
    A acc = to_acc<TI>(slots[0][i]);
    for (int r = 1; r < nslots; ++r) acc = combine<OP, A>(acc, to_acc<TI>(slots[r][i]));
    if (has_scale) acc = apply_scale<A>(acc, scale);
    out[i] = from_acc<TO, A>(acc);
  }
}

#define AMEM_FN inline
#define AMEM_BODY inline
#include "coll_bodies.inl"
#undef AMEM_FN
#undef AMEM_BODY

}  // namespace hostx

int host_run_collective(const CollArgs& a, const LaunchPlan& plan) {
  int s_abort = 0;
  if (a.kind == kCollSendRecv) {
    // One thread plays every (entry, lane) block.  Sends go first: a slot-sized piece fits the
    // two-deep credit window, larger transfers interleave round by round with the receives.
    size_t slot = a.p2p_slot_bytes;
    int lanes[2 * kMaxRanks];
    size_t max_rounds = 0;
    for (int e = 0; e < a.n_p2p; ++e) {
      lanes[e] = p2p_lanes(a.p2p[e].bytes, slot, a.p2p_max_lanes);
      size_t rounds = (a.p2p[e].bytes + (size_t)lanes[e] * slot - 1) / ((size_t)lanes[e] * slot);
      if (rounds > max_rounds) max_rounds = rounds;
    }
    // Execute round by round so that a single thread never waits on credit it must itself
    // return: round k of every send, then round k of every receive.
    for (size_t k = 0; k < max_rounds; ++k) {
      for (int pass = 0; pass < 2; ++pass) {
        for (int e = 0; e < a.n_p2p; ++e) {
          if ((a.p2p[e].is_send != 0) != (pass == 0)) continue;
          size_t rb = (size_t)lanes[e] * slot;
          if (k * rb >= a.p2p[e].bytes) continue;
          CollArgs one = a;
          one.n_p2p = 1;
          one.p2p[0] = a.p2p[e];
          size_t len = a.p2p[e].bytes - k * rb < rb ? a.p2p[e].bytes - k * rb : rb;
          if (one.p2p[0].is_send) one.p2p[0].src = (const char*)a.p2p[e].src + k * rb;
          else one.p2p[0].dst = (char*)a.p2p[e].dst + k * rb;
          one.p2p[0].bytes = len;
          int use = (int)((len + slot - 1) / slot);
          for (int lane = 0; lane < use; ++lane) hostx::body_sendrecv(one, 0, lane, lanes[e], &s_abort);
        }
      }
    }
    return s_abort ? kDevP2PTimeout : kDevOk;
  }
  bool ok = true;
  bool reducing = a.kind == kCollAllReduce || a.kind == kCollReduceScatter || a.kind == kCollReduce;
  if (reducing) {
#define HOST_CALL(TI, TO, OP) hostx::run_body<TI, TO, OP, true>(a, 0, 1, &s_abort, plan.chunk_elems)
    AMEM_DISPATCH_REDUCE(a.dtype, a.out_dtype, a.redop, HOST_CALL);
#undef HOST_CALL
  } else {
    hostx::run_body<unsigned char, unsigned char, kSum, false>(a, 0, 1, &s_abort, plan.chunk_elems);
  }
  if (!ok) return kDevBadArgs;
  return s_abort ? kDevBarrierTimeout : kDevOk;
}

}  // namespace amem
