// See moe_noalloc.h.  The scratch array and the host code that needs its device address live
// in this one file: in host code the array's name is only a stand-in symbol, never a device
// pointer, so the address is fetched with cudaGetSymbolAddress and handed to the kernels.
#include "moe_noalloc.h"

#include <cstddef>
#include <cstring>
#include <mutex>

#include "../core/log.h"
#include "../core/status.h"
#include "moe.h"

namespace amem {
namespace {

// the kernels size their shared-memory tables and the control block's exchange rows for kMoeMaxExperts
static_assert(kNoAllocMaxExperts <= kMoeMaxExperts, "the built-in scratch must not promise more experts than the kernels handle");

struct NoAllocScratch {
  CtrlBlock ctrl;                                       // protocol words of the one-rank run
  uint32_t status[kStatusWords];                        // error words (device memory here)
  int seg_hist[kMoeSegments * kNoAllocMaxExperts];      // per-segment expert histograms
  int seg_base[kMoeSegments * kNoAllocMaxExperts];      // their exclusive scans
  int send_off[kNoAllocMaxExperts];                     // first row of every expert
};

// ~330 KB per GPU, held from the moment the CUDA module of this library is loaded on that GPU (its
// first use there) to process exit.
static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

std::mutex g_mu;
NoAllocScratch* g_dev_ptr[64] = {nullptr};

// Once per device, with that device current.
Status scratch_for_current_device(NoAllocScratch** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(kCudaError, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(kInvalidArgument, "device index %d out of range", dev);
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_dev_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return fail(kCudaError, "cudaGetSymbolAddress of the built-in scratch failed on device %d: %s", dev, cudaGetErrorString(e));
    }
    g_dev_ptr[dev] = (NoAllocScratch*)p;
  }
  *out = g_dev_ptr[dev];
  return kSuccess;
}

}  // namespace
}  // namespace amem

using namespace amem;

extern "C" int amemMoePermuteNoAlloc(const void* x, const int* topk_idx, int T, int k, int d, int E, void* recv_x, int capacity_rows,
                                     int* expert_counts, int* expert_offsets, int* send_pos, cudaStream_t stream) {
  if (E > kNoAllocMaxExperts)
    return fail(kInvalidArgument, "amemMoePermuteNoAlloc: %d experts exceed the built-in scratch, which holds at most %d", E, kNoAllocMaxExperts);
  if (E <= 0 || T < 0 || k <= 0 || d <= 0 || d % 8 || capacity_rows <= 0)
    return fail(kInvalidArgument, "amemMoePermuteNoAlloc: bad shape T=%d k=%d d=%d (multiple of 8) E=%d capacity=%d", T, k, d, E, capacity_rows);
  if ((long long)T * k > 0x7fffffffLL) return fail(kInvalidArgument, "amemMoePermuteNoAlloc: T*k does not fit 31 bits");
  if (!x || !topk_idx || !recv_x || !expert_counts || !expert_offsets || !send_pos)
    return fail(kInvalidArgument, "amemMoePermuteNoAlloc: null buffer");
  NoAllocScratch* s = nullptr;
  Status st = scratch_for_current_device(&s);
  if (st != kSuccess) return st;
  // The array keeps the last call's contents: the ticket counter, the epochs and the error
  // words must start at zero (histograms, scans and offsets are fully rewritten by the kernels).
  cudaError_t e = cudaMemsetAsync(s, 0, offsetof(NoAllocScratch, seg_hist), stream);
  if (e != cudaSuccess) return fail(kCudaError, "cudaMemsetAsync on the built-in scratch: %s", cudaGetErrorString(e));
  MoeArgs a;
  memset(&a, 0, sizeof(a));
  a.coll.rank = 0;
  a.coll.nranks = 1;
  a.coll.ctrl[0] = &s->ctrl;
  a.coll.status = s->status;
  a.coll.timeout_ns = 1000000000ull;
  a.T = T;
  a.k = k;
  a.d = d;
  a.E = E;
  a.capacity_rows = capacity_rows;
  a.x = x;
  a.topk_idx = topk_idx;
  a.recv[0] = (char*)recv_x;
  a.seg_hist = s->seg_hist;
  a.seg_base = s->seg_base;
  a.send_off = s->send_off;
  a.send_pos = send_pos;
  a.expert_counts = expert_counts;
  a.expert_offsets = expert_offsets;
  return launch_moe_dispatch(a, stream);
}
