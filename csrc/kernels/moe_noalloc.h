// amemMoePermuteNoAlloc: single-GPU MoE routing permutation that allocates nothing.
//
// This entry point has no counterpart in the reference.  It exists for callers that must not,
// or cannot, obtain device memory at the moment they need to group tokens by expert:
//   * a process whose communicators are paused (ncclPause): the communicator's receive
//     buffers do not exist then and tracked allocations are refused until ncclResume;
//   * an engine that shares the GPU with another one and has already handed every byte it may
//     use to its own pool, so a cudaMalloc here could fail or eat the neighbour's budget;
//   * code that runs where an allocation would stall or break what surrounds it.
// It runs the same count / plan / scatter kernels as amemMoeDispatch on a one-rank
// "communicator", but the scratch they need (per-segment expert histograms and their scans,
// per-expert row offsets, one protocol control block and status words: about 330 KB) sits in a
// file-scope device array inside the library instead of in allocated memory.
//
// Limits and rules:
//   * at most kNoAllocMaxExperts experts; more is rejected with ncclInvalidArgument and a
//     message (amemLastError) -- the array is sized for exactly that many;
//   * the caller passes every input and output buffer, including recv_x (bf16
//     [capacity_rows, d]); rows that would land at or beyond capacity_rows are not written and
//     get send_pos = -1, and expert_counts / expert_offsets describe the rows that were stored
//     (expert_offsets[E] <= capacity_rows), so nothing indexed by them reaches past recv_x; a
//     caller that needs to know how many rows were left out counts the -1 entries of send_pos.
//     Nothing else can go wrong on the device in a one-rank run (there is no peer to wait for),
//     which is why the entry point has no device-side status to read back;
//   * every GPU that loads the library holds the array until the process exits;
//   * all calls on a device share the array and it keeps the previous call's contents; the
//     entry point clears what has to start at zero itself, but two calls that overlap on the
//     GPU (different streams without ordering) race on it: keep them stream-ordered;
//   * the first call on each device looks the array's device address up
//     (cudaGetSymbolAddress) and caches it; make that first call outside any stream capture.
#pragma once
#include <cuda_runtime.h>

namespace amem {
static const int kNoAllocMaxExperts = 256;
}

extern "C" {
// x: bf16 [T, d]; topk_idx: int32 [T, k] with expert ids in [0, E); recv_x: bf16
// [capacity_rows, d] receives the rows grouped by expert (token order inside an expert);
// expert_counts: int32 [E]; expert_offsets: int32 [E + 1]; send_pos: int32 [T * k], the row each
// (token, choice) went to.  d must be a multiple of 8.  Returns an ncclResult_t value.
int amemMoePermuteNoAlloc(const void* x, const int* topk_idx, int T, int k, int d, int E, void* recv_x, int capacity_rows,
                          int* expert_counts, int* expert_offsets, int* send_pos, cudaStream_t stream);
}
