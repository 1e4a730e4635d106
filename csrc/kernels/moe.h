// MoE expert-parallel dispatch / combine (host-visible description).
//
// dispatch: every (token, choice) pair is written straight into the destination rank's
//           receive buffer at its final, expert-sorted row, so the routing permutation IS the
//           all-to-all: no local permute pass, no staging copy.  Row order inside an expert is
//           (source rank, token order) and is computed with scans, not atomics, so the layout
//           is identical from run to run.
// combine : the token owner pulls the k expert outputs of each token directly from the expert
//           ranks' output buffers (peer loads over NVLink), multiplies by the routing weights
//           and sums in fp32: the un-permute, the all-to-all back and the weighted sum in one
//           pass with no landing buffer.
#pragma once
#include <cuda_runtime.h>

#include "../core/status.h"
#include "coll_args.h"

namespace amem {

static const int kMoeMaxExperts = 256;   // CtrlBlock::xchg row length
static const int kMoeSegments = 128;     // CTAs of the count / scatter kernels

struct MoeArgs {
  CollArgs coll;
  int T, k, d;              // tokens on this rank, choices per token, hidden size (bf16 elements)
  int E;                    // experts over the whole communicator (E % nranks == 0)
  int capacity_rows;        // rows each rank's receive buffer can hold
  const void* x;            // bf16 [T, d]
  const int* topk_idx;      // int32 [T, k], global expert ids
  const float* topk_w;      // fp32 [T, k] (combine)
  char* recv[kMaxRanks];    // dispatch: every rank's receive buffer, bf16 [capacity_rows, d]
  char* ybuf[kMaxRanks];    // combine: every rank's expert-output buffer, bf16 [capacity_rows, d]
  void* out;                // combine: bf16 [T, d]
  // work buffers in this rank's own memory
  int* seg_hist;            // [kMoeSegments][E]
  int* seg_base;            // [kMoeSegments][E]  exclusive scan of seg_hist over segments
  int* send_off;            // [E]  first row, in the owner's buffer, of my pairs for expert e
  int* send_pos;            // [T*k] destination row of each pair (-1: dropped for capacity)
  int* expert_counts;       // [E / nranks] rows received per local expert
  int* expert_offsets;      // [E / nranks + 1] exclusive scan of expert_counts (last = total rows)
  int* dropped_rows;        // optional, one int: rows routed to this rank that did not fit capacity_rows
};

// Capacity.  A rank can be sent more rows than its buffers hold (routing is data dependent).
// That is a result of the call, not an error of the communicator: the rows that would land at
// or beyond capacity_rows are not sent (their send_pos is -1 and combine gives them weight 0),
// expert_counts / expert_offsets describe only the rows that were stored (so offsets never
// point past the buffer), and *dropped_rows says how many were left out on this rank.

Status launch_moe_dispatch(const MoeArgs& a, cudaStream_t stream);
Status launch_moe_combine(const MoeArgs& a, cudaStream_t stream);
// Emulated communicator: all ranks in one cooperative grid per phase.
Status launch_moe_dispatch_emu(const MoeArgs* host_all, const MoeArgs* dev_all, int nranks, cudaStream_t stream);
Status launch_moe_combine_emu(const MoeArgs* host_all, const MoeArgs* dev_all, int nranks, cudaStream_t stream);

}  // namespace amem
