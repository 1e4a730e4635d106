// Host-side entry points of the kernel layer: launchers and the variant picker.
#pragma once
#include <cuda_runtime.h>

#include "../core/status.h"
#include "coll_args.h"

namespace amem {

// Launches one rank's kernel on `stream`.
Status launch_collective(const CollArgs& a, const LaunchPlan& plan, cudaStream_t stream);
// Launches every rank of an emulated (single-GPU) communicator as one cooperative grid.
// `dev_all` points to `nranks` CollArgs in device-readable memory; `a` is any rank's copy
// (used for type dispatch only).
// One thread waits, the way every collective kernel waits for a peer, until *flag >= want or
// timeout_ns have passed; a wait that runs out is recorded in `status` (host-visible words) like a
// collective's and the kernel returns normally.
Status launch_wait_probe(const uint32_t* flag, uint32_t want, unsigned long long timeout_ns, uint32_t* status, cudaStream_t stream);
Status launch_collective_emu(const CollArgs* dev_all, const CollArgs& a, int nranks, const LaunchPlan& plan, cudaStream_t stream);
int sendrecv_blocks(const CollArgs& a);

struct TunerInput {
  int kind;
  size_t count;       // elements, with the per-kind meaning of CollArgs::count
  int dtype, redop;
  int nranks;
  size_t stage_bytes, p2p_slot_bytes;
  bool nvls;          // multicast mapping available
  int max_blocks;     // upper bound for this communicator (emulated comms use a small one)
  int forced_algo;    // kAlgoAuto or a variant forced by AMEM_ALGO / the API
  bool window = false;      // all-reduce: both operands lie in registered windows at vector-aligned offsets
  bool window_mc = false;   // ... and the windows have multicast mappings
};

// Deterministic in its inputs: every rank, and the same rank before and after a pause,
// gets the same variant, grid and chunking, which keeps results bitwise reproducible.
LaunchPlan plan_collective(const TunerInput& in);

}  // namespace amem
