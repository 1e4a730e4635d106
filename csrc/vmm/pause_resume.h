// Pause / resume engine.
//
// pause_scope : save STATEFUL local allocations to pinned host shadows (batched async
//               copies on a side stream), unmap + release every imported mapping, then
//               unbind multicast, unmap + release every local allocation, then an optional
//               cross-rank barrier so that on return the driver has really reclaimed the
//               pages (they survive until the last importer lets go).  Virtual addresses
//               stay reserved.
// resume_scope: create + map at the same addresses (+ multicast re-bind) and start the
//               host-to-device restores, agree across ranks that every create succeeded
//               (else everybody rolls back to PAUSED), exchange file descriptors in two
//               blocking phases (all sends, then all receives), import + map the peers'
//               memory at the old addresses (access granted once per contiguous window),
//               wait for the restores, and agree a second time — which is also the closing
//               barrier — that every rank got through (else, again, everybody rolls back).
//
// Reference behaviour being re-designed: amem_memPause / amem_memResume
// (amem_nccl_plugin/amem_nccl.cpp:467-574, 577-677): serial synchronous copies, one RPC
// per allocation per peer, a 500 ms polling loop for re-imports, no barrier, no rollback.
#pragma once
#include <cstdint>
#include <vector>

#include "backend.h"
#include "registry.h"

namespace amem {

// Cross-rank services the engine needs; implemented by the communicator over its socket
// mesh.  A process-level scope (no communicator) passes nullptr.
class PeerExchange {
 public:
  virtual ~PeerExchange() {}
  virtual int rank() const = 0;
  virtual int nranks() const = 0;
  virtual Status barrier() = 0;
  // Logical AND of `mine` over all ranks.
  virtual Status all_ok(bool mine, bool* all) = 0;
  // The same two in halves: `begin` only sends, `end` only receives.  A thread that serves
  // several communicators (or several ranks of one) begins all of them before it ends any, so
  // the exchanges overlap and ranks that share the thread cannot wait for each other.
  virtual Status barrier_begin() { return kSuccess; }
  virtual Status barrier_end() { return barrier(); }
  virtual Status vote_begin(bool mine) { pending_vote_ = mine; return kSuccess; }
  virtual Status vote_end(bool* all) { return all_ok(pending_vote_, all); }
  virtual Status send_fd(int to, uint32_t sym_id, uint64_t size, int fd) = 0;
  virtual Status recv_fd(int from, uint32_t* sym_id, uint64_t* size, int* fd) = 0;
  // Tells `to` that the handle of segment `sym_id` will not come (the export failed), so that
  // its receive returns at once instead of running into the deadline.
  virtual Status send_no_fd(int to, uint32_t sym_id) { (void)to; (void)sym_id; return kSuccess; }
  // Called at the start of every pause or resume pass; messages that an abandoned earlier pass
  // left behind are told apart from this pass's by it.
  virtual void begin_attempt() {}

 protected:
  bool pending_vote_ = true;
};

struct PauseResumeStats {
  // pause phases, microseconds of host wall clock
  double quiesce_us, offload_us, release_import_us, release_local_us, pause_barrier_us, pause_total_us;
  // resume phases
  double create_map_us, agree_us, exchange_us, import_us, preload_us, resume_barrier_us, resume_total_us;
  uint64_t bytes_offloaded, bytes_preloaded;
  uint64_t bytes_released_local, bytes_released_peer;
  uint64_t n_offload, n_release_local, n_release_peer;
  uint64_t free_before_pause, free_after_pause, free_after_resume;
};

struct EngineOptions {
  bool barrier = true;          // cross-rank barrier at the end of pause and of resume
  int offload_free_tag = -1;    // allocations with this caller tag are dropped without a copy
};

// One communicator (or the process-level allocations, owner 0) taking part in a pass.
struct EngineScope {
  uint64_t owner = 0;
  int dev = 0;
  PeerExchange* px = nullptr;      // nullptr: nothing to exchange (one rank, or process-level memory)
  EngineOptions opt;
  PauseResumeStats* stats = nullptr;
  Status result = kSuccess;        // outcome for this scope
};

// One pass over several scopes: every phase runs once for all of them (one quiesce, all saves
// queued together, all per-peer driver calls side by side, the cross-rank messages of every
// communicator sent before any is awaited), so a process with a world, a tensor-parallel and an
// expert-parallel communicator pays the exchange once, not three times.  Ranks of one
// communicator that share the calling thread are served by the same pass.
//
// Outcomes.  pause: a failure before anything was released leaves every scope as it was (still
// usable); later failures are reported but the pass completes, so every scope ends PAUSED.
// resume: per communicator, two agreements — after re-creating the local memory and after
// importing the peers' and restoring contents; if either fails on any rank, every rank of that
// communicator undoes the attempt and is PAUSED again, and ncclResume can be retried.  A scope is
// never left in between.  Returns the first scope's error; `result` of each scope has its own.
Status pause_scopes(Registry& reg, VmmBackend* be, std::vector<EngineScope>& scopes);
Status resume_scopes(Registry& reg, VmmBackend* be, std::vector<EngineScope>& scopes);

// Single-scope forms.
Status pause_scope(Registry& reg, VmmBackend* be, uint64_t owner, int dev, PeerExchange* px,
                   const EngineOptions& opt, PauseResumeStats* stats);
Status resume_scope(Registry& reg, VmmBackend* be, uint64_t owner, int dev, PeerExchange* px,
                    const EngineOptions& opt, PauseResumeStats* stats);

}  // namespace amem
