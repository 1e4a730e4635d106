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
//               memory at the old addresses, wait for the restores and barrier.
//
// Reference behaviour being re-designed: amem_memPause / amem_memResume
// (amem_nccl_plugin/amem_nccl.cpp:467-574, 577-677): serial synchronous copies, one RPC
// per allocation per peer, a 500 ms polling loop for re-imports, no barrier, no rollback.
#pragma once
#include <cstdint>

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
  virtual Status send_fd(int to, uint32_t sym_id, uint64_t size, int fd) = 0;
  virtual Status recv_fd(int from, uint32_t* sym_id, uint64_t* size, int* fd) = 0;
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

Status pause_scope(Registry& reg, VmmBackend* be, uint64_t owner, int dev, PeerExchange* px,
                   const EngineOptions& opt, PauseResumeStats* stats);
Status resume_scope(Registry& reg, VmmBackend* be, uint64_t owner, int dev, PeerExchange* px,
                    const EngineOptions& opt, PauseResumeStats* stats);

}  // namespace amem
