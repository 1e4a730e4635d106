// Per-process registry of every VMM allocation the library owns or has imported.
//
// Counterpart of the reference's allocTable/handleTable pair and amem_allocMdata record
// (amem_nccl_plugin/gmm_client.h:136-152, amem_nccl.h:87-138).  Differences by design:
//  * importers are recorded when the communicator builds a symmetric segment (the library
//    creates both sides), so no register-peer RPC is needed afterwards;
//  * each record carries a category: STATEFUL contents are saved to a host shadow on pause,
//    SCRATCH contents are dead between collectives and are dropped without a copy;
//  * all mutation happens under one mutex and counters are atomics (the reference mutates
//    its tables from a worker thread without a lock, amem_nccl.cpp:303,365,391).
#pragma once
#include <atomic>
#include <cstdint>
#include <functional>
#include <map>
#include <mutex>
#include <vector>

#include "../core/status.h"

namespace amem {

enum MemState : int { kMemInvalid = 0, kMemAlloc = 1, kMemOffloading = 2, kMemHole = 3, kMemPreloading = 4 };
// Process/communicator life cycle (docs/images/process_status.png of the reference).
enum RunState : int { kRunInit = 0, kRunPausing = 1, kRunPaused = 2, kRunResuming = 3, kRunResumed = 4 };

// Same numbering as the reference's amem_allocType (amem_nccl.h:52-64).
enum AllocType : int { kLocalPosix = 0, kLocalFabric = 1, kLocalSymm = 2, kPeerPosix = 3, kPeerFabric = 4, kPeerSymm = 5 };
inline bool from_peer(int type) { return type > kLocalSymm; }

// Caller tags keep the reference's numbering (amem_nccl.h:67-80) so that ncclMemStats
// output lines up with its "caller_N" lines.
enum CallerTag : int { kTagDefault = 0, kTagP2P = 1, kTagFabric = 2, kTagPosix = 3, kTagSymm = 4, kTagNvls = 5, kTagP2PPeer = 7, kTagProxy = 9, kTagSymmPeer = 10, kMaxCaller = 16 };

// kStateful: saved to a host shadow on pause; kScratch: dropped without a copy; kResident: small
// protocol state that stays mapped through a pause (not released, not re-imported).
enum Category : int { kStateful = 0, kScratch = 1, kResident = 2 };

struct Allocation {
  uint64_t va = 0;
  size_t size = 0;
  uint64_t handle = 0;      // backend physical handle; 0 while in HOLE state
  int dev = 0;
  int type = kLocalPosix;
  int category = kStateful;
  int tag = kTagDefault;
  uint64_t owner = 0;       // communicator id, 0 = process-level (ncclMemAlloc)
  uint32_t sym_id = 0;      // symmetric segment id inside the owner
  int exporter_rank = -1;   // imported records: owner-comm rank that owns the memory
  uint32_t importers = 0;   // local records: bitmap of owner-comm ranks that mapped it
  uint64_t mc_handle = 0;   // multicast object this allocation is bound to (0 = none)
  size_t mc_offset = 0;
  // [clear_offset, clear_offset + clear_bytes) must read zero whenever fresh physical memory is
  // mapped here (protocol areas whose stale contents could be mistaken for signals)
  size_t clear_offset = 0, clear_bytes = 0;
  void* shadow = nullptr;   // pinned host copy, allocated at first pause, kept afterwards
  int state = kMemInvalid;
};

struct MemStats {
  uint64_t bytes_by_tag[kMaxCaller];
  uint64_t stateful_bytes, scratch_bytes, imported_bytes, multicast_bytes;
  uint64_t live_bytes, paused_bytes;   // physical memory mapped now / released by pause
  uint64_t shadow_bytes;               // pinned host memory held for shadows
  uint64_t n_local, n_imported;
  uint64_t pause_count, resume_count;
  int group_id;
  int paused;                          // 1 when the whole process is paused
};

class Registry {
 public:
  static Registry& instance();

  // Rejects (kInvalidUsage) when the owner or the process is paused, like the reference
  // (amem_nccl.cpp:133-137).
  Status add(const Allocation& a);
  Status remove(uint64_t va);
  bool find(uint64_t va, Allocation* out);
  bool find_by_handle(uint64_t handle, Allocation* out);
  // Finds the record whose [va, va+size) contains `addr`.
  bool find_containing(uint64_t addr, Allocation* out);
  Status add_importer(uint64_t va, int rank);
  Status update(const Allocation& a);   // replace the record with the same va

  // Snapshot of records with the given owner (all owners when `any_owner`), sorted by
  // (owner, sym_id, exporter_rank, va) so every rank walks them in the same order.
  std::vector<Allocation> snapshot(uint64_t owner, bool any_owner);

  void stats(MemStats* out);
  void dump_stats(bool verbose);

  // Group id is settable only before the first tracked allocation (amem_nccl.cpp:679-694).
  Status set_group_id(int id);
  int group_id();

  // Pause bookkeeping per owner.  The process counts as paused when pause was requested
  // for all owners and not yet resumed.
  void set_owner_state(uint64_t owner, int run_state);
  int owner_state(uint64_t owner);
  void set_process_paused(bool p);
  bool process_paused();
  bool is_paused(uint64_t owner) { return process_paused() || owner_state(owner) == kRunPaused || owner_state(owner) == kRunPausing || owner_state(owner) == kRunResuming; }
  void forget_owner(uint64_t owner);
  void count_pause() { pause_count_.fetch_add(1); }
  void count_resume() { resume_count_.fetch_add(1); }
  size_t size();

 private:
  Registry();
  std::mutex mu_;
  std::map<uint64_t, Allocation> by_va_;
  std::map<uint64_t, uint64_t> by_handle_;
  std::map<uint64_t, int> owner_state_;
  bool process_paused_ = false;
  bool ever_added_ = false;
  int group_id_ = 0;
  std::atomic<uint64_t> pause_count_{0}, resume_count_{0};
};

}  // namespace amem
