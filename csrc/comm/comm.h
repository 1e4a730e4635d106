// Communicator: ranks, socket mesh, symmetric VMM segments (control + staging, optionally
// bound to an NVLink multicast object), launch of the collectives, pause / resume.
//
// In the reference the communicator is NCCL's own and AMem only learns about its memory
// through ~25 hooks patched into NCCL (nccl_patch/nccl_2.27.5-1.diff:231-684).  Here the
// library builds the communicator itself, so every allocation is born in the registry with
// its importers known, and there is exactly one physical allocation per segment per rank
// (the reference's 8-rank run re-created 549 separate allocations on every resume).
#pragma once
#include <condition_variable>
#include <memory>
#include <mutex>
#include <vector>

#include "../ipc/rendezvous.h"
#include "../kernels/coll_args.h"
#include "../vmm/backend.h"
#include "../vmm/pause_resume.h"
#include "../vmm/registry.h"

typedef struct CUstream_st* cudaStream_t;

namespace amem {

struct Segment {
  uint32_t sym_id = 0;
  size_t size = 0;
  int category = kStateful;
  int tag = kTagP2P;
  uint64_t window = 0;            // reserved VA window of nranks * size
  uint64_t va[kMaxRanks] = {0};   // where each rank's memory is mapped in THIS process
  uint64_t mc_handle = 0;         // multicast object (0 = none)
  uint64_t mc_va = 0;             // VA of the multicast mapping
};

// A registered window: memory from ncclMemAlloc that every rank of the communicator has mapped
// (and, with NVLS, bound to one multicast object), so collectives can work on it in place.
struct Window {
  uint64_t base = 0;     // the user's address of this rank's memory
  size_t size = 0;       // bytes (the whole allocation)
  Segment seg;           // seg.va[r]: rank r's memory as mapped here (seg.va[rank] == base); seg.mc_va: multicast mapping
};

class EmuGroup;

struct CommConfig {
  size_t stage_bytes = 0;      // 0 = default for the backend
  size_t p2p_slot_bytes = 0;
  int nvls = -1;               // -1 auto, 0 off, 1 on when supported
  int max_blocks = 0;          // 0 = default
};

class Comm {
 public:
  static Status create(const UniqueId& id, int nranks, int rank, const CommConfig& cfg, VmmBackend* be, Comm** out);
  // Collective over the parent.  color < 0 yields *out == nullptr.
  Status split(int color, int key, const CommConfig& cfg, Comm** out);
  // New communicator over the ranks of this one that are NOT in `exclude` (ncclCommShrink); only
  // the surviving ranks call it, the excluded ones may be gone.
  Status shrink(const int* exclude, int n_exclude, const CommConfig& cfg, Comm** out);
  // Debug guard (AMEM_CANARY=1): one extra granule after the staging layout is kept at zero; a
  // kernel that writes past its region shows up here.  Checked before every pause, at destroy
  // and on request; kInternalError names the first dirty offset.
  Status check_canary();
  size_t canary_bytes() const { return canary_bytes_; }
  Status debug_dirty_canary();  // test hook: writes one non-zero word into the guard
  Status destroy();
  void abort();

  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  int device() const { return dev_; }
  // Registry owner key: unique per rank object, because several ranks of one communicator may
  // share a process (and therefore the registry).
  uint64_t id() const { return mesh_ ? mesh_->comm_id() + 2ull * (uint64_t)rank_ : 0; }
  // Same on every rank of the communicator.
  uint64_t group_key() const { return mesh_ ? mesh_->comm_id() : 0; }
  bool emulated() const { return emu_ != nullptr; }
  bool nvls() const { return stage_.mc_va != 0; }
  VmmBackend* backend() const { return be_; }
  const Segment& ctrl_segment() const { return ctrl_; }
  const Segment& stage_segment() const { return stage_; }
  Mesh* mesh() { return mesh_; }

  // Collectives.  `count` has NCCL's meaning for each kind.  out_dtype != dtype, scale and
  // algo are the fused / forced extensions (pass dtype, 1.0f/false, kAlgoAuto otherwise).
  Status collective(int kind, const void* send, void* recv, size_t count, int dtype, int out_dtype, int redop,
                    int root, float scale, bool has_scale, int algo, cudaStream_t stream);
  // Point-to-point; queued when a group is open on this thread.
  Status p2p(bool is_send, const void* src, void* dst, size_t bytes, int peer, cudaStream_t stream);
  static Status group_start();
  static Status group_end();
  static Status group_simulate_end(float* est_us);

  // Fills kernel arguments for fused kernels built on top of the communicator.
  void fill_args(CollArgs* a) const;
  Status check_usable(const char* what);
  Status check_async();         // reports device-side errors recorded in the status words
  Status prepare_stream(cudaStream_t stream);
  uint32_t* status_words() { return status_; }
  unsigned long long timeout_ns() const { return timeout_ns_; }
  int max_blocks() const { return max_blocks_; }
  EmuGroup* emu() { return emu_.get(); }

  Status pause(PauseResumeStats* st);
  Status resume(PauseResumeStats* st);
  bool paused() const { return paused_; }
  const PauseResumeStats& last_stats() const { return stats_; }

  // Collective allocation of an additional symmetric segment (user windows, fused-op buffers).
  Status sym_alloc(size_t size, int category, int tag, Segment* out);
  Status sym_free(Segment* seg);

  // Work memory of the fused kernels in this rank's own device memory (not shared with peers):
  // a tracked SCRATCH allocation of this communicator, grown on demand, released by ncclPause
  // and re-made by ncclResume with undefined contents, freed at destroy.
  Status local_scratch(int which, size_t bytes, void** out);

  // Registered windows (ncclCommWindowRegister): collective over the communicator.  `buff` must
  // lie in memory from ncclMemAlloc; the whole allocation is registered and its size must be the
  // same on every rank.  From then on the allocation belongs to this communicator's pause /
  // resume scope: its contents are saved and restored, the peers' mappings of it and its
  // multicast binding are dropped and re-made with everything else.
  Status window_register(void* buff, size_t size, Window** out);
  Status window_deregister(Window* w);
  // The window that holds [p, p+bytes), or nullptr.
  Window* find_window(const void* p, size_t bytes);
  size_t window_count() const { return windows_.size(); }

  // Cached scratch segments of the fused kernels (0: gathered activations, 1: reduce-scatter
  // partial slots, 2: MoE receive buffers, 3: MoE return buffers); grown collectively when a
  // call needs more.
  Status fused_segment(int which, size_t bytes, Segment** out);
  // Address, in this process, of rank r's fused-kernel flag area (inside its control segment).
  void* fused_flags(int r) const { return (void*)(ctrl_.va[r] + ((sizeof(CtrlBlock) + 255) & ~(size_t)255)); }

  // Process-wide operations over every live communicator, in creation order.
  static Status pause_all(PauseResumeStats* st);
  static Status resume_all(PauseResumeStats* st);
  static std::vector<Comm*> all();

 private:
  Comm() {}
  ~Comm();
  Status init(const UniqueId& id, int nranks, int rank, const CommConfig& cfg, VmmBackend* be);
  // Creates a multicast object over `seg` (whose local memory is the registry record at
  // `local_va`), binds every rank's memory and maps it; on failure the segment simply has none.
  Status setup_multicast(Segment* seg, uint64_t local_va);
  Status drop_window(Window* w, bool collective);
  Status clear_ll_area();
  Status flush_p2p(cudaStream_t stream);
  Status after_resume(Status engine_result);   // caller holds mu_
  Status run(const CollArgs& a, const LaunchPlan& plan, cudaStream_t stream);

  VmmBackend* be_ = nullptr;
  Mesh* mesh_ = nullptr;
  int rank_ = 0, nranks_ = 1, dev_ = 0;
  Segment ctrl_, stage_;
  Segment fused_[4];
  std::vector<Window*> windows_;
  uint64_t local_va_[2] = {0, 0};
  size_t local_bytes_[2] = {0, 0};
  uint32_t next_sym_ = 1;
  size_t p2p_slot_bytes_ = 0;
  size_t gran_ = 0;
  uint32_t* status_ = nullptr;   // host-mapped (device backend) or plain host memory (mock)
  bool status_pinned_ = false;
  unsigned long long timeout_ns_ = 0;
  int max_blocks_ = 64;
  size_t canary_bytes_ = 0;
  bool paused_ = false, aborted_ = false;
  int async_error_ = 0;
  cudaStream_t last_stream_ = nullptr;
  bool have_last_stream_ = false;
  void* order_event_ = nullptr;
  std::shared_ptr<EmuGroup> emu_;
  PauseResumeStats stats_{};
  EngineOptions opt_;
  // p2p operations queued by the calling thread while a group is open
  std::vector<CollArgs::P2P> pending_;
  cudaStream_t pending_stream_ = nullptr;
  std::mutex mu_;
};

}  // namespace amem
