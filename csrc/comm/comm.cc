#include "comm.h"

#include <cuda_runtime.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>

#include "../core/log.h"
#include "../kernels/gemm_sm100.h"
#include "../kernels/launch.h"
#include "emu.h"
#include "../vmm/tracked.h"

namespace amem {

static std::mutex g_comms_mu;
static std::vector<Comm*> g_comms;

static size_t round_up(size_t x, size_t g) { return (x + g - 1) / g * g; }

struct RankInfo {
  int pid;
  int dev;
  int mc_ok;
  int is_device;
};

std::vector<Comm*> Comm::all() {
  std::lock_guard<std::mutex> g(g_comms_mu);
  return g_comms;
}

Status Comm::create(const UniqueId& id, int nranks, int rank, const CommConfig& cfg, VmmBackend* be, Comm** out) {
  if (!be) return fail(kInvalidUsage, "no usable memory backend (no CUDA device and AMEM_BACKEND != mock)");
  if (nranks > kMaxRanks) return fail(kInvalidArgument, "communicators span one NVLink domain: at most %d ranks, got %d", kMaxRanks, nranks);
  Comm* c = new Comm();
  Status st = c->init(id, nranks, rank, cfg, be);
  if (st != kSuccess) {
    std::string keep = last_error_slot();
    delete c;
    last_error_slot() = keep;
    return st;
  }
  {
    std::lock_guard<std::mutex> g(g_comms_mu);
    g_comms.push_back(c);
  }
  *out = c;
  return kSuccess;
}

Status Comm::init(const UniqueId& id, int nranks, int rank, const CommConfig& cfg, VmmBackend* be) {
  be_ = be;
  rank_ = rank;
  nranks_ = nranks;
  dev_ = 0;
  if (be_->is_device()) {
    if (cudaGetDevice(&dev_) != cudaSuccess) return fail(kCudaError, "cudaGetDevice failed");
    cudaFree(0);  // make sure the primary context exists before driver VMM calls
  }
  AMEM_TRY(Mesh::connect(id, rank, nranks, &mesh_));
  Registry::instance().set_owner_state(this->id(), kRunInit);

  // Who is where: decides emulation (all ranks share one process and one device).
  RankInfo mine{(int)getpid(), dev_, be_->mc_supported(dev_) ? 1 : 0, be_->is_device() ? 1 : 0};
  std::vector<RankInfo> infos(nranks);
  AMEM_TRY(mesh_->allgather(&mine, sizeof(mine), infos.data()));
  bool same_proc_dev = nranks > 1, all_mc = true;
  for (int r = 0; r < nranks; ++r) {
    if (infos[r].is_device != mine.is_device) return fail(kInvalidUsage, "ranks use different memory backends");
    if (infos[r].pid != mine.pid || infos[r].dev != mine.dev) same_proc_dev = false;
    all_mc = all_mc && infos[r].mc_ok;
  }
  if (be_->is_device() && nranks > 1 && !same_proc_dev) {
    for (int r = 0; r < nranks; ++r)
      for (int q = r + 1; q < nranks; ++q)
        if (infos[r].dev == infos[q].dev)
          return fail(kInvalidUsage, "ranks %d and %d share GPU %d: ranks that wait on each other need a GPU each "
                      "(or all ranks in one process on one GPU, which is emulated as a single grid)", r, q, infos[r].dev);
  }
  bool emulate = be_->is_device() && same_proc_dev;
  if (emulate) emu_ = EmuGroup::get(group_key(), nranks);

  // Sizes.
  AMEM_TRY(be_->granularity(dev_, &gran_));
  bool device = be_->is_device();
  size_t stage = cfg.stage_bytes ? cfg.stage_bytes : (size_t)env_long("AMEM_STAGE_MB", device ? 288 : 12) << 20;
  p2p_slot_bytes_ = cfg.p2p_slot_bytes ? cfg.p2p_slot_bytes : (size_t)env_long("AMEM_P2P_SLOT_KB", device ? 64 : 8) << 10;
  if (stage < p2p_area_bytes(p2p_slot_bytes_) + (1u << 20))
    return fail(kInvalidArgument, "staging of %zu bytes is too small for the point-to-point area", stage);
  max_blocks_ = cfg.max_blocks ? cfg.max_blocks : (int)env_long("AMEM_MAX_BLOCKS", emulate ? 8 : 128);
  if (!device) max_blocks_ = 1;
  if (max_blocks_ > kMaxBlocks) max_blocks_ = kMaxBlocks;
  timeout_ns_ = (unsigned long long)env_long("AMEM_DEVICE_TIMEOUT_MS", 20000) * 1000000ull;
  opt_.barrier = env_long("AMEM_PAUSE_BARRIER", 1) != 0;
  opt_.offload_free_tag = (int)env_long("AMEM_NCCL_OFFLOAD_FREE_TAG", -1);

  // Status words the kernels can reach without a copy.
  if (device) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, kStatusWords * sizeof(uint32_t), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess)
      return fail(kCudaError, "cudaHostAlloc(status) failed");
    status_ = (uint32_t*)p;
    status_pinned_ = true;
  } else {
    status_ = (uint32_t*)calloc(kStatusWords, sizeof(uint32_t));
  }
  memset(status_, 0, kStatusWords * sizeof(uint32_t));

  // Control segment (stateful) and staging segment (scratch).
  // The control segment is 2 MiB.  By default it stays resident through a pause: that halves
  // the handles every rank has to export, import and map again on resume, for 2 MiB that are
  // not returned.  AMEM_PAUSE_CONTROL=1 releases it too (saved to and restored from host memory).
  int ctrl_cat = env_long("AMEM_PAUSE_CONTROL", 0) ? kStateful : kResident;
  AMEM_TRY(sym_alloc(round_up(sizeof(CtrlBlock) + (1u << 16), gran_), ctrl_cat, kTagP2P, &ctrl_));
  AMEM_TRY(be_->memset_zero(ctrl_.va[rank_], ctrl_.size, dev_));
  AMEM_TRY(be_->copies_sync(dev_));
  canary_bytes_ = env_long("AMEM_CANARY", 0) ? gran_ : 0;
  AMEM_TRY(sym_alloc(round_up(stage, gran_) + canary_bytes_, kScratch, kTagP2P, &stage_));
  if (canary_bytes_) {
    AMEM_TRY(be_->memset_zero(stage_.va[rank_] + stage_.size - canary_bytes_, canary_bytes_, dev_));
    AMEM_TRY(be_->copies_sync(dev_));
  }
  AMEM_TRY(clear_ll_area());
  int want_nvls = cfg.nvls >= 0 ? cfg.nvls : (int)env_long("AMEM_NVLS", 1);
  if (device && !emulate && nranks > 1 && all_mc && want_nvls) {
    Status st = setup_multicast(&stage_, stage_.va[rank_]);
    if (st != kSuccess) LOGW("rank %d: NVLS disabled: %s", rank_, last_error_slot().c_str());
  }
  AMEM_TRY(mesh_->barrier());  // everybody's control block is zeroed and mapped
  LOGD("comm %#llx rank %d/%d dev %d backend %s emu %d nvls %d stage %zu MiB", (unsigned long long)this->id(), rank_,
       nranks_, dev_, be_->name(), emulate ? 1 : 0, nvls() ? 1 : 0, stage_.size >> 20);
  return kSuccess;
}

// Every rank creates `size` bytes, then maps everybody's memory side by side in one reserved
// window: window + r * size is rank r's memory as seen from this process.
Status Comm::sym_alloc(size_t size, int category, int tag, Segment* out) {
  Segment s;
  s.sym_id = next_sym_++;
  s.size = round_up(size, gran_);
  s.category = category;
  s.tag = tag;
  Registry& reg = Registry::instance();
  if (reg.is_paused(id())) return fail(kInvalidUsage, "symmetric allocation while the communicator is paused");
  AMEM_TRY(be_->reserve(s.size * nranks_, gran_, &s.window));
  for (int r = 0; r < nranks_; ++r) s.va[r] = s.window + (uint64_t)r * s.size;
  uint64_t h = 0;
  AMEM_TRY(be_->create(dev_, s.size, &h));
  Status st = be_->map(s.va[rank_], s.size, h, dev_);
  if (st != kSuccess) {
    be_->release(h);
    return st;
  }
  Allocation rec;
  rec.va = s.va[rank_];
  rec.size = s.size;
  rec.handle = h;
  rec.dev = dev_;
  rec.type = kLocalPosix;
  rec.category = category;
  rec.tag = tag;
  rec.owner = id();
  rec.sym_id = s.sym_id;
  rec.exporter_rank = -1;
  rec.importers = nranks_ > 1 ? (((1u << nranks_) - 1u) & ~(1u << rank_)) : 0;
  AMEM_TRY(reg.add(rec));
  if (nranks_ > 1) {
    int fd = -1;
    AMEM_TRY(be_->export_fd(h, &fd));
    st = kSuccess;
    for (int r = 0; r < nranks_ && st == kSuccess; ++r)
      if (r != rank_) st = mesh_->send_fd(r, s.sym_id, s.size, fd);
    close(fd);
    AMEM_TRY(st);
    for (int r = 0; r < nranks_; ++r) {
      if (r == rank_) continue;
      uint32_t sym = 0;
      uint64_t sz = 0;
      int pfd = -1;
      AMEM_TRY(mesh_->recv_fd(r, &sym, &sz, &pfd));
      if (sym != s.sym_id || sz != s.size) {
        close(pfd);
        return fail(kInternalError, "symmetric allocation out of step with rank %d (segment %u/%u, %llu/%zu bytes)", r, sym, s.sym_id,
                    (unsigned long long)sz, s.size);
      }
      uint64_t ph = 0;
      st = be_->import_fd(pfd, s.size, &ph);
      close(pfd);
      AMEM_TRY(st);
      st = be_->map(s.va[r], s.size, ph, dev_);
      be_->release(ph);   // the mapping keeps the peer's memory alive; one driver call less on every pause
      if (st != kSuccess) return st;
      Allocation imp;
      imp.va = s.va[r];
      imp.size = s.size;
      imp.handle = 0;
      imp.dev = dev_;
      imp.type = kPeerPosix;
      imp.category = category;
      imp.tag = kTagP2PPeer;
      imp.owner = id();
      imp.sym_id = s.sym_id;
      imp.exporter_rank = r;
      AMEM_TRY(reg.add(imp));
    }
  }
  *out = s;
  return kSuccess;
}

Status Comm::fused_segment(int which, size_t bytes, Segment** out) {
  if (which < 0 || which >= 4) return fail(kInvalidArgument, "fused segment index %d", which);
  Segment& s = fused_[which];
  if (s.window && s.size >= bytes) {
    *out = &s;
    return kSuccess;
  }
  // Grow: every rank takes this path in the same call (sizes derive from the call's shape).
  if (s.window) {
    if (be_->is_device()) AMEM_TRY(be_->device_sync(dev_));
    if (nranks_ > 1) AMEM_TRY(mesh_->barrier());  // peers are done with the old mapping
    AMEM_TRY(sym_free(&s));
  }
  AMEM_TRY(sym_alloc(bytes, kScratch, kTagSymm, &s));
  if (nranks_ > 1) AMEM_TRY(mesh_->barrier());
  // The gathered-A buffer of the all-gather -> GEMM kernel also gets a multicast mapping where the
  // communicator has one for its staging: a row then crosses this GPU's links once (one
  // multimem.st, replicated by the switch) instead of once per peer.  Every rank decides the same
  // way (setup_multicast agrees collectively); without it the kernel stores to each peer.
  if (which == 0 && nranks_ > 2 && stage_.mc_va && gemm_ag_uses_mover_warps(nranks_) && env_long("AMEM_AG_MC", 1)) {
    if (setup_multicast(&s, s.va[rank_]) != kSuccess) LOGI("all-gather buffer: no multicast mapping, using per-peer stores");
  }
  *out = &s;
  return kSuccess;
}

// The flag-in-data slots must never hold a word that looks like a packet of a coming operation:
// fresh physical memory (at creation and after every resume) is cleared, flags start at 1.
Status Comm::clear_ll_area() {
  const size_t layout = stage_.size - canary_bytes_;
  const size_t ll = ll_area_bytes(p2p_slot_bytes_);
  AMEM_TRY(be_->memset_zero(stage_.va[rank_] + layout - ll, ll, dev_));
  AMEM_TRY(be_->copies_sync(dev_));
  // and again whenever resume maps new memory here (the engine does it before its closing
  // agreement, so no peer can be writing packets yet); the guard granule behind it likewise
  Allocation rec;
  if (Registry::instance().find(stage_.va[rank_], &rec)) {
    rec.clear_offset = layout - ll;
    rec.clear_bytes = ll + canary_bytes_;
    AMEM_TRY(Registry::instance().update(rec));
  }
  return kSuccess;
}

Status Comm::local_scratch(int which, size_t bytes, void** out) {
  if (which < 0 || which >= 2) return fail(kInvalidArgument, "local scratch index %d", which);
  std::lock_guard<std::mutex> g(mu_);
  if (local_va_[which] && local_bytes_[which] >= bytes) {
    *out = (void*)local_va_[which];
    return kSuccess;
  }
  if (local_va_[which]) {
    AMEM_TRY(tracked_free(be_, local_va_[which]));
    local_va_[which] = 0;
    local_bytes_[which] = 0;
  }
  AMEM_TRY(tracked_alloc(be_, id(), dev_, bytes, kScratch, kTagDefault, &local_va_[which], &local_bytes_[which]));
  *out = (void*)local_va_[which];
  return kSuccess;
}

Status Comm::sym_free(Segment* seg) {
  Registry& reg = Registry::instance();
  for (int r = 0; r < nranks_; ++r) {
    Allocation a;
    if (!reg.find(seg->va[r], &a)) continue;
    if (a.state != kMemHole) {
      if (a.mc_handle && r == rank_) be_->mc_unbind(a.mc_handle, dev_, a.mc_offset, a.size);
      be_->unmap(a.va, a.size);
      if (a.handle) be_->release(a.handle);
    }
    if (a.shadow) be_->host_free(a.shadow, a.size);
    reg.remove(a.va);
  }
  if (seg->mc_va) {
    be_->unmap(seg->mc_va, seg->size);
    be_->free_va(seg->mc_va, seg->size);
    be_->release(seg->mc_handle);
  }
  if (seg->window) be_->free_va(seg->window, seg->size * nranks_);
  *seg = Segment();
  return kSuccess;
}

// One multicast object per communicator: rank 0 creates it and passes the handle around, every
// rank adds its device, binds its staging memory and maps the multicast address range.  The
// object and its mapping survive pause; only the binding is undone and redone
// (the reference does the same for NCCL's NVLS buffers, amem_nccl.cpp:536-538,614-616).
Status Comm::setup_multicast(Segment* seg, uint64_t local_va) {
  uint64_t mc = 0;
  Status st = kSuccess;
  size_t mc_gran = 0;
  const size_t size = seg->size;
  st = be_->mc_granularity(nranks_, size, &mc_gran);
  bool ok = st == kSuccess && mc_gran && size % mc_gran == 0;
  if (ok && rank_ == 0) {
    st = be_->mc_create(nranks_, size, &mc);
    ok = st == kSuccess;
  }
  bool all = false;
  AMEM_TRY(mesh_->all_ok(ok, &all));
  if (!all) {
    if (mc) be_->release(mc);
    return fail(kInvalidUsage, "multicast object could not be created (granularity %zu, segment %zu)", mc_gran, size);
  }
  if (rank_ == 0) {
    int fd = -1;
    AMEM_TRY(be_->export_fd(mc, &fd));
    for (int r = 1; r < nranks_ && st == kSuccess; ++r) st = mesh_->send_fd(r, 0xffffffffu, size, fd);
    close(fd);
    AMEM_TRY(st);
  } else {
    uint32_t sym = 0;
    uint64_t sz = 0;
    int fd = -1;
    AMEM_TRY(mesh_->recv_fd(0, &sym, &sz, &fd));
    st = be_->import_fd(fd, 0, &mc);
    close(fd);
    AMEM_TRY(st);
  }
  ok = be_->mc_add_device(mc, dev_) == kSuccess;
  AMEM_TRY(mesh_->all_ok(ok, &all));  // every device must be added before the first bind
  Allocation rec;
  uint64_t va = 0;
  if (all) {
    ok = Registry::instance().find(local_va, &rec) && be_->mc_bind(mc, 0, rec.handle, size) == kSuccess;
    if (ok) {
      ok = be_->reserve(size, mc_gran, &va) == kSuccess;
      if (ok && be_->map(va, size, mc, dev_) != kSuccess) {
        be_->free_va(va, size);
        va = 0;
        ok = false;
      }
      if (!ok) be_->mc_unbind(mc, dev_, 0, size);
    }
    bool bound = ok;
    AMEM_TRY(mesh_->all_ok(ok, &all));
    if (!all && bound) {
      be_->unmap(va, size);
      be_->free_va(va, size);
      be_->mc_unbind(mc, dev_, 0, size);
    }
  }
  if (!all) {
    be_->release(mc);
    return fail(kInvalidUsage, "multicast bind/map failed on some rank");
  }
  rec.mc_handle = mc;
  rec.mc_offset = 0;
  rec.type = kLocalSymm;
  rec.tag = rec.owner == id() && local_va == stage_.va[rank_] ? kTagNvls : rec.tag;
  AMEM_TRY(Registry::instance().update(rec));
  seg->mc_handle = mc;
  seg->mc_va = va;
  return kSuccess;
}

// ---- registered windows ---------------------------------------------------------------
// The reference learns of such memory through three NCCL hooks: symmetric windows
// (nccl_patch/nccl_2.27.5-1.diff:56-58), user buffers registered with peers (:630-632, which calls
// amem_addPeerInfo, amem_nccl_plugin/amem_nccl.cpp:359-381) and the proxy's imports of them
// (:640-644).  Here registration itself builds the peer mappings, so the records exist from the
// start: the local allocation moves into this communicator's scope with its importers known, and
// every peer's memory is an imported record of that scope.
Status Comm::window_register(void* buff, size_t size, Window** out) {
  AMEM_TRY(check_usable("ncclCommWindowRegister"));
  Registry& reg = Registry::instance();
  Allocation rec;
  bool found = buff && reg.find_containing((uint64_t)buff, &rec) && !from_peer(rec.type) && rec.owner == 0 &&
               (uint64_t)buff + size <= rec.va + rec.size;
  struct Info {
    uint64_t size;
    int ok;
  } mine{found ? rec.size : 0, found ? 1 : 0};
  std::vector<Info> infos(nranks_);
  AMEM_TRY(mesh_->allgather(&mine, sizeof(mine), infos.data()));
  for (int r = 0; r < nranks_; ++r) {
    if (!infos[r].ok)
      return fail(kInvalidArgument, "ncclCommWindowRegister: rank %d did not pass memory from ncclMemAlloc (or it is registered already)", r);
    if (infos[r].size != mine.size)
      return fail(kInvalidArgument, "ncclCommWindowRegister: allocations differ in size across ranks (%llu bytes here, %llu on rank %d)",
                  (unsigned long long)mine.size, (unsigned long long)infos[r].size, r);
  }
  Window* w = new Window();
  w->base = rec.va;
  w->size = rec.size;
  Segment& s = w->seg;
  s.sym_id = next_sym_++;
  s.size = rec.size;
  s.category = kStateful;
  s.tag = kTagSymm;
  Status st = kSuccess;
  if (nranks_ > 1) st = be_->reserve(s.size * nranks_, gran_, &s.window);
  if (st != kSuccess) {
    delete w;
    return st;
  }
  for (int r = 0; r < nranks_; ++r) s.va[r] = r == rank_ ? rec.va : s.window + (uint64_t)r * s.size;
  // my allocation joins this communicator's scope
  rec.owner = id();
  rec.sym_id = s.sym_id;
  rec.tag = kTagSymm;
  rec.importers = nranks_ > 1 ? (((1u << nranks_) - 1u) & ~(1u << rank_)) : 0;
  AMEM_TRY(reg.update(rec));
  if (nranks_ > 1) {
    int fd = -1;
    AMEM_TRY(be_->export_fd(rec.handle, &fd));
    for (int r = 0; r < nranks_ && st == kSuccess; ++r)
      if (r != rank_) st = mesh_->send_fd(r, s.sym_id, s.size, fd);
    close(fd);
    AMEM_TRY(st);
    for (int r = 0; r < nranks_; ++r) {
      if (r == rank_) continue;
      uint32_t sym = 0;
      uint64_t sz = 0;
      int pfd = -1;
      AMEM_TRY(mesh_->recv_fd(r, &sym, &sz, &pfd));
      if (sym != s.sym_id || sz != s.size) {
        close(pfd);
        return fail(kInternalError, "window registration out of step with rank %d (segment %u/%u)", r, sym, s.sym_id);
      }
      uint64_t ph = 0;
      st = be_->import_fd(pfd, s.size, &ph);
      close(pfd);
      AMEM_TRY(st);
      st = be_->map(s.va[r], s.size, ph, dev_);
      be_->release(ph);   // the mapping keeps the peer's memory alive
      if (st != kSuccess) return st;
      Allocation imp;
      imp.va = s.va[r];
      imp.size = s.size;
      imp.handle = 0;
      imp.dev = dev_;
      imp.type = kPeerSymm;
      imp.category = kStateful;
      imp.tag = kTagSymmPeer;
      imp.owner = id();
      imp.sym_id = s.sym_id;
      imp.exporter_rank = r;
      AMEM_TRY(reg.add(imp));
    }
    if (nvls()) {   // the communicator can do multicast: give the window an object of its own
      Status ms = setup_multicast(&s, rec.va);
      if (ms != kSuccess) LOGW("rank %d: window without multicast: %s", rank_, last_error_slot().c_str());
    }
    AMEM_TRY(mesh_->barrier());
  }
  windows_.push_back(w);
  *out = w;
  return kSuccess;
}

Status Comm::drop_window(Window* w, bool collective) {
  Registry& reg = Registry::instance();
  if (collective && nranks_ > 1 && !aborted_) {
    if (be_->is_device() && !paused_) be_->device_sync(dev_);
    mesh_->barrier();   // peers are done with my memory before anybody unmaps
  }
  Segment& s = w->seg;
  for (int r = 0; r < nranks_; ++r) {
    if (r == rank_) continue;
    Allocation a;
    if (!reg.find(s.va[r], &a)) continue;
    if (a.state != kMemHole) {
      be_->unmap(a.va, a.size);
      if (a.handle) be_->release(a.handle);
    }
    reg.remove(a.va);
  }
  Allocation mine;
  if (reg.find(w->base, &mine)) {   // back to a plain ncclMemAlloc allocation of the process
    if (mine.mc_handle && mine.state != kMemHole) be_->mc_unbind(mine.mc_handle, dev_, mine.mc_offset, mine.size);
    mine.mc_handle = 0;
    mine.mc_offset = 0;
    mine.type = kLocalPosix;
    mine.tag = kTagPosix;
    mine.importers = 0;
    mine.sym_id = 0;
    // a paused communicator hands a paused allocation to the process scope, which must then be
    // told that it has something to bring back
    bool hole = mine.state == kMemHole;
    mine.owner = 0;
    reg.update(mine);
    if (hole && reg.owner_state(0) != kRunPaused) reg.set_owner_state(0, kRunPaused);
  }
  if (s.mc_va) {
    be_->unmap(s.mc_va, s.size);
    be_->free_va(s.mc_va, s.size);
    be_->release(s.mc_handle);
  }
  if (s.window) be_->free_va(s.window, s.size * nranks_);
  windows_.erase(std::remove(windows_.begin(), windows_.end(), w), windows_.end());
  delete w;
  return kSuccess;
}

Status Comm::window_deregister(Window* w) {
  if (std::find(windows_.begin(), windows_.end(), w) == windows_.end()) return fail(kInvalidArgument, "not a window of this communicator");
  return drop_window(w, true);
}

Window* Comm::find_window(const void* p, size_t bytes) {
  uint64_t a = (uint64_t)p;
  for (Window* w : windows_)
    if (a >= w->base && a + bytes <= w->base + w->size) return w;
  return nullptr;
}

Comm::~Comm() {
  if (status_) {
    if (status_pinned_) cudaFreeHost(status_);
    else free(status_);
  }
  if (order_event_) cudaEventDestroy((cudaEvent_t)order_event_);
  delete mesh_;
}

Status Comm::check_canary() {
  if (!canary_bytes_ || paused_) return kSuccess;
  if (be_->is_device()) AMEM_TRY(be_->device_sync(dev_));
  std::vector<uint64_t> host(canary_bytes_ / 8);
  void* pinned = nullptr;
  AMEM_TRY(be_->host_alloc(canary_bytes_, &pinned));
  Status st = be_->copy_to_host_async(pinned, stage_.va[rank_] + stage_.size - canary_bytes_, canary_bytes_, dev_);
  if (st == kSuccess) st = be_->copies_sync(dev_);
  if (st == kSuccess) memcpy(host.data(), pinned, canary_bytes_);
  be_->host_free(pinned, canary_bytes_);
  AMEM_TRY(st);
  for (size_t i = 0; i < host.size(); ++i)
    if (host[i]) {
      return fail(kInternalError, "rank %d: staging guard is dirty at offset %zu past the layout (value %#llx): a kernel wrote out of bounds",
                  rank_, i * 8, (unsigned long long)host[i]);
    }
  return kSuccess;
}

Status Comm::debug_dirty_canary() {
  if (!canary_bytes_ || paused_) return fail(kInvalidUsage, "no staging guard to write to (AMEM_CANARY=1, communicator not paused)");
  static const uint64_t word = 0xdeadbeefcafef00dull;
  AMEM_TRY(be_->copy_to_device_async(stage_.va[rank_] + stage_.size - canary_bytes_ + 4096, &word, sizeof(word), dev_));
  return be_->copies_sync(dev_);
}

Status Comm::destroy() {
  {
    std::lock_guard<std::mutex> g(g_comms_mu);
    g_comms.erase(std::remove(g_comms.begin(), g_comms.end(), this), g_comms.end());
  }
  if (be_->is_device()) be_->device_sync(dev_);
  Status guard = aborted_ ? kSuccess : check_canary();
  if (guard != kSuccess) LOGE("%s", last_error_slot().c_str());
  // Peers must be done with my memory before I unmap it.
  if (!aborted_ && mesh_ && nranks_ > 1) mesh_->barrier();
  while (!windows_.empty()) drop_window(windows_.back(), false);
  for (int i = 0; i < 2; ++i)
    if (local_va_[i]) {
      tracked_free(be_, local_va_[i]);
      local_va_[i] = 0;
    }
  for (auto& s : fused_)
    if (s.window) sym_free(&s);
  sym_free(&stage_);
  sym_free(&ctrl_);
  uint64_t cid = id(), gkey = group_key();
  Registry::instance().forget_owner(cid);
  emu_.reset();
  EmuGroup::drop(gkey);
  delete this;
  return guard;
}

void Comm::abort() {
  aborted_ = true;
  if (mesh_) mesh_->shutdown_all();
}

}  // namespace amem
