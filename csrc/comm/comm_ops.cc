// Communicator operations: collectives, grouped point-to-point, split, pause / resume.
#include <cuda_runtime.h>
#include <unistd.h>

#include <algorithm>
#include <cstring>
#include <functional>
#include <thread>

#include "../core/log.h"
#include "../kernels/launch.h"
#include "comm.h"
#include "emu.h"

namespace amem {

static thread_local int t_group_depth = 0;
static thread_local std::vector<Comm*> t_group_comms;

void Comm::fill_args(CollArgs* a) const {
  memset(a, 0, sizeof(*a));
  a->rank = rank_;
  a->nranks = nranks_;
  for (int r = 0; r < nranks_; ++r) {
    a->ctrl[r] = (CtrlBlock*)ctrl_.va[r];
    a->stage[r] = (char*)stage_.va[r];
  }
  a->mc_stage = (char*)stage_.mc_va;
  a->stage_bytes = stage_.size - canary_bytes_;  // the guard granule is not part of the layout
  a->p2p_slot_bytes = p2p_slot_bytes_;
  a->status = status_;
  a->timeout_ns = timeout_ns_;
  a->p2p_max_lanes = emu_ ? 2 : kP2PBlocks;
  static const long nvls_split = env_long("AMEM_NVLS_SPLIT", 4);
  a->nvls_split = (int)nvls_split;
  a->scale = 1.0f;
}

Status Comm::check_async() {
  if (async_error_) return fail((Status)async_error_, "communicator is in an error state");
  uint32_t code = __atomic_load_n(&status_[0], __ATOMIC_ACQUIRE);
  if (code != 0) {
    async_error_ = kInternalError;
    aborted_ = true;
    return fail(kInternalError, "device-side wait ran out (code %u): rank %u waited for rank %u in block %u at epoch %u", code,
                status_[1], status_[2], status_[3], status_[4]);
  }
  return kSuccess;
}

Status Comm::check_usable(const char* what) {
  // The reference only logs a backtrace here and lets NCCL run into unmapped memory
  // (amem_nccl.cpp:452-464); refusing the call keeps the process alive.
  if (paused_ || Registry::instance().is_paused(id())) {
    LOGE("%s called while the communicator's memory is paused", what);
    if (log_level_ref().load() >= kDebug) log_backtrace();
    return fail(kInvalidUsage, "%s called while the communicator's memory is paused; call ncclResume first", what);
  }
  if (aborted_) return fail(kInternalError, "%s on an aborted communicator", what);
  return check_async();
}

// Operations of one communicator are ordered: if the caller switches streams, the new stream
// waits for everything the communicator enqueued on the previous one (staging reuse relies on
// stream order).
Status Comm::prepare_stream(cudaStream_t stream) {
  if (!be_->is_device()) return kSuccess;
  int cur = -1;
  cudaGetDevice(&cur);
  if (cur != dev_) return fail(kInvalidUsage, "current CUDA device is %d but the communicator lives on device %d", cur, dev_);
  if (have_last_stream_ && last_stream_ != stream) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(stream, &cs);
    if (cs == cudaStreamCaptureStatusNone) {
      if (!order_event_) {
        cudaEvent_t e;
        if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return fail(kCudaError, "cudaEventCreate failed");
        order_event_ = e;
      }
      if (cudaEventRecord((cudaEvent_t)order_event_, last_stream_) != cudaSuccess ||
          cudaStreamWaitEvent(stream, (cudaEvent_t)order_event_, 0) != cudaSuccess) {
        cudaGetLastError();
        return fail(kCudaError, "could not order the new stream after the communicator's previous stream");
      }
    }
  }
  last_stream_ = stream;
  have_last_stream_ = true;
  return kSuccess;
}

Status Comm::run(const CollArgs& a, const LaunchPlan& plan, cudaStream_t stream) {
  if (!be_->is_device()) {
    int rc = host_run_collective(a, plan);
    if (rc == kDevBadArgs) return fail(kInvalidArgument, "unsupported datatype %d -> %d with operator %d", a.dtype, a.out_dtype, a.redop);
    if (rc != kDevOk) return check_async();
    return kSuccess;
  }
  AMEM_TRY(prepare_stream(stream));
  if (emu_) {
    LaunchPlan p = plan;
    int n = nranks_;
    int tag = a.kind * 256 + a.algo * 16 + a.dtype;
    return emu_->rendezvous(rank_, tag, &a, sizeof(a), stream, [p, n](const void* host_all, const void* dev_all, cudaStream_t s) {
      const CollArgs* h = (const CollArgs*)host_all;
      LaunchPlan q = p;
      if (h[0].kind == kCollSendRecv) {
        q.blocks = 1;
        for (int r = 0; r < n; ++r) q.blocks = std::max(q.blocks, sendrecv_blocks(h[r]));
      }
      return launch_collective_emu((const CollArgs*)dev_all, h[0], n, q, s);
    });
  }
  return launch_collective(a, plan, stream);
}

Status Comm::collective(int kind, const void* send, void* recv, size_t count, int dtype, int out_dtype, int redop, int root,
                        float scale, bool has_scale, int algo, cudaStream_t stream) {
  static const char* names[] = {"ncclAllReduce", "ncclAllGather", "ncclReduceScatter", "ncclBroadcast", "ncclReduce", "ncclAllToAll"};
  AMEM_TRY(check_usable(names[kind]));
  size_t es = dtype_size(dtype);
  if (es == 0 || dtype_size(out_dtype) == 0) return fail(kInvalidArgument, "unknown datatype %d", dtype);
  if (!send || !recv) return fail(kInvalidArgument, "null buffer");
  if ((kind == kCollBroadcast || kind == kCollReduce) && (root < 0 || root >= nranks_)) return fail(kInvalidArgument, "root %d out of range", root);
  if (redop < kSum || redop > kAvg) return fail(kInvalidArgument, "unknown reduction operator %d", redop);
  if (count == 0) return kSuccess;
  CollArgs a;
  fill_args(&a);
  a.kind = kind;
  a.send = send;
  a.recv = recv;
  a.count = count;
  a.dtype = dtype;
  a.out_dtype = out_dtype;
  a.redop = redop;
  a.root = root;
  a.scale = scale;
  a.has_scale = has_scale ? 1 : 0;
  bool reducing = kind == kCollAllReduce || kind == kCollReduceScatter || kind == kCollReduce;
  if (reducing && redop == kAvg) {
    a.scale = (has_scale ? scale : 1.0f) / (float)nranks_;
    a.has_scale = 1;
  }
  if (!reducing) {  // pure data movement runs on bytes
    a.count = count * es;
    a.dtype = a.out_dtype = kU8;
    a.redop = kSum;
  }
  TunerInput ti;
  ti.kind = kind;
  ti.count = a.count;
  ti.dtype = a.dtype;
  ti.redop = redop;
  ti.nranks = nranks_;
  ti.stage_bytes = stage_.size - canary_bytes_;
  ti.p2p_slot_bytes = p2p_slot_bytes_;
  ti.nvls = nvls();
  ti.max_blocks = max_blocks_;
  ti.forced_algo = algo;
  // Both operands inside registered windows, at the same offsets on every rank (the caller's
  // contract, as for NCCL's symmetric windows): the all-reduce can work on them in place.
  Window* ws = nullptr;
  Window* wr = nullptr;
  if (kind == kCollAllReduce && nranks_ > 1 && dtype == out_dtype && !windows_.empty()) {
    ws = find_window(send, count * es);
    wr = find_window(recv, count * es);
    if (ws && wr) {
      ti.window = true;
      size_t so = (uint64_t)send - ws->base, ro = (uint64_t)recv - wr->base;
      // between two GPUs the switch has nothing to add (plain peer loads and stores measured faster there)
      ti.window_mc = nranks_ > 2 && ws->seg.mc_va && wr->seg.mc_va && (count * es) % 16 == 0 && so % 16 == 0 && ro % 16 == 0;
    }
  }
  // Reduce-scatter FROM a window and all-gather INTO a window go through the window's multicast
  // mapping (sum of fp32 / fp16 / bf16 without a cast for the former); three ranks or more.
  if (nranks_ > 2 && !windows_.empty() && (algo == kAlgoAuto || algo == kAlgoWindow)) {
    if (kind == kCollReduceScatter && dtype == out_dtype && (redop == kSum || redop == kAvg) && (dtype == kF32 || dtype == kBF16 || dtype == kF16)) {
      Window* w = find_window(send, count * es * nranks_);
      size_t so = w ? (uint64_t)send - w->base : 0;
      if (w && w->seg.mc_va && (count * es) % 16 == 0 && so % 16 == 0 && ((uint64_t)recv & 15) == 0 && count * es >= (256u << 10)) {
        a.algo = kAlgoWindow;
        a.mc_send = (const char*)w->seg.mc_va + so;
        LaunchPlan wp;
        wp.algo = kAlgoWindow;
        wp.threads = 512;
        wp.chunk_elems = count;
        wp.blocks = (int)std::max<size_t>(1, std::min<size_t>((size_t)max_blocks_, count * es / (64u << 10)));
        return run(a, wp, stream);
      }
    }
    if (kind == kCollAllGather) {
      Window* w = find_window(recv, count * es * nranks_);
      size_t ro = w ? (uint64_t)recv - w->base : 0;
      if (w && w->seg.mc_va && (count * es) % 16 == 0 && ro % 16 == 0 && ((uint64_t)send & 15) == 0 && count * es >= (256u << 10)) {
        // (in place works too: the multicast store also lands in this rank's own copy)
        a.algo = kAlgoWindow;
        a.mc_recv = (char*)w->seg.mc_va + ro;
        LaunchPlan wp;
        wp.algo = kAlgoWindow;
        wp.threads = 512;
        wp.chunk_elems = a.count;
        wp.blocks = (int)std::max<size_t>(1, std::min<size_t>((size_t)max_blocks_, count * es / (64u << 10)));
        return run(a, wp, stream);
      }
    }
  }
  LaunchPlan plan = plan_collective(ti);
  if (plan.algo == kAlgoWindow) {
    size_t so = (uint64_t)send - ws->base, ro = (uint64_t)recv - wr->base;
    for (int r = 0; r < nranks_; ++r) {
      a.win_send[r] = (const char*)ws->seg.va[r] + so;
      a.win_recv[r] = (char*)wr->seg.va[r] + ro;
    }
    a.mc_send = ti.window_mc ? (const char*)ws->seg.mc_va + so : nullptr;
    a.mc_recv = ti.window_mc ? (char*)wr->seg.mc_va + ro : nullptr;
  }
  if (kind == kCollAllReduce && algo != kAlgoAuto && plan.algo != algo)
    return fail(kInvalidArgument, "all-reduce variant %d is not available for this size/type on this communicator", algo);
  a.algo = plan.algo;
  return run(a, plan, stream);
}

Status Comm::group_start() {
  ++t_group_depth;
  return kSuccess;
}

Status Comm::group_end() {
  if (t_group_depth <= 0) return fail(kInvalidUsage, "ncclGroupEnd without ncclGroupStart");
  if (--t_group_depth > 0) return kSuccess;
  Status first = kSuccess;
  std::vector<Comm*> comms;
  comms.swap(t_group_comms);
  for (Comm* c : comms) {
    Status st = c->flush_p2p(c->pending_stream_);
    if (st != kSuccess && first == kSuccess) first = st;
  }
  return first;
}

// Closes the group without launching anything: the queued point-to-point operations are
// dropped and their total is priced with the measured peer-copy rate (ncclGroupSimulateEnd).
Status Comm::group_simulate_end(float* est_us) {
  if (t_group_depth <= 0) return fail(kInvalidUsage, "ncclGroupSimulateEnd without ncclGroupStart");
  if (--t_group_depth > 0) {
    if (est_us) *est_us = 0.f;
    return kSuccess;
  }
  std::vector<Comm*> comms;
  comms.swap(t_group_comms);
  double us = 0;
  for (Comm* c : comms) {
    size_t out_bytes = 0, in_bytes = 0;
    for (auto& e : c->pending_) (e.is_send ? out_bytes : in_bytes) += e.bytes;
    c->pending_.clear();
    // launch + flag latency, then the busier direction at ~770 GB/s per direction
    us += 8.0 + (double)std::max(out_bytes, in_bytes) / 770e3;
  }
  if (est_us) *est_us = (float)us;
  return kSuccess;
}

Status Comm::p2p(bool is_send, const void* src, void* dst, size_t bytes, int peer, cudaStream_t stream) {
  AMEM_TRY(check_usable(is_send ? "ncclSend" : "ncclRecv"));
  if (peer < 0 || peer >= nranks_) return fail(kInvalidArgument, "peer %d out of range", peer);
  CollArgs::P2P e;
  e.peer = peer;
  e.is_send = is_send ? 1 : 0;
  e.src = src;
  e.dst = dst;
  e.bytes = bytes;
  if (pending_.empty()) pending_stream_ = stream;
  pending_.push_back(e);
  if (t_group_depth > 0) {
    if (std::find(t_group_comms.begin(), t_group_comms.end(), this) == t_group_comms.end()) t_group_comms.push_back(this);
    return kSuccess;
  }
  return flush_p2p(stream);
}

Status Comm::flush_p2p(cudaStream_t stream) {
  std::vector<CollArgs::P2P> ops;
  ops.swap(pending_);
  if (ops.empty()) return kSuccess;
  // Transfers to myself never touch the network: pair each self-send with a self-receive.
  std::vector<CollArgs::P2P> net;
  std::vector<CollArgs::P2P> self_send, self_recv;
  for (auto& e : ops) {
    if (e.peer != rank_) net.push_back(e);
    else (e.is_send ? self_send : self_recv).push_back(e);
  }
  if (self_send.size() != self_recv.size()) return fail(kInvalidUsage, "send to self without a matching receive in the same group");
  for (size_t i = 0; i < self_send.size(); ++i) {
    if (self_send[i].bytes != self_recv[i].bytes) return fail(kInvalidArgument, "self send/recv sizes differ");
    if (!self_send[i].bytes) continue;
    if (be_->is_device()) {
      AMEM_TRY(prepare_stream(stream));
      if (cudaMemcpyAsync(self_recv[i].dst, self_send[i].src, self_send[i].bytes, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
        return fail(kCudaError, "self copy failed");
    } else {
      memmove(self_recv[i].dst, self_send[i].src, self_send[i].bytes);
    }
  }
  // Zero-byte transfers carry no credit traffic on either side.
  net.erase(std::remove_if(net.begin(), net.end(), [](const CollArgs::P2P& e) { return e.bytes == 0; }), net.end());
  if (net.empty() && !emu_) return kSuccess;
  // One launch carries at most one send and one receive per peer (their credit counters are per
  // peer and direction).  A group with more runs in rounds: round k holds every peer's k-th send
  // and k-th receive.  Operations between two ranks match in call order on both sides, so the
  // k-th send to a peer meets that peer's k-th receive in ITS round k: every round is a complete
  // matched set and no round waits for a later one.  Any number of operations per group.
  std::vector<std::vector<CollArgs::P2P>> rounds;
  std::vector<int> n_send(nranks_, 0), n_recv(nranks_, 0);
  for (auto& e : net) {
    int k = e.is_send ? n_send[e.peer]++ : n_recv[e.peer]++;
    if ((int)rounds.size() <= k) rounds.resize(k + 1);
    rounds[k].push_back(e);
  }
  if (rounds.empty()) rounds.resize(1);   // emulated ranks still meet when this rank has nothing to move
  for (auto& ops_k : rounds) {
    CollArgs a;
    fill_args(&a);
    a.kind = kCollSendRecv;
    a.dtype = a.out_dtype = kU8;
    a.n_p2p = (int)ops_k.size();
    for (size_t i = 0; i < ops_k.size(); ++i) a.p2p[i] = ops_k[i];
    LaunchPlan plan;
    plan.algo = 0;
    plan.blocks = 1;
    plan.threads = 512;
    plan.chunk_elems = 0;
    AMEM_TRY(run(a, plan, stream));
  }
  return kSuccess;
}

Status Comm::split(int color, int key, const CommConfig& cfg, Comm** out) {
  AMEM_TRY(check_usable("ncclCommSplit"));
  struct Vote {
    int color, key;
    UniqueId id;
  };
  Vote mine;
  mine.color = color;
  mine.key = key;
  AMEM_TRY(make_unique_id(&mine.id));
  std::vector<Vote> all(nranks_);
  AMEM_TRY(mesh_->allgather(&mine, sizeof(mine), all.data()));
  *out = nullptr;
  if (color < 0) return kSuccess;
  std::vector<int> members;
  for (int r = 0; r < nranks_; ++r)
    if (all[r].color == color) members.push_back(r);
  std::stable_sort(members.begin(), members.end(), [&](int x, int y) { return all[x].key < all[y].key; });
  int new_rank = (int)(std::find(members.begin(), members.end(), rank_) - members.begin());
  // The child meets under the id proposed by its lowest parent rank.
  int leader = *std::min_element(members.begin(), members.end());
  return Comm::create(all[leader].id, (int)members.size(), new_rank, cfg, be_, out);
}

Status Comm::shrink(const int* exclude, int n_exclude, const CommConfig& cfg, Comm** out) {
  *out = nullptr;
  if (n_exclude < 0 || (n_exclude > 0 && !exclude)) return fail(kInvalidArgument, "ncclCommShrink: bad exclusion list");
  std::vector<bool> gone(nranks_, false);
  for (int i = 0; i < n_exclude; ++i) {
    if (exclude[i] < 0 || exclude[i] >= nranks_) return fail(kInvalidArgument, "ncclCommShrink: rank %d is not in this communicator", exclude[i]);
    gone[exclude[i]] = true;
  }
  if (gone[rank_]) return fail(kInvalidArgument, "ncclCommShrink: the calling rank %d is in the exclusion list", rank_);
  std::vector<int> alive;
  for (int r = 0; r < nranks_; ++r)
    if (!gone[r]) alive.push_back(r);
  // The lowest surviving rank proposes the id of the child and tells every other survivor over
  // the pairwise sockets; excluded ranks are never contacted (they may have died).
  UniqueId id;
  const int leader = alive[0];
  if (rank_ == leader) {
    AMEM_TRY(make_unique_id(&id));
    for (size_t i = 1; i < alive.size(); ++i) AMEM_TRY(mesh_->send_blob(alive[i], &id, sizeof(id)));
  } else {
    AMEM_TRY(mesh_->recv_blob(leader, &id, sizeof(id)));
  }
  int new_rank = (int)(std::find(alive.begin(), alive.end(), rank_) - alive.begin());
  return Comm::create(id, (int)alive.size(), new_rank, cfg, be_, out);
}

Status Comm::pause(PauseResumeStats* st) {
  std::lock_guard<std::mutex> g(mu_);
  if (paused_) return kSuccess;
  if (!pending_.empty()) return fail(kInvalidUsage, "ncclPause inside an open group");
  AMEM_TRY(check_canary());
  Status s = pause_scope(Registry::instance(), be_, id(), dev_, mesh_, opt_, &stats_);
  // a failure after the first release still ends PAUSED (and is reported), so that ncclResume
  // can bring the memory back; a failure before it leaves the communicator running
  paused_ = Registry::instance().owner_state(id()) == kRunPaused;
  if (st) *st = stats_;
  return s;
}

Status Comm::after_resume(Status s) {
  paused_ = Registry::instance().owner_state(id()) == kRunPaused;
  return s;   // (the engine re-zeroes the flag-in-data slots and the guard granule of fresh memory)
}

Status Comm::resume(PauseResumeStats* st) {
  std::lock_guard<std::mutex> g(mu_);
  if (!paused_) return kSuccess;
  Status s = resume_scope(Registry::instance(), be_, id(), dev_, mesh_, opt_, &stats_);
  s = after_resume(s);
  if (st) *st = stats_;
  return s;
}

static void accumulate(PauseResumeStats* into, const PauseResumeStats& s, bool pause_part) {
  // bytes and counts add up over the scopes; the phase times are those of the one pass
  if (pause_part) {
    into->quiesce_us = s.quiesce_us;
    into->offload_us = s.offload_us;
    into->release_import_us = s.release_import_us;
    into->release_local_us = s.release_local_us;
    into->pause_barrier_us = s.pause_barrier_us;
    into->free_before_pause = s.free_before_pause;
    into->free_after_pause = s.free_after_pause;
    into->bytes_offloaded += s.bytes_offloaded;
    into->bytes_released_local += s.bytes_released_local;
    into->bytes_released_peer += s.bytes_released_peer;
    into->n_offload += s.n_offload;
    into->n_release_local += s.n_release_local;
    into->n_release_peer += s.n_release_peer;
  } else {
    into->create_map_us = s.create_map_us;
    into->agree_us = s.agree_us;
    into->exchange_us = s.exchange_us;
    into->import_us = s.import_us;
    into->preload_us = s.preload_us;
    into->resume_barrier_us = s.resume_barrier_us;
    into->free_after_resume = s.free_after_resume;
    into->bytes_preloaded += s.bytes_preloaded;
  }
}

static std::mutex g_all_mu;   // one process-wide pause or resume at a time

// Process-wide pause: ONE engine pass over every communicator of the process plus the
// allocations that belong to no communicator (ncclMemAlloc).  Every rank holds its communicators
// in the same creation order, so the per-communicator messages line up; within the pass all
// communicators' messages are sent before any is awaited.  Ranks of one communicator that live in
// this process (emulated ranks, ncclCommInitAll) are served by the same pass.  New allocations
// are refused until resume.
Status Comm::pause_all(PauseResumeStats* st) {
  std::lock_guard<std::mutex> all_lock(g_all_mu);
  Registry& reg = Registry::instance();
  PauseResumeStats total;
  memset(&total, 0, sizeof(total));
  double t0 = now_ms();
  std::vector<Comm*> comms = Comm::all();
  VmmBackend* be = comms.empty() ? default_backend() : comms[0]->backend();
  if (!be) return kSuccess;
  std::vector<Comm*> active;
  for (Comm* c : comms) {
    std::lock_guard<std::mutex> g(c->mu_);
    if (c->paused_) continue;
    if (!c->pending_.empty()) return fail(kInvalidUsage, "ncclPause inside an open group");
    AMEM_TRY(c->check_canary());
    active.push_back(c);
  }
  std::vector<PauseResumeStats> stats(active.size() + 1);
  for (auto& s : stats) memset(&s, 0, sizeof(s));
  std::vector<EngineScope> scopes(active.size() + 1);
  for (size_t i = 0; i < active.size(); ++i) {
    scopes[i].owner = active[i]->id();
    scopes[i].dev = active[i]->dev_;
    scopes[i].px = active[i]->mesh_;
    scopes[i].opt = active[i]->opt_;
    scopes[i].stats = &stats[i];
  }
  EngineScope& proc = scopes.back();   // process-level allocations
  proc.owner = 0;
  proc.dev = 0;
  if (be->is_device()) cudaGetDevice(&proc.dev);
  proc.opt.offload_free_tag = (int)env_long("AMEM_NCCL_OFFLOAD_FREE_TAG", -1);
  proc.stats = &stats.back();
  Status s = pause_scopes(reg, be, scopes);
  std::string why = last_error_slot();
  bool all_paused = reg.owner_state(0) == kRunPaused;
  for (size_t i = 0; i < active.size(); ++i) {
    Comm* c = active[i];
    c->paused_ = reg.owner_state(c->id()) == kRunPaused;
    all_paused = all_paused && c->paused_;
    c->stats_ = stats[i];
  }
  for (auto& x : stats) accumulate(&total, x, true);
  if (all_paused) reg.set_process_paused(true);
  total.pause_total_us = (now_ms() - t0) * 1000.0;
  if (st) *st = total;
  last_error_slot() = why;
  return s;
}

Status Comm::resume_all(PauseResumeStats* st) {
  std::lock_guard<std::mutex> all_lock(g_all_mu);
  Registry& reg = Registry::instance();
  PauseResumeStats total;
  memset(&total, 0, sizeof(total));
  double t0 = now_ms();
  std::vector<Comm*> comms = Comm::all();
  VmmBackend* be = comms.empty() ? default_backend() : comms[0]->backend();
  if (!be) return kSuccess;
  reg.set_process_paused(false);
  std::vector<Comm*> active;
  for (Comm* c : comms)
    if (c->paused_) active.push_back(c);
  std::vector<PauseResumeStats> stats(active.size() + 1);
  for (auto& s : stats) memset(&s, 0, sizeof(s));
  std::vector<EngineScope> scopes(active.size() + 1);
  for (size_t i = 0; i < active.size(); ++i) {
    scopes[i].owner = active[i]->id();
    scopes[i].dev = active[i]->dev_;
    scopes[i].px = active[i]->mesh_;
    scopes[i].opt = active[i]->opt_;
    scopes[i].stats = &stats[i];
  }
  EngineScope& proc = scopes.back();
  proc.owner = 0;
  proc.dev = 0;
  if (be->is_device()) cudaGetDevice(&proc.dev);
  proc.opt.offload_free_tag = (int)env_long("AMEM_NCCL_OFFLOAD_FREE_TAG", -1);
  proc.stats = &stats.back();
  Status s = resume_scopes(reg, be, scopes);
  std::string why = last_error_slot();
  bool any_paused = reg.owner_state(0) == kRunPaused;
  for (size_t i = 0; i < active.size(); ++i) {
    Comm* c = active[i];
    std::lock_guard<std::mutex> g(c->mu_);
    Status a = c->after_resume(scopes[i].result);
    if (a != kSuccess && s == kSuccess) {
      s = a;
      why = last_error_slot();
    }
    any_paused = any_paused || c->paused_;
    PauseResumeStats keep = c->stats_;   // pause half stays, resume half is replaced
    accumulate(&keep, stats[i], false);
    keep.bytes_preloaded = stats[i].bytes_preloaded;
    keep.resume_total_us = stats[i].resume_total_us;
    c->stats_ = keep;
  }
  for (auto& x : stats) accumulate(&total, x, false);
  if (any_paused) reg.set_process_paused(true);   // something did not come back: still refuse collectives; ncclResume may be retried
  total.resume_total_us = (now_ms() - t0) * 1000.0;
  if (st) *st = total;
  last_error_slot() = why;
  return s;
}

}  // namespace amem
