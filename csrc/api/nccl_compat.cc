// C API: NCCL-compatible entry points plus the AMem pause/resume calls, on top of amem::Comm.
//
// Reference for the five added calls: nccl_patch/nccl_2.27.5-1.diff:63-112 (they ignore the
// communicator argument and always return ncclSuccess there).  Here the argument selects the
// scope and failures are reported.
#include <cuda_runtime.h>

#include <cstring>
#include <mutex>
#include <thread>
#include <utility>
#include <vector>

#include "../comm/comm.h"
#include "../vmm/tracked.h"
#include "../core/log.h"
#include "../include/nccl.h"
#include "../kernels/launch.h"
#include "../ipc/uds.h"

using namespace amem;

namespace {

static_assert(sizeof(ncclUniqueId) == sizeof(UniqueId), "unique id size");
static_assert(sizeof(amemMemStats_t) == sizeof(MemStats), "amemMemStats_t must mirror MemStats");
static_assert(sizeof(amemPauseResumeStats_t) == sizeof(PauseResumeStats), "amemPauseResumeStats_t must mirror PauseResumeStats");

inline ncclResult_t R(Status s) {
  if (s != kSuccess && log_level_ref().load() >= kWarn) LOGW("%s: %s", status_name(s), last_error_slot().c_str());
  return (ncclResult_t)s;
}
inline Comm* C(ncclComm_t c) { return reinterpret_cast<Comm*>(c); }

// AMEM_ENABLE=0 turns pause/resume into no-ops (the reference defaults to disabled and needs
// AMEM_ENABLE=1, amem_nccl.cpp:711; this library exists to pause, so it defaults to on).
bool amem_enabled() {
  static int v = (int)env_long("AMEM_ENABLE", 1);
  return v != 0;
}

PauseResumeStats g_process_stats;

CommConfig config_from(const ncclConfig_t* cfg) {
  CommConfig c;
  if (cfg && cfg->maxCTAs != NCCL_CONFIG_UNDEF_INT && cfg->maxCTAs > 0) c.max_blocks = cfg->maxCTAs;
  return c;
}

// Operators made by ncclRedOpCreatePreMulSum: id = ncclNumOps + slot; value = the scalar.
std::mutex g_ops_mu;
std::vector<std::pair<bool, float>> g_premul;  // (in use, scalar)

bool resolve_op(int op, int* redop, float* scale, bool* has_scale) {
  *scale = 1.0f;
  *has_scale = false;
  if (op >= 0 && op < (int)ncclNumOps) {
    *redop = op;
    return true;
  }
  std::lock_guard<std::mutex> g(g_ops_mu);
  int slot = op - (int)ncclNumOps;
  if (slot < 0 || slot >= (int)g_premul.size() || !g_premul[slot].first) return false;
  *redop = kSum;
  *scale = g_premul[slot].second;
  *has_scale = true;
  return true;
}

}  // namespace

extern "C" {

const char* amemLastError(void) { return last_error_slot().c_str(); }
const char* ncclGetLastError(ncclComm_t) { return last_error_slot().c_str(); }
const char* ncclGetErrorString(ncclResult_t r) { return status_name((int)r); }

ncclResult_t ncclGetVersion(int* version) {
  if (!version) return ncclInvalidArgument;
  *version = NCCL_VERSION_CODE;
  return ncclSuccess;
}

ncclResult_t ncclGetUniqueId(ncclUniqueId* out) {
  if (!out) return ncclInvalidArgument;
  return R(make_unique_id(reinterpret_cast<UniqueId*>(out)));
}

ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank, ncclConfig_t* config) {
  if (!comm) return ncclInvalidArgument;
  UniqueId uid;
  memcpy(&uid, &id, sizeof(uid));
  Comm* c = nullptr;
  Status s = Comm::create(uid, nranks, rank, config_from(config), default_backend(), &c);
  *comm = reinterpret_cast<ncclComm_t>(c);
  return R(s);
}

ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
  return ncclCommInitRankConfig(comm, nranks, id, rank, nullptr);
}

// One process drives ndev GPUs: the ranks bootstrap concurrently on helper threads.
ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist) {
  if (!comms || ndev < 1) return ncclInvalidArgument;
  ncclUniqueId id;
  ncclResult_t r = ncclGetUniqueId(&id);
  if (r != ncclSuccess) return r;
  std::vector<ncclResult_t> res(ndev, ncclSuccess);
  std::vector<std::thread> th;
  bool device = default_backend() && default_backend()->is_device();
  for (int i = 0; i < ndev; ++i) {
    th.emplace_back([&, i] {
      if (device) cudaSetDevice(devlist ? devlist[i] : i);
      res[i] = ncclCommInitRank(&comms[i], ndev, id, i);
    });
  }
  for (auto& t : th) t.join();
  for (auto x : res)
    if (x != ncclSuccess) return x;
  return ncclSuccess;
}

ncclResult_t ncclCommFinalize(ncclComm_t comm) {
  if (!comm) return ncclInvalidArgument;
  Comm* c = C(comm);
  if (c->backend()->is_device() && !c->paused()) c->backend()->device_sync(c->device());
  return ncclSuccess;
}

ncclResult_t ncclCommDestroy(ncclComm_t comm) {
  if (!comm) return ncclSuccess;
  return R(C(comm)->destroy());
}

ncclResult_t ncclCommAbort(ncclComm_t comm) {
  if (!comm) return ncclSuccess;
  C(comm)->abort();
  return R(C(comm)->destroy());
}

ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* config) {
  if (!comm || !newcomm) return ncclInvalidArgument;
  Comm* c = nullptr;
  Status s = C(comm)->split(color, key, config_from(config), &c);
  *newcomm = reinterpret_cast<ncclComm_t>(c);
  return R(s);
}

ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError) {
  if (!comm || !asyncError) return ncclInvalidArgument;
  *asyncError = (ncclResult_t)C(comm)->check_async();
  return ncclSuccess;
}
ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) {
  if (!comm || !count) return ncclInvalidArgument;
  *count = C(comm)->nranks();
  return ncclSuccess;
}
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device) {
  if (!comm || !device) return ncclInvalidArgument;
  *device = C(comm)->device();
  return ncclSuccess;
}
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) {
  if (!comm || !rank) return ncclInvalidArgument;
  *rank = C(comm)->rank();
  return ncclSuccess;
}
// Local registration (not collective, as in NCCL): the buffer is checked and remembered; peers
// reach user buffers through this library's own staging, so nothing is mapped anywhere.  Memory
// that peers should reach in place is registered with ncclCommWindowRegister.
ncclResult_t ncclCommRegister(const ncclComm_t comm, void* buff, size_t size, void** handle) {
  if (!comm || !buff || !handle) return ncclInvalidArgument;
  (void)size;
  *handle = buff;
  return ncclSuccess;
}
ncclResult_t ncclCommDeregister(const ncclComm_t comm, void* handle) {
  if (!comm || !handle) return ncclInvalidArgument;
  return ncclSuccess;
}

// Collective.  `buff` must come from ncclMemAlloc; the whole allocation becomes a window that
// every rank maps (and that is bound to a multicast object when the communicator has NVLS).
// All-reduce calls whose two buffers lie in windows then run in place on them.  The window is
// tracked: ncclPause saves and releases it with the communicator, ncclResume brings it back at
// the same addresses on every rank.
ncclResult_t ncclCommWindowRegister(ncclComm_t comm, void* buff, size_t size, ncclWindow_t* win, int) {
  if (!comm || !win) return ncclInvalidArgument;
  Window* w = nullptr;
  Status s = C(comm)->window_register(buff, size, &w);
  *win = reinterpret_cast<ncclWindow_t>(w);
  return R(s);
}
ncclResult_t ncclCommWindowDeregister(ncclComm_t comm, ncclWindow_t win) {
  if (!comm || !win) return ncclInvalidArgument;
  if (C(comm)->paused()) return R(fail(kInvalidUsage, "ncclCommWindowDeregister while the communicator is paused"));
  return R(C(comm)->window_deregister(reinterpret_cast<Window*>(win)));
}

ncclResult_t ncclCommInitRankScalable(ncclComm_t* newcomm, int nranks, int myrank, int nId, ncclUniqueId* commIds, ncclConfig_t* config) {
  if (!commIds || nId < 1) return ncclInvalidArgument;
  return ncclCommInitRankConfig(newcomm, nranks, commIds[0], myrank, config);
}

// The surviving ranks of `comm` (all but excludeRanksList) form a new communicator; the parent is
// left as it is (shrinkFlags is accepted for source compatibility: there is no in-flight
// network state to abort, a parent with a lost rank is simply destroyed or aborted afterwards).
ncclResult_t ncclCommShrink(ncclComm_t comm, int* excludeRanksList, int excludeRanksCount, ncclComm_t* newcomm, ncclConfig_t* config, int) {
  if (!comm || !newcomm) return ncclInvalidArgument;
  Comm* c = nullptr;
  Status s = C(comm)->shrink(excludeRanksList, excludeRanksCount, config_from(config), &c);
  *newcomm = reinterpret_cast<ncclComm_t>(c);
  return R(s);
}

ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype, ncclScalarResidence_t residence, ncclComm_t) {
  if (!op || !scalar) return ncclInvalidArgument;
  unsigned char raw[8] = {0};
  size_t es = dtype_size(datatype);
  if (es == 0) return ncclInvalidArgument;
  if (residence == ncclScalarDevice) {
    if (cudaMemcpy(raw, scalar, es, cudaMemcpyDeviceToHost) != cudaSuccess) return ncclUnhandledCudaError;
  } else {
    memcpy(raw, scalar, es);
  }
  float v;
  switch ((int)datatype) {
    case kF32: memcpy(&v, raw, 4); break;
    case kF64: { double d; memcpy(&d, raw, 8); v = (float)d; break; }
    case kF16: { uint16_t h; memcpy(&h, raw, 2); uint32_t sign = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023; float f;
                 if (e == 0) f = (float)m / 1024.0f / 16384.0f; else if (e == 31) f = 65504.0f; else { uint32_t bits = ((e + 112) << 23) | (m << 13); memcpy(&f, &bits, 4); }
                 v = sign ? -f : f; break; }
    case kBF16: { uint16_t h; memcpy(&h, raw, 2); uint32_t bits = (uint32_t)h << 16; memcpy(&v, &bits, 4); break; }
    case kI32: { int i; memcpy(&i, raw, 4); v = (float)i; break; }
    case kI64: { long long i; memcpy(&i, raw, 8); v = (float)i; break; }
    default: return R(fail(kInvalidArgument, "pre-multiplied sum is not supported for datatype %d", (int)datatype));
  }
  std::lock_guard<std::mutex> g(g_ops_mu);
  size_t slot = 0;
  while (slot < g_premul.size() && g_premul[slot].first) ++slot;
  if (slot == g_premul.size()) g_premul.emplace_back(false, 1.0f);
  g_premul[slot] = {true, v};
  *op = (ncclRedOp_t)((int)ncclNumOps + (int)slot);
  return ncclSuccess;
}

ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t) {
  std::lock_guard<std::mutex> g(g_ops_mu);
  int slot = (int)op - (int)ncclNumOps;
  if (slot < 0 || slot >= (int)g_premul.size()) return ncclInvalidArgument;
  g_premul[slot].first = false;
  return ncclSuccess;
}

// ---- memory ---------------------------------------------------------------------------
ncclResult_t ncclMemAlloc(void** ptr, size_t size) {
  if (!ptr || size == 0) return ncclInvalidArgument;
  VmmBackend* be = default_backend();
  if (!be) return R(fail(kInvalidUsage, "no usable memory backend"));
  int dev = 0;
  if (be->is_device()) {
    if (cudaGetDevice(&dev) != cudaSuccess) return ncclUnhandledCudaError;
    cudaFree(0);
  }
  if (Registry::instance().is_paused(0)) return R(fail(kInvalidUsage, "ncclMemAlloc while paused"));
  uint64_t va = 0;
  Status s = tracked_alloc(be, 0, dev, size, kStateful, kTagPosix, &va, nullptr);
  if (s != kSuccess) return R(s);
  *ptr = (void*)va;
  return ncclSuccess;
}

ncclResult_t ncclMemFree(void* ptr) {
  if (!ptr) return ncclSuccess;
  Allocation a;
  if (!Registry::instance().find((uint64_t)ptr, &a) || from_peer(a.type))
    return R(fail(kInvalidArgument, "ncclMemFree: pointer was not returned by ncclMemAlloc"));
  if (a.owner != 0) return R(fail(kInvalidUsage, "ncclMemFree: the buffer is still registered as a window (ncclCommWindowDeregister first)"));
  return R(tracked_free(default_backend(), a.va));
}

// ---- collectives ----------------------------------------------------------------------
#define NEED_COMM(c) if (!(c)) return R(fail(kInvalidArgument, "null communicator"))

ncclResult_t ncclAllReduce(const void* s, void* r, size_t count, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  int redop;
  float scale;
  bool has;
  if (!resolve_op(op, &redop, &scale, &has)) return R(fail(kInvalidArgument, "unknown reduction operator %d", (int)op));
  return R(C(comm)->collective(kCollAllReduce, s, r, count, dt, dt, redop, 0, scale, has, kAlgoAuto, st));
}
ncclResult_t amemAllReduceAlgo(const void* s, void* r, size_t count, ncclDataType_t dt, ncclRedOp_t op, int algo, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  return R(C(comm)->collective(kCollAllReduce, s, r, count, dt, dt, op, 0, 1.0f, false, algo, st));
}
ncclResult_t ncclReduce(const void* s, void* r, size_t count, ncclDataType_t dt, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  int redop;
  float scale;
  bool has;
  if (!resolve_op(op, &redop, &scale, &has)) return R(fail(kInvalidArgument, "unknown reduction operator %d", (int)op));
  return R(C(comm)->collective(kCollReduce, s, r, count, dt, dt, redop, root, scale, has, kAlgoAuto, st));
}
ncclResult_t ncclBroadcast(const void* s, void* r, size_t count, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  return R(C(comm)->collective(kCollBroadcast, s, r, count, dt, dt, kSum, root, 1.0f, false, kAlgoAuto, st));
}
ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t dt, int root, ncclComm_t comm, cudaStream_t st) {
  return ncclBroadcast(buff, buff, count, dt, root, comm, st);
}
ncclResult_t ncclReduceScatter(const void* s, void* r, size_t recvcount, ncclDataType_t dt, ncclRedOp_t op, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  int redop;
  float scale;
  bool has;
  if (!resolve_op(op, &redop, &scale, &has)) return R(fail(kInvalidArgument, "unknown reduction operator %d", (int)op));
  return R(C(comm)->collective(kCollReduceScatter, s, r, recvcount, dt, dt, redop, 0, scale, has, kAlgoAuto, st));
}
ncclResult_t amemReduceScatterScaleCast(const void* s, void* r, size_t recvcount, ncclDataType_t in_t, ncclDataType_t out_t, float scale,
                                        ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  return R(C(comm)->collective(kCollReduceScatter, s, r, recvcount, in_t, out_t, kSum, 0, scale, true, kAlgoAuto, st));
}
ncclResult_t ncclAllGather(const void* s, void* r, size_t sendcount, ncclDataType_t dt, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  return R(C(comm)->collective(kCollAllGather, s, r, sendcount, dt, dt, kSum, 0, 1.0f, false, kAlgoAuto, st));
}
ncclResult_t ncclAlltoAll(const void* s, void* r, size_t count, ncclDataType_t dt, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  return R(C(comm)->collective(kCollAllToAll, s, r, count, dt, dt, kSum, 0, 1.0f, false, kAlgoAuto, st));
}
ncclResult_t ncclSend(const void* s, size_t count, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  return R(C(comm)->p2p(true, s, nullptr, count * dtype_size(dt), peer, st));
}
ncclResult_t ncclRecv(void* r, size_t count, ncclDataType_t dt, int peer, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  return R(C(comm)->p2p(false, nullptr, r, count * dtype_size(dt), peer, st));
}
// Variable-size all-to-all (MPI_Alltoallv argument convention, counts and displacements in
// elements): one grouped launch of a send and a receive per peer, the form NCCL applications
// write by hand (nccl-tests' alltoall is the same grouped send/recv); the block a rank keeps for
// itself is paired inside the group and never touches the network.
ncclResult_t amemAlltoAllv(const void* sendbuff, const size_t* sendcounts, const size_t* sdispls, void* recvbuff,
                           const size_t* recvcounts, const size_t* rdispls, ncclDataType_t dt, ncclComm_t comm, cudaStream_t st) {
  NEED_COMM(comm);
  if (!sendcounts || !sdispls || !recvcounts || !rdispls) return ncclInvalidArgument;
  const size_t es = dtype_size(dt);
  if (es == 0) return ncclInvalidArgument;
  Comm* c = C(comm);
  const int n = c->nranks(), me = c->rank();
  if (sendcounts[me] != recvcounts[me]) return R(fail(kInvalidArgument, "amemAlltoAllv: rank %d keeps %zu elements but expects %zu", me, sendcounts[me], recvcounts[me]));
  Status s = Comm::group_start();
  if (s != kSuccess) return R(s);
  for (int k = 0; k < n && s == kSuccess; ++k) {
    const int to = (me + k) % n, from = (me - k + n) % n;
    if (sendcounts[to]) s = c->p2p(true, (const char*)sendbuff + sdispls[to] * es, nullptr, sendcounts[to] * es, to, st);
    if (s == kSuccess && recvcounts[from]) s = c->p2p(false, nullptr, (char*)recvbuff + rdispls[from] * es, recvcounts[from] * es, from, st);
  }
  Status e = Comm::group_end();
  return R(s != kSuccess ? s : e);
}
ncclResult_t ncclGroupStart(void) {
  // A paused process may not batch work either (the reference guards group calls too,
  // nccl_2.27.5-1.diff:205-229).
  if (Registry::instance().process_paused()) return R(fail(kInvalidUsage, "ncclGroupStart while paused"));
  return R(Comm::group_start());
}
ncclResult_t ncclGroupEnd(void) { return R(Comm::group_end()); }
ncclResult_t ncclGroupSimulateEnd(ncclSimInfo_t* simInfo) {
  if (simInfo && (simInfo->size != sizeof(ncclSimInfo_t) || simInfo->magic != 0x74685283u))
    return R(fail(kInvalidArgument, "ncclGroupSimulateEnd: simInfo was not set up with NCCL_SIM_INFO_INITIALIZER"));
  float us = 0.f;
  Status st = Comm::group_simulate_end(&us);
  if (st == kSuccess && simInfo) simInfo->estimatedTime = us;
  return R(st);
}
void ncclResetDebugInit(void) { log_level_ref().store((int)env_long("GMM_LOG", kInfo)); }

// ---- AMem -----------------------------------------------------------------------------
ncclResult_t ncclPause(ncclComm_t* comm) {
  if (!amem_enabled()) return ncclSuccess;
  if (comm && *comm) return R(C(*comm)->pause(nullptr));
  return R(Comm::pause_all(&g_process_stats));
}
ncclResult_t ncclResume(ncclComm_t* comm) {
  if (!amem_enabled()) return ncclSuccess;
  if (comm && *comm) return R(C(*comm)->resume(nullptr));
  PauseResumeStats s;
  Status st = Comm::resume_all(&s);
  // keep the pause half recorded by the preceding ncclPause
  g_process_stats.create_map_us = s.create_map_us;
  g_process_stats.agree_us = s.agree_us;
  g_process_stats.exchange_us = s.exchange_us;
  g_process_stats.import_us = s.import_us;
  g_process_stats.preload_us = s.preload_us;
  g_process_stats.resume_barrier_us = s.resume_barrier_us;
  g_process_stats.resume_total_us = s.resume_total_us;
  g_process_stats.bytes_preloaded = s.bytes_preloaded;
  g_process_stats.free_after_resume = s.free_after_resume;
  return R(st);
}
ncclResult_t ncclMemStats(void) {
  Registry::instance().dump_stats(log_level_ref().load() >= kDebug);
  return ncclSuccess;
}
ncclResult_t ncclSetGroupID(int id) { return R(Registry::instance().set_group_id(id)); }
ncclResult_t ncclGetGroupID(int* id) {
  if (!id) return ncclInvalidArgument;
  *id = Registry::instance().group_id();
  return ncclSuccess;
}

ncclResult_t amemMemStatsGet(amemMemStats_t* out) {
  if (!out) return ncclInvalidArgument;
  Registry::instance().stats(reinterpret_cast<MemStats*>(out));
  return ncclSuccess;
}
ncclResult_t amemPauseResumeStatsGet(ncclComm_t comm, amemPauseResumeStats_t* out) {
  if (!out) return ncclInvalidArgument;
  const PauseResumeStats& s = comm ? C(comm)->last_stats() : g_process_stats;
  memcpy(out, &s, sizeof(s));
  return ncclSuccess;
}
ncclResult_t amemCommInfo(ncclComm_t comm, int* emulated, int* nvls, size_t* stage_bytes) {
  NEED_COMM(comm);
  if (emulated) *emulated = C(comm)->emulated() ? 1 : 0;
  if (nvls) *nvls = C(comm)->nvls() ? 1 : 0;
  if (stage_bytes) *stage_bytes = C(comm)->stage_segment().size;
  return ncclSuccess;
}
// The variant, grid and chunk the library would use for one collective on a communicator of
// `nranks` GPUs with the default staging (host arithmetic only; no communicator needed).
// kind: 0 all-reduce, 1 all-gather, 2 reduce-scatter, 3 broadcast, 4 reduce, 5 all-to-all;
// count has the meaning of the matching NCCL call.  algo out: 1 one-shot, 2 two-shot, 3 NVLS, 0 n/a.
ncclResult_t amemTunerPlan(int kind, size_t count, ncclDataType_t dtype, int nranks, int nvls, size_t stage_bytes, int* algo,
                           int* blocks, size_t* chunk_elems) {
  if (kind < 0 || kind > kCollAllToAll || nranks < 1 || nranks > kMaxRanks || dtype_size(dtype) == 0) return ncclInvalidArgument;
  TunerInput ti;
  ti.kind = kind;
  ti.count = count;
  ti.dtype = dtype;
  ti.redop = kSum;
  ti.nranks = nranks;
  ti.stage_bytes = stage_bytes ? stage_bytes : ((size_t)288 << 20);
  ti.p2p_slot_bytes = (size_t)64 << 10;
  ti.nvls = nvls != 0;
  ti.max_blocks = 128;
  ti.forced_algo = kAlgoAuto;
  LaunchPlan p = plan_collective(ti);
  if (algo) *algo = p.algo;
  if (blocks) *blocks = p.blocks;
  if (chunk_elems) *chunk_elems = p.chunk_elems;
  return ncclSuccess;
}
// Checks the staging guard of `comm` now (AMEM_CANARY=1; ncclSuccess when the guard is off).
ncclResult_t amemCheckCanary(ncclComm_t comm) {
  NEED_COMM(comm);
  return R(C(comm)->check_canary());
}
// Test hook: simulates an out-of-bounds write behind the staging layout.
ncclResult_t amemDebugDirtyCanary(ncclComm_t comm) {
  NEED_COMM(comm);
  return R(C(comm)->debug_dirty_canary());
}
ncclResult_t amemInject(const char* what, int nth, int param) {
  if (!what) return ncclInvalidArgument;
  if (!strncmp(what, "uds:", 4)) {
    uds_inject(what + 4, nth, param);
    return ncclSuccess;
  }
  if (!strncmp(what, "vmm:", 4)) {
    VmmBackend* be = default_backend();
    if (!be) return ncclInvalidUsage;
    be->inject_failure(what + 4, nth);
    return ncclSuccess;
  }
  return ncclInvalidArgument;
}
ncclResult_t amemBackendTimings(char* buf, size_t len, int reset) {
  VmmBackend* be = default_backend();
  if (!be || !buf || !len) return ncclInvalidArgument;
  std::string s = be->timings(reset != 0);
  snprintf(buf, len, "%s", s.c_str());
  return ncclSuccess;
}
ncclResult_t amemDeviceWaitProbe(int timeout_ms, int flag_is_set, int* code, float* waited_ms) {
  if (timeout_ms <= 0 || timeout_ms > 10000) return R(fail(kInvalidArgument, "amemDeviceWaitProbe: timeout %d ms (1 .. 10000)", timeout_ms));
  uint32_t* flag = nullptr;
  uint32_t* status = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  Status st = kSuccess;
  float ms = 0.f;
  if (cudaMalloc((void**)&flag, sizeof(uint32_t)) != cudaSuccess || cudaHostAlloc((void**)&status, kStatusWords * sizeof(uint32_t), cudaHostAllocMapped) != cudaSuccess ||
      cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) {
    cudaGetLastError();
    st = fail(kCudaError, "amemDeviceWaitProbe: could not allocate its two words and events");
  }
  if (st == kSuccess) {
    memset(status, 0, kStatusWords * sizeof(uint32_t));
    const uint32_t init = flag_is_set ? 1u : 0u;
    if (cudaMemcpy(flag, &init, sizeof(init), cudaMemcpyHostToDevice) != cudaSuccess) st = fail(kCudaError, "amemDeviceWaitProbe: cudaMemcpy failed");
  }
  if (st == kSuccess) {
    cudaEventRecord(e0, 0);
    st = launch_wait_probe(flag, 1u, (unsigned long long)timeout_ms * 1000000ull, status, 0);
    cudaEventRecord(e1, 0);
    cudaError_t e = cudaEventSynchronize(e1);
    if (st == kSuccess && e != cudaSuccess) st = fail(kCudaError, "amemDeviceWaitProbe: %s", cudaGetErrorString(e));
    if (st == kSuccess) cudaEventElapsedTime(&ms, e0, e1);
  }
  if (st == kSuccess) {
    if (code) *code = (int)status[0];
    if (waited_ms) *waited_ms = ms;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  if (status) cudaFreeHost(status);
  if (flag) cudaFree(flag);
  return R(st);
}

int amemBackendIsDevice(void) {
  VmmBackend* be = default_backend();
  return be && be->is_device() ? 1 : 0;
}
ncclResult_t amemBackendUsage(size_t* physical_bytes, size_t* mappings, const char** backend_name) {
  VmmBackend* be = default_backend();
  if (!be) return ncclInvalidUsage;
  if (physical_bytes) *physical_bytes = be->live_physical_bytes();
  if (mappings) *mappings = be->live_mappings();
  if (backend_name) *backend_name = be->name();
  return ncclSuccess;
}

}  // extern "C"
