// C entry points of the fused compute + collective operations (tensor-parallel GEMMs).
// The reference has no counterpart: its tensor-parallel users call cuBLAS and NCCL back to
// back; here the collective rides inside the GEMM kernel (kernels/gemm_sm100.cu).
#include <cuda_runtime.h>

#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "../comm/comm.h"
#include "../comm/emu.h"
#include "../core/log.h"
#include "../include/nccl.h"
#include "../kernels/gemm_ag_cta_movers.h"
#include "../kernels/gemm_sm100.h"
#include "../kernels/moe.h"
#include "../vmm/tracked.h"

using namespace amem;

namespace {

inline ncclResult_t R(Status s) {
  if (s != kSuccess) LOGW("%s: %s", status_name(s), last_error_slot().c_str());
  return (ncclResult_t)s;
}

Status check_shape(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(kInvalidArgument, "empty GEMM %d x %d x %d", M, N, K);
  if (N % 8 || K % 8) return fail(kInvalidArgument, "N and K must be multiples of 8 (16-byte rows), got N=%d K=%d", N, K);
  return kSuccess;
}

void fill_fused(Comm* c, GemmParams* p) {
  c->fill_args(&p->coll);
  for (int r = 0; r < c->nranks(); ++r) p->fflags[r] = (FusedFlags*)c->fused_flags(r);
}

Status run_gemm(Comm* c, GemmLaunch& g, cudaStream_t stream) {
  if (c && c->emulated()) {
    int n = c->nranks();
    return c->emu()->rendezvous(c->rank(), 1000 + g.p.mode, &g, sizeof(g), stream,
                                [n](const void* host_all, const void*, cudaStream_t s) { return launch_gemm_emu((const GemmLaunch*)host_all, n, s); });
  }
  return launch_gemm(g, stream);
}

int emu_grid(int nranks) {
  int sms = gemm_default_grid(0);
  int per = sms / nranks;  // one CTA per SM and every CTA of every rank must be resident
  return per < 3 ? 3 : (per > 16 ? 16 : per);
}

}  // namespace

namespace {
struct SplitKWs {
  float* partials = nullptr;
  uint32_t* counters = nullptr;
};
// One workspace per (device, stream); null when none exists and none can be made right now.
SplitKWs* splitk_workspace(int dev, cudaStream_t stream, int ctas) {
  static std::mutex mu;
  static std::map<std::pair<int, cudaStream_t>, SplitKWs> all;
  std::lock_guard<std::mutex> lk(mu);
  auto key = std::make_pair(dev, stream);
  auto it = all.find(key);
  if (it != all.end()) return it->second.partials ? &it->second : nullptr;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return nullptr;  // not recorded: a later launch outside the capture may allocate
  }
  // Tracked, process-level memory: the partial tiles are SCRATCH (dead between launches), the
  // counters are STATEFUL (they must read zero at every launch, also after a pause).
  SplitKWs w;
  size_t ctr_bytes = gemm_splitk_ctr_words(ctas) * sizeof(uint32_t);
  VmmBackend* be = cuda_backend();
  uint64_t pv = 0, cv = 0;
  if (!be || tracked_alloc(be, 0, dev, gemm_splitk_ws_bytes(ctas), kScratch, kTagDefault, &pv, nullptr) != kSuccess ||
      tracked_alloc(be, 0, dev, ctr_bytes, kStateful, kTagDefault, &cv, nullptr) != kSuccess ||
      cudaMemset((void*)cv, 0, ctr_bytes) != cudaSuccess) {
    cudaGetLastError();
    if (pv) tracked_free(be, pv);
    if (cv) tracked_free(be, cv);
    pv = cv = 0;  // remembered as "no workspace": the GEMM runs unsplit on this stream
  }
  w.partials = (float*)pv;
  w.counters = (uint32_t*)cv;
  auto ins = all.emplace(key, w);
  return ins.first->second.partials ? &ins.first->second : nullptr;
}

// Tiling of the plain GEMM for one problem: tile width, tile height, split of the last wave.
struct GemmPlan {
  int bn, tall, slices;
};
GemmPlan plan_gemm(int M, int N, int K, int sms, bool can_split) {
  const int k_blocks = (K + kGemmBK - 1) / kGemmBK;
  // Tile height: 256-row tiles feed two accumulators from one B tile (less shared-memory fill
  // per FLOP, the limit of the 128-row main loop) but their epilogue is not hidden behind the
  // next tile, so they pay only with a long K.  AMEM_GEMM_TALL = 0 / 1 forces, -1 decides.
  const long tall_env = env_long("AMEM_GEMM_TALL", -1);
  int slices = 1, slices_tall = 1;
  const int bn_flat = gemm_pick_bn((M + kGemmBM - 1) / kGemmBM, N, sms, can_split ? k_blocks : 0, &slices);
  const int bn_tall = gemm_pick_bn((M + 2 * kGemmBM - 1) / (2 * kGemmBM), N, sms, can_split ? k_blocks : 0, &slices_tall);
  bool tall = tall_env >= 0 ? tall_env != 0 : gemm_tall_pays(M, N, k_blocks, sms, bn_flat, slices, bn_tall, slices_tall);
  if (M <= kGemmBM) tall = false;
  GemmPlan p;
  p.tall = tall ? 1 : 0;
  p.bn = tall ? bn_tall : bn_flat;
  p.slices = tall ? slices_tall : slices;
  return p;
}
}  // namespace

namespace {
// A communicator-free launch still needs protocol words (epoch, operation counter) and status
// words the host can read: one small block of each per device, made on first use.  The device
// block is a tracked RESIDENT allocation: the plain and grouped GEMMs stay usable while
// everything else of the process is paused.
Status gemm_process_words(int dev, CtrlBlock** ctrl_out, uint32_t** status_out) {
  static std::mutex init_mu;
  static CtrlBlock* ctrl[64] = {nullptr};
  static uint32_t* status_dev[64] = {nullptr};
  if (dev < 0 || dev >= 64) return fail(kInvalidArgument, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(init_mu);
  if (!ctrl[dev]) {
    uint64_t va = 0;
    VmmBackend* be = cuda_backend();
    cudaFree(0);
    if (!be) return fail(kInvalidUsage, "no CUDA memory backend");
    AMEM_TRY(tracked_alloc(be, 0, dev, sizeof(CtrlBlock) + sizeof(FusedFlags), kResident, kTagDefault, &va, nullptr));
    cudaMemset((void*)va, 0, sizeof(CtrlBlock) + sizeof(FusedFlags));
    ctrl[dev] = (CtrlBlock*)va;
  }
  if (!status_dev[dev]) {
    uint32_t* st = nullptr;
    if (cudaHostAlloc((void**)&st, kStatusWords * 4, cudaHostAllocMapped) != cudaSuccess) return fail(kCudaError, "cudaHostAlloc of the status words failed");
    memset(st, 0, kStatusWords * 4);
    status_dev[dev] = st;
  }
  *ctrl_out = ctrl[dev];
  *status_out = status_dev[dev];
  return kSuccess;
}
}  // namespace

extern "C" {

// The tiling amemGemmBf16 would use on a GPU with `sms` SMs (no GPU needed: planning is host
// arithmetic).  Outputs may be null.
ncclResult_t amemGemmPlan(int M, int N, int K, int sms, int* tile_rows, int* tile_cols, int* tail_slices) {
  Status s = check_shape(M, N, K);
  if (s != kSuccess) return R(s);
  if (sms <= 0) return R(fail(kInvalidArgument, "amemGemmPlan: sms must be positive"));
  GemmPlan p = plan_gemm(M, N, K, sms, env_long("AMEM_GEMM_SPLITK", 1) != 0);
  if (tile_rows) *tile_rows = p.tall ? 2 * kGemmBM : kGemmBM;
  if (tile_cols) *tile_cols = p.bn;
  if (tail_slices) *tail_slices = p.slices;
  return ncclSuccess;
}

// What amemAllGatherGemm does on a communicator of `nranks` ranks whose shards have `rows_per_rank`
// rows of K bf16 (host arithmetic, no GPU needed).  *mover_warps: 1 = mover warps inside every CTA,
// 0 = dedicated mover CTAs; *rows_per_flag: rows of a shard that one ready flag announces;
// *flags_per_rank: ready flags one source rank uses.  Outputs may be null.
ncclResult_t amemAllGatherGemmPlan(int nranks, int rows_per_rank, int K, int* mover_warps, int* rows_per_flag, int* flags_per_rank) {
  if (nranks < 1 || nranks > kMaxRanks || rows_per_rank <= 0 || K <= 0 || K % 8)
    return R(fail(kInvalidArgument, "amemAllGatherGemmPlan: nranks=%d rows_per_rank=%d K=%d", nranks, rows_per_rank, K));
  const bool warps = nranks == 1 || gemm_ag_uses_mover_warps(nranks);
  const int per_flag = warps ? gemm_ag_unit_rows(rows_per_rank, K) : agcta::kAgUnitRows;
  const int flags = (rows_per_rank + per_flag - 1) / per_flag;
  if (flags > (warps ? kMaxAgUnits : agcta::kMaxUnits))
    return R(fail(kInvalidArgument, "amemAllGatherGemmPlan: %d rows per rank need %d ready flags", rows_per_rank, flags));
  if (mover_warps) *mover_warps = warps ? 1 : 0;
  if (rows_per_flag) *rows_per_flag = per_flag;
  if (flags_per_rank) *flags_per_rank = flags;
  return ncclSuccess;
}

ncclResult_t amemGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t stream) {
  Status s = check_shape(M, N, K);
  if (s != kSuccess) return R(s);
  int dev = 0;
  cudaGetDevice(&dev);
  CtrlBlock* ctrl_dev = nullptr;
  uint32_t* status_words = nullptr;
  if ((s = gemm_process_words(dev, &ctrl_dev, &status_words)) != kSuccess) return R(s);
  GemmLaunch g;
  memset(&g, 0, sizeof(g));
  g.p.M = M;
  g.p.N = N;
  g.p.K = K;
  g.p.mode = kGemmPlain;
  g.p.C = C;
  g.p.ldc = N;
  g.p.rows_per_rank = M;
  g.p.coll.rank = 0;
  g.p.coll.nranks = 1;
  g.p.coll.ctrl[0] = ctrl_dev;
  g.p.coll.status = status_words;
  g.p.coll.timeout_ns = 5ull * 1000000000ull;
  g.p.fflags[0] = (FusedFlags*)(ctrl_dev + 1);
  int sms = gemm_default_grid(dev);
  // Split-K of the last wave needs a workspace (fp32 partial tiles + counters), kept per
  // (device, stream) so that launches on different streams never share one.  It is allocated on
  // the first launch of a stream; a stream that is being captured gets no split unless it
  // already has one (allocation is not allowed there).  AMEM_GEMM_SPLITK=0 turns the split off.
  const long splitk_on = env_long("AMEM_GEMM_SPLITK", 1);  // read per call: benches flip it
  // (while the process is paused the workspace is not mapped: the GEMM then runs unsplit)
  SplitKWs* ws = splitk_on && !Registry::instance().is_paused(0) ? splitk_workspace(dev, stream, sms) : nullptr;
  GemmPlan plan = plan_gemm(M, N, K, sms, ws != nullptr);
  const bool tall = plan.tall != 0;
  int slices = plan.slices;
  g.p.tall = plan.tall;
  g.p.bn = plan.bn;
  const int tile_rows = tall ? 2 * kGemmBM : kGemmBM;
  if ((s = make_tensor_map_bf16(&g.map_a, A, M, K, K, tile_rows)) != kSuccess) return R(s);
  g.map_a_local = g.map_a;
  if ((s = make_tensor_map_bf16(&g.map_b, B, N, K, K, g.p.bn)) != kSuccess) return R(s);
  int tiles = ((M + tile_rows - 1) / tile_rows) * ((N + g.p.bn - 1) / g.p.bn);
  g.grid = (tiles < sms && slices <= 1) ? tiles : sms;
  if (ws && slices > 1) {
    g.p.sk_slices = slices;
    g.p.sk_ws = ws->partials;
    g.p.sk_ctr = ws->counters;
  }
  s = launch_gemm(g, stream);
  if (s == kSuccess && status_words[0]) {
    // an earlier launch gave up on a wait: its split-K counters may be left mid-count
    if (ws) cudaMemsetAsync(ws->counters, 0, gemm_splitk_ctr_words(sms) * sizeof(uint32_t), stream);
    s = fail(kInternalError, "tcgen05 GEMM reported a device-side wait timeout (code %u)", status_words[0]);
  }
  return R(s);
}

// Grouped GEMM: C[rows of group e, :] = A[rows of group e, :] * B[e]^T for every group, one launch.
// A: bf16 [rows_cap, K]; group_off: DEVICE int32 [groups + 1] (row offsets, e.g. expert_offsets of
// amemMoeDispatch — the host never reads them); B: bf16 [groups, N, K]; C: bf16 [rows_cap, N], or
// [rows_cap, N / 2] with epilogue = 1 (SwiGLU of 32-column gate / up blocks, see GemmEpilogue).
// rows_hint: the number of rows the caller expects (sizes the tile width; any value is correct).
ncclResult_t amemGroupedGemmBf16(const void* A, const void* B, void* C, const int* group_off, int groups, int rows_cap, int rows_hint,
                                 int N, int K, int epilogue, cudaStream_t stream) {
  Status s = check_shape(rows_cap, N, K);
  if (s != kSuccess) return R(s);
  if (!A || !B || !C || !group_off) return R(fail(kInvalidArgument, "grouped GEMM: null buffer"));
  if (groups <= 0 || groups > 256) return R(fail(kInvalidArgument, "grouped GEMM: %d groups (1..256)", groups));
  if (epilogue != kEpiStore && epilogue != kEpiSwiGLU) return R(fail(kInvalidArgument, "grouped GEMM: unknown epilogue %d", epilogue));
  if (epilogue == kEpiSwiGLU && N % 64) return R(fail(kInvalidArgument, "grouped GEMM: the SwiGLU epilogue needs N to be a multiple of 64, got %d", N));
  if ((long long)groups * N > 0x7fffffffLL) return R(fail(kInvalidArgument, "grouped GEMM: groups * N does not fit 31 bits"));
  int dev = 0;
  cudaGetDevice(&dev);
  CtrlBlock* ctrl = nullptr;
  uint32_t* status = nullptr;
  if ((s = gemm_process_words(dev, &ctrl, &status)) != kSuccess) return R(s);
  GemmLaunch g;
  memset(&g, 0, sizeof(g));
  g.p.M = rows_cap;
  g.p.N = N;
  g.p.K = K;
  g.p.mode = kGemmGrouped;
  g.p.C = C;
  g.p.ldc = epilogue == kEpiSwiGLU ? N / 2 : N;
  g.p.rows_per_rank = rows_cap;
  g.p.group_off = group_off;
  g.p.groups = groups;
  g.p.epilogue = epilogue;
  g.p.coll.rank = 0;
  g.p.coll.nranks = 1;
  g.p.coll.ctrl[0] = ctrl;
  g.p.coll.status = status;
  g.p.coll.timeout_ns = 5ull * 1000000000ull;
  g.p.fflags[0] = (FusedFlags*)(ctrl + 1);
  const int sms = gemm_default_grid(dev);
  // every group ends in a partly filled row tile: count about half a tile of waste per group
  const int hint = rows_hint > 0 ? rows_hint : rows_cap;
  const int row_tiles = (hint + kGemmBM - 1) / kGemmBM + groups / 2;
  int bn = gemm_pick_bn(row_tiles, N, sms);
  if (epilogue == kEpiSwiGLU) bn = bn >= 224 ? 256 : (bn >= 160 ? 192 : 128);
  g.p.bn = bn;
  if ((s = make_tensor_map_bf16(&g.map_a, A, rows_cap, K, K, kGemmBM)) != kSuccess) return R(s);
  g.map_a_local = g.map_a;
  if ((s = make_tensor_map_bf16(&g.map_b, B, (uint64_t)groups * N, K, K, g.p.bn)) != kSuccess) return R(s);
  g.grid = sms;
  s = launch_gemm(g, stream);
  if (s == kSuccess && status[0]) s = fail(kInternalError, "tcgen05 GEMM reported a device-side wait timeout (code %u)", status[0]);
  return R(s);
}

}  // extern "C"

namespace {
// All-gather -> GEMM on the schedule with dedicated mover CTAs (gemm_ag_cta_movers.cu): CTAs
// [0, comm_ctas) stream the local shard to the peers with bulk copies through their operand ring
// and announce every 32 rows; the other CTAs compute, local shard first.
Status ag_gemm_cta_movers(Comm* c, const void* a_shard, const void* B, void* C, int M, int N, int K, cudaStream_t stream) {
  namespace v = agcta;
  const int n = c->nranks(), rpr = M / n;
  if ((rpr + v::kAgUnitRows - 1) / v::kAgUnitRows > v::kMaxUnits) return fail(kInvalidArgument, "more than %d rows per rank", v::kAgUnitRows * v::kMaxUnits);
  v::GemmLaunch g;
  memset(&g, 0, sizeof(g));
  c->fill_args(&g.p.coll);
  for (int r = 0; r < n; ++r) g.p.fflags[r] = (v::FusedFlags*)c->fused_flags(r);
  g.p.M = M;
  g.p.N = N;
  g.p.K = K;
  g.p.C = C;
  g.p.ldc = N;
  g.p.rows_per_rank = rpr;
  g.p.a_local = a_shard;
  g.p.mode = v::kGemmAllGather;
  Segment* seg = nullptr;
  AMEM_TRY(c->fused_segment(0, (size_t)M * K * 2, &seg));
  for (int r = 0; r < n; ++r) g.p.ag_buf[r] = (void*)seg->va[r];
  AMEM_TRY(v::make_tensor_map_bf16(&g.map_a, g.p.ag_buf[c->rank()], M, K, K, v::kGemmBM));
  AMEM_TRY(v::make_tensor_map_bf16(&g.map_a_local, a_shard, rpr, K, K, v::kGemmBM));
  if (c->emulated()) {
    g.grid = emu_grid(n);
    g.p.comm_ctas = 1;
  } else {
    g.grid = v::gemm_default_grid(c->device());
    g.p.comm_ctas = (int)env_long("AMEM_AG_COMM_CTAS", 16);
    if (g.p.comm_ctas < 1) g.p.comm_ctas = 1;
    if (g.p.comm_ctas > g.grid / 2) g.p.comm_ctas = g.grid / 2;
  }
  g.p.bn = v::gemm_pick_bn(n * ((rpr + v::kGemmBM - 1) / v::kGemmBM), N, g.grid - g.p.comm_ctas);
  AMEM_TRY(v::make_tensor_map_bf16(&g.map_b, B, N, K, K, g.p.bn));
  if (c->emulated())
    return c->emu()->rendezvous(c->rank(), 1100 + g.p.mode, &g, sizeof(g), stream,
                                [n](const void* host_all, const void*, cudaStream_t s) { return v::launch_gemm_emu((const v::GemmLaunch*)host_all, n, s); });
  return v::launch_gemm(g, stream);
}
}  // namespace

extern "C" {

// C[M, N] = allgather_rows(a_shard)[M, K] * B[N, K]^T.  Every rank passes its M/nranks rows;
// B and C are per rank (column-parallel weight shard and its output).
ncclResult_t amemAllGatherGemm(const void* a_shard, const void* B, void* C, int M, int N, int K, ncclComm_t comm, cudaStream_t stream) {
  if (!comm) return ncclInvalidArgument;
  Comm* c = reinterpret_cast<Comm*>(comm);
  Status s = c->check_usable("amemAllGatherGemm");
  if (s != kSuccess) return R(s);
  if ((s = check_shape(M, N, K)) != kSuccess) return R(s);
  int n = c->nranks();
  if (M % n) return R(fail(kInvalidArgument, "M=%d is not divisible by %d ranks", M, n));
  int rpr = M / n;
  if ((s = c->prepare_stream(stream)) != kSuccess) return R(s);
  if (n > 1 && !gemm_ag_uses_mover_warps(n)) return R(ag_gemm_cta_movers(c, a_shard, B, C, M, N, K, stream));
  GemmLaunch g;
  memset(&g, 0, sizeof(g));
  fill_fused(c, &g.p);
  g.p.M = M;
  g.p.N = N;
  g.p.K = K;
  g.p.C = C;
  g.p.ldc = N;
  g.p.rows_per_rank = rpr;
  g.p.a_local = a_shard;
  g.p.ag_unit_rows = gemm_ag_unit_rows(rpr, K);
  if (long ur = env_long("AMEM_AG_UNIT_ROWS", 0); ur > g.p.ag_unit_rows) g.p.ag_unit_rows = (int)std::min<long>(ur, rpr);   // coarser flags (never finer than the minimum)
  g.p.ag_mover = (int)env_long("AMEM_AG_MOVER", 1);
  g.p.ag_mover_warps = (int)std::max<long>(1, env_long("AMEM_AG_MOVER_WARPS", 2));
  g.p.ag_epi_help = (int)env_long("AMEM_AG_EPI_HELP", 0);
  // Every CTA computes (one extra warp of each moves data), so the tiling is planned like the plain
  // GEMM's: tile height, tile width and the split of the last wave along K.  The emulation runs all
  // ranks in one grid on one stream: they would share the split workspace, so it runs unsplit.
  g.grid = c->emulated() ? emu_grid(n) : gemm_default_grid(c->device());
  SplitKWs* ws = nullptr;
  if (n > 1 && !c->emulated() && env_long("AMEM_GEMM_SPLITK", 1) && !Registry::instance().is_paused(0))
    ws = splitk_workspace(c->device(), stream, g.grid);
  GemmPlan plan = plan_gemm(M, N, K, g.grid, ws != nullptr);
  if (rpr <= kGemmBM && plan.tall) {
    plan.tall = 0;
    plan.bn = gemm_pick_bn(n * ((rpr + kGemmBM - 1) / kGemmBM), N, g.grid, ws ? (K + kGemmBK - 1) / kGemmBK : 0, &plan.slices);
  }
  const int tile_rows = plan.tall ? 2 * kGemmBM : kGemmBM;
  g.p.tall = plan.tall;
  g.p.bn = plan.bn;
  if (ws && plan.slices > 1) {
    g.p.sk_slices = plan.slices;
    g.p.sk_ws = ws->partials;
    g.p.sk_ctr = ws->counters;
  }
  if (n == 1) {
    g.p.mode = kGemmPlain;
    if ((s = make_tensor_map_bf16(&g.map_a, a_shard, M, K, K, tile_rows)) != kSuccess) return R(s);
    g.map_a_local = g.map_a;
  } else {
    g.p.mode = kGemmAllGather;
    Segment* seg = nullptr;
    if ((s = c->fused_segment(0, (size_t)M * K * 2, &seg)) != kSuccess) return R(s);
    for (int r = 0; r < n; ++r) g.p.ag_buf[r] = (void*)seg->va[r];
    g.p.ag_mc = (K % 8 == 0) ? (void*)seg->mc_va : nullptr;
    if ((s = make_tensor_map_bf16(&g.map_a, g.p.ag_buf[c->rank()], M, K, K, tile_rows)) != kSuccess) return R(s);
    if ((s = make_tensor_map_bf16(&g.map_a_local, a_shard, rpr, K, K, tile_rows)) != kSuccess) return R(s);
  }
  if ((s = make_tensor_map_bf16(&g.map_b, B, N, K, K, g.p.bn)) != kSuccess) return R(s);
  s = run_gemm(c, g, stream);
  if (s != kSuccess && ws) cudaMemsetAsync(ws->counters, 0, gemm_splitk_ctr_words(g.grid) * sizeof(uint32_t), stream);
  return R(s);
}

// out[M/nranks, N] = reduce_scatter_rows(A[M, K] * B[N, K]^T): every rank holds a K-slice
// (row-parallel weight shard) and ends up with its M/nranks rows of the sum.
ncclResult_t amemGemmReduceScatter(const void* A, const void* B, void* out, int M, int N, int K, ncclComm_t comm, cudaStream_t stream) {
  if (!comm) return ncclInvalidArgument;
  Comm* c = reinterpret_cast<Comm*>(comm);
  Status s = c->check_usable("amemGemmReduceScatter");
  if (s != kSuccess) return R(s);
  if ((s = check_shape(M, N, K)) != kSuccess) return R(s);
  int n = c->nranks();
  if (M % n) return R(fail(kInvalidArgument, "M=%d is not divisible by %d ranks", M, n));
  int rpr = M / n;
  if ((rpr + kGemmBM - 1) / kGemmBM > kMaxUnits) return R(fail(kInvalidArgument, "more than %d rows per rank", kGemmBM * kMaxUnits));
  if ((s = c->prepare_stream(stream)) != kSuccess) return R(s);
  GemmLaunch g;
  memset(&g, 0, sizeof(g));
  fill_fused(c, &g.p);
  g.p.M = M;
  g.p.N = N;
  g.p.K = K;
  g.p.rows_per_rank = rpr;
  g.p.rs_out = out;
  g.grid = c->emulated() ? emu_grid(n) : gemm_default_grid(c->device());
  g.p.bn = gemm_pick_bn(n * ((rpr + kGemmBM - 1) / kGemmBM), N, g.grid);
  if (n == 1) {
    g.p.mode = kGemmPlain;
    g.p.C = out;
    g.p.ldc = N;
  } else {
    g.p.mode = kGemmReduceScatter;
    Segment* seg = nullptr;
    // tile-major partials: every (row block, column block) occupies a full 128 x 256 tile
    size_t tiles = (size_t)((rpr + kGemmBM - 1) / kGemmBM) * (size_t)((N + g.p.bn - 1) / g.p.bn);
    if ((s = c->fused_segment(1, (size_t)n * tiles * kGemmBM * g.p.bn * 2, &seg)) != kSuccess) return R(s);
    for (int r = 0; r < n; ++r) g.p.rs_buf[r] = (void*)seg->va[r];
  }
  if ((s = make_tensor_map_bf16(&g.map_a, A, M, K, K, kGemmBM)) != kSuccess) return R(s);
  g.map_a_local = g.map_a;
  if ((s = make_tensor_map_bf16(&g.map_b, B, N, K, K, g.p.bn)) != kSuccess) return R(s);
  return R(run_gemm(c, g, stream));
}

// ---- MoE expert parallelism -------------------------------------------------------------
// Collective: (re)allocates the symmetric receive and expert-output buffers of `capacity_rows`
// rows of d bf16 each and returns this rank's views.  Both are scratch: dropped on pause.
ncclResult_t amemMoeBuffers(ncclComm_t comm, int capacity_rows, int d, void** recv_x, void** y) {
  if (!comm || capacity_rows <= 0 || d <= 0 || d % 8) return ncclInvalidArgument;
  Comm* c = reinterpret_cast<Comm*>(comm);
  Status s = c->check_usable("amemMoeBuffers");
  if (s != kSuccess) return R(s);
  Segment *a = nullptr, *b = nullptr;
  size_t bytes = (size_t)capacity_rows * d * 2;
  if ((s = c->fused_segment(2, bytes, &a)) != kSuccess) return R(s);
  if ((s = c->fused_segment(3, bytes, &b)) != kSuccess) return R(s);
  if (recv_x) *recv_x = (void*)a->va[c->rank()];
  if (y) *y = (void*)b->va[c->rank()];
  return ncclSuccess;
}

static Status moe_args(Comm* c, int T, int k, int d, int E, int capacity_rows, MoeArgs* a) {
  if (T < 0 || k <= 0 || d <= 0 || d % 8 || E <= 0 || E > kMoeMaxExperts || E % c->nranks())
    return fail(kInvalidArgument, "MoE shape: T=%d k=%d d=%d (multiple of 8) E=%d (<= %d, divisible by %d ranks)", T, k, d, E, kMoeMaxExperts, c->nranks());
  if (capacity_rows <= 0) return fail(kInvalidArgument, "MoE capacity_rows must be positive, got %d", capacity_rows);
  Segment *rx = nullptr, *yb = nullptr;
  size_t bytes = (size_t)capacity_rows * d * 2;
  AMEM_TRY(c->fused_segment(2, bytes, &rx));
  AMEM_TRY(c->fused_segment(3, bytes, &yb));
  memset(a, 0, sizeof(*a));
  c->fill_args(&a->coll);
  a->T = T;
  a->k = k;
  a->d = d;
  a->E = E;
  a->capacity_rows = capacity_rows;
  for (int r = 0; r < c->nranks(); ++r) {
    a->recv[r] = (char*)rx->va[r];
    a->ybuf[r] = (char*)yb->va[r];
  }
  // small per-communicator work area: tracked scratch of the communicator (every word of it is
  // rewritten by each dispatch before it is read, so nothing has to survive a pause)
  void* wp = nullptr;
  size_t ints = (size_t)kMoeSegments * kMoeMaxExperts * 2 + kMoeMaxExperts + 64;
  AMEM_TRY(c->local_scratch(0, ints * sizeof(int), &wp));
  int* w = (int*)wp;
  a->seg_hist = w;
  a->seg_base = w + (size_t)kMoeSegments * kMoeMaxExperts;
  a->send_off = w + (size_t)kMoeSegments * kMoeMaxExperts * 2;
  a->dropped_rows = w + (size_t)kMoeSegments * kMoeMaxExperts * 2 + kMoeMaxExperts;
  return kSuccess;
}

// Routes this rank's T tokens to their experts' ranks.  On return (stream order) this rank's
// receive buffer holds the rows of its local experts, grouped by expert in (source rank, token)
// order; expert_counts[E/nranks] and expert_offsets[E/nranks + 1] describe the groups and
// send_pos[T*k] remembers where every (token, choice) went (needed by amemMoeCombine).
//
// Capacity: a rank that is routed more rows than capacity_rows keeps the first capacity_rows of
// them (rows are ordered by expert, then source rank, then token); the rest are not sent, their
// send_pos is -1 (amemMoeCombine gives them weight zero), expert_counts / expert_offsets count
// only stored rows, and *dropped_rows (optional device int) receives how many this rank left
// out.  The communicator stays usable: overflow is a result of the call, not an error state.
ncclResult_t amemMoeDispatchCounted(const void* x, const int* topk_idx, int T, int k, int d, int E, int capacity_rows, int* expert_counts,
                                    int* expert_offsets, int* send_pos, int* dropped_rows, ncclComm_t comm, cudaStream_t stream);
ncclResult_t amemMoeDispatch(const void* x, const int* topk_idx, int T, int k, int d, int E, int capacity_rows, int* expert_counts,
                             int* expert_offsets, int* send_pos, ncclComm_t comm, cudaStream_t stream) {
  return amemMoeDispatchCounted(x, topk_idx, T, k, d, E, capacity_rows, expert_counts, expert_offsets, send_pos, nullptr, comm, stream);
}
ncclResult_t amemMoeDispatchCounted(const void* x, const int* topk_idx, int T, int k, int d, int E, int capacity_rows, int* expert_counts,
                                    int* expert_offsets, int* send_pos, int* dropped_rows, ncclComm_t comm, cudaStream_t stream) {
  if (!comm) return ncclInvalidArgument;
  Comm* c = reinterpret_cast<Comm*>(comm);
  Status s = c->check_usable("amemMoeDispatch");
  if (s != kSuccess) return R(s);
  MoeArgs a;
  if ((s = moe_args(c, T, k, d, E, capacity_rows, &a)) != kSuccess) return R(s);
  if ((s = c->prepare_stream(stream)) != kSuccess) return R(s);
  a.x = x;
  a.topk_idx = topk_idx;
  a.expert_counts = expert_counts;
  a.expert_offsets = expert_offsets;
  a.send_pos = send_pos;
  if (dropped_rows) a.dropped_rows = dropped_rows;
  if (c->emulated()) {
    int n = c->nranks();
    return R(c->emu()->rendezvous(c->rank(), 2001, &a, sizeof(a), stream, [n](const void* h, const void* dv, cudaStream_t st) {
      return launch_moe_dispatch_emu((const MoeArgs*)h, (const MoeArgs*)dv, n, st);
    }));
  }
  return R(launch_moe_dispatch(a, stream));
}

// out[T, d] = sum_j topk_w[t, j] * (expert output row of (t, j)), read from the expert ranks'
// output buffers (the `y` of amemMoeBuffers, rows in the layout the dispatch produced).
ncclResult_t amemMoeCombine(const int* topk_idx, const float* topk_w, const int* send_pos, void* out, int T, int k, int d, int E,
                            int capacity_rows, ncclComm_t comm, cudaStream_t stream) {
  if (!comm) return ncclInvalidArgument;
  Comm* c = reinterpret_cast<Comm*>(comm);
  Status s = c->check_usable("amemMoeCombine");
  if (s != kSuccess) return R(s);
  MoeArgs a;
  if ((s = moe_args(c, T, k, d, E, capacity_rows, &a)) != kSuccess) return R(s);
  if ((s = c->prepare_stream(stream)) != kSuccess) return R(s);
  a.topk_idx = topk_idx;
  a.topk_w = topk_w;
  a.send_pos = const_cast<int*>(send_pos);
  a.out = out;
  if (c->emulated()) {
    int n = c->nranks();
    return R(c->emu()->rendezvous(c->rank(), 2002, &a, sizeof(a), stream, [n](const void* h, const void* dv, cudaStream_t st) {
      return launch_moe_combine_emu((const MoeArgs*)h, (const MoeArgs*)dv, n, st);
    }));
  }
  return R(launch_moe_combine(a, stream));
}

}  // extern "C"
