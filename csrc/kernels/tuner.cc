// Variant picker: one-shot / two-shot / NVLS for all-reduce, grid size and chunking for
// everything.  The thresholds were set from bus-bandwidth sweeps on 8 x B200 over NVSwitch;
// AMEM_ALGO (oneshot|twoshot|nvls), AMEM_ONESHOT_MAX_KB and AMEM_BLOCKS override them.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../core/log.h"
#include "launch.h"

namespace amem {

static int env_algo() {
  static int v = [] {
    std::string s = env_str("AMEM_ALGO", "");
    if (s == "oneshot") return (int)kAlgoOneShot;
    if (s == "twoshot") return (int)kAlgoTwoShot;
    if (s == "nvls") return (int)kAlgoNvls;
    return (int)kAlgoAuto;
  }();
  return v;
}

LaunchPlan plan_collective(const TunerInput& in) {
  LaunchPlan p;
  p.threads = 512;
  p.algo = kAlgoAuto;
  const size_t es = dtype_size(in.dtype);
  const int n = in.nranks;
  const size_t Q = quarter_bytes(in.stage_bytes, in.p2p_slot_bytes);
  const size_t slot = slot_bytes_of(Q, n);
  static const long oneshot_kb = env_long("AMEM_ONESHOT_MAX_KB", 256);
  static const long blocks_env = env_long("AMEM_BLOCKS", 0);
  size_t bytes = in.count * es;  // payload that defines the work of one rank
  switch (in.kind) {
    case kCollAllGather: case kCollAllToAll: bytes *= (size_t)n; break;
    case kCollReduceScatter: bytes *= (size_t)n; break;
    default: break;
  }
  if (in.kind == kCollAllReduce) {
    int want = in.forced_algo != kAlgoAuto ? in.forced_algo : env_algo();
    // Between two GPUs the switch has nothing to add: plain peer stores (two-shot) measured
    // 1.7x the NVLS rate there, so NVLS is only picked by default from three ranks up.
    bool nvls_ok = in.nvls && n > 1 && (in.redop == kSum || in.redop == kAvg) &&
                   (in.dtype == kF32 || in.dtype == kBF16 || in.dtype == kF16);
    // Between two GPUs one-shot moves exactly the bytes two-shot does, with one barrier instead
    // of two: measured faster up to 16 MiB (1 MiB: 27.6 vs 39.1 us; 8 MiB: 43.0 vs 52.6 us).
    static const bool oneshot_set = getenv("AMEM_ONESHOT_MAX_KB") != nullptr;
    size_t one_max = std::min(slot, (n == 2 && !oneshot_set) ? ((size_t)16 << 20) : ((size_t)oneshot_kb << 10));
    // Registered windows: in place, no staging.  Taken from AMEM_WINDOW_MIN_KB (default 512) up;
    // below that the one-shot exchange through staging has one barrier less.
    static const long win_min_kb = env_long("AMEM_WINDOW_MIN_KB", 512);
    if (in.window && want == kAlgoAuto && n > 1 && in.count * es >= ((size_t)win_min_kb << 10)) want = kAlgoWindow;
    if (want == kAlgoWindow && !in.window) want = kAlgoAuto;
    if (want == kAlgoNvls && !nvls_ok) want = kAlgoAuto;
    if (want == kAlgoOneShot && in.count * es > slot) want = kAlgoAuto;
    if (want == kAlgoAuto) {
      if (in.count * es <= one_max) want = kAlgoOneShot;
      else if (nvls_ok && n > 2) want = kAlgoNvls;
      else want = kAlgoTwoShot;
    }
    p.algo = want;
  }
  // All-gather may push through the multicast mapping (multimem.st: one store instead of n-1);
  // opt-in with AMEM_AG_NVLS=1 or AMEM_ALGO=nvls until it has been measured to win.
  if (in.kind == kCollAllGather && in.nvls && n > 1) {
    static const long ag_nvls = env_long("AMEM_AG_NVLS", 0);
    if (ag_nvls || env_algo() == kAlgoNvls || in.forced_algo == kAlgoNvls) p.algo = kAlgoNvls;
  }
  // Small all-to-all as flag-in-data packets, no barrier: opt-in with AMEM_LL=1.  Measured on 8 GPUs it
  // lost to the barrier form at every size (2 KiB: 38 vs 27 us; 512 KiB: 72 vs 36 us): 8-byte packets
  // polled word by word cost more than one barrier saves.  The payload of one peer must fit half a slot.
  static const long ll_on = env_long("AMEM_LL", 0);
  const bool ll = in.kind == kCollAllToAll && n > 1 && ll_on && in.count * es <= ll_slot_bytes(in.p2p_slot_bytes) / 2;
  if (ll) p.algo = kAlgoLL;
  // Reduce to a root: from 1 MiB up, through the switch (the root pulls one reduced stream) instead of
  // n - 1 pushes into the root.  Sum of fp32 / fp16 / bf16, three ranks or more, 16-byte aligned counts.
  if (in.kind == kCollReduce && in.nvls && n > 2 && (in.redop == kSum || in.redop == kAvg) &&
      (in.dtype == kF32 || in.dtype == kBF16 || in.dtype == kF16) && in.count * es >= (1u << 20) && env_algo() != kAlgoTwoShot)
    p.algo = kAlgoNvls;
  // Grid: one block per 32 KiB of work up to the communicator's cap; latency-bound sizes use
  // few blocks because every block waits on its own set of peer flags.
  size_t per_block = 32 << 10;
  if (in.kind == kCollAllReduce && p.algo == kAlgoOneShot) per_block = 16 << 10;
  long blocks = (long)((bytes + per_block - 1) / per_block);
  if (blocks < 1) blocks = 1;
  if (blocks > in.max_blocks) blocks = in.max_blocks;
  if (in.kind == kCollAllReduce && p.algo == kAlgoWindow) {
    // every block streams through the switch (or the peers) with many loads in flight; enough
    // blocks to fill the links, not one per 32 KiB
    static const long win_blocks = env_long("AMEM_WINDOW_BLOCKS", 0);
    long want_b = (long)((bytes / (size_t)n + (64 << 10) - 1) / (64 << 10));
    blocks = std::max<long>(1, std::min<long>(want_b, win_blocks > 0 ? win_blocks : in.max_blocks));
  }
  // always the same number of blocks: the blocks' operation counts (the packets' flag) then move in
  // lockstep, so a word's flag depends on the operation only, never on which block wrote it
  if (ll) blocks = std::min<long>(4, in.max_blocks);
  if (blocks_env > 0 && !ll) blocks = std::min<long>(blocks_env, in.max_blocks);
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  p.blocks = (int)blocks;
  // Chunk: messages that span several chunks overlap their NVLink and HBM phases (see
  // coll_bodies.inl), so aim for about eight chunks, but never chunks so small that the
  // per-chunk barrier (a few microseconds) shows, nor larger than the staging region.
  const size_t H = 2 * Q;
  // A chunk of the credit pipeline costs about 12 us over its share of the transfer (measured
  // between two GPUs: the two warp groups each run at half the block's memory parallelism), so
  // chunks are as large as staging allows: messages up to `single_bytes` go as one chunk, larger
  // ones in about eight chunks of at least `min_bytes`, never more than `max_bytes`.
  // AMEM_SINGLE_MB / AMEM_CHUNK_MB / AMEM_CHUNKS override the three numbers (experiments).
  static const long env_single_mb = env_long("AMEM_SINGLE_MB", 0), env_min_mb = env_long("AMEM_CHUNK_MB", 0);
  static const long env_parts = std::max<long>(1, env_long("AMEM_CHUNKS", 8));
  auto pick = [&](size_t total_bytes, size_t single_bytes, size_t min_bytes, size_t max_bytes) {
    if (env_single_mb > 0) single_bytes = (size_t)env_single_mb << 20;
    if (env_min_mb > 0) min_bytes = (size_t)env_min_mb << 20;
    size_t c = total_bytes <= single_bytes ? total_bytes : total_bytes / (size_t)env_parts;
    if (total_bytes > single_bytes && c < min_bytes) c = min_bytes;
    if (c > max_bytes) c = max_bytes;
    c = (c + 4095) & ~(size_t)4095;
    if (c > max_bytes) c = max_bytes & ~(size_t)4095;
    return c ? c : (size_t)4096;
  };
  switch (in.kind) {
    case kCollAllReduce:
      if (p.algo == kAlgoNvls) {
        // A message above 32 MiB goes in AMEM_NVLS_CHUNKS chunks (default 8) of at least
        // AMEM_NVLS_CHUNK_MB (default 16): more, smaller chunks fill the three-stage pipeline
        // sooner, but each chunk costs two rounds of credits.
        static const long parts = std::max<long>(1, env_long("AMEM_NVLS_CHUNKS", 8));
        static const long min_mb = std::max<long>(1, env_long("AMEM_NVLS_CHUNK_MB", 16));
        const size_t total = in.count * es, lo = (size_t)min_mb << 20, cap = (H / 3) & ~(size_t)4095;
        size_t c = total <= ((size_t)32 << 20) ? total : std::max(lo, total / (size_t)parts);
        c = std::min(c, cap);
        c = (c + 4095) & ~(size_t)4095;
        if (c > cap) c = cap;
        p.chunk_elems = std::max<size_t>(c, 4096) / es;
      }
      else p.chunk_elems = pick(in.count * es, 64u << 20, 32u << 20, (slot_bytes_of(H / 2, n)) * (size_t)n) / es;
      break;
    case kCollBroadcast: p.chunk_elems = pick(in.count * es, 16u << 20, 8u << 20, Q) / es; break;  // one chunk up to 16 MiB, then about eight
    case kCollReduce: p.chunk_elems = (p.algo == kAlgoNvls ? H : slot) / es; break;
    default: p.chunk_elems = pick(in.count * es, 64u << 20, 32u << 20, slot) / es; break;  // per-rank bytes
  }
  if (p.chunk_elems == 0) p.chunk_elems = 1;
  return p;
}

}  // namespace amem
