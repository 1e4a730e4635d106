// tcgen05 / TMEM / TMA GEMM for sm_100a, alone and fused with its neighbouring collective.
//
//   plain            C = A * B^T
//   all-gather->GEMM  A's row shards live on different ranks.  One extra warp of EVERY CTA streams
//                    a slice of this rank's shard into every peer's gathered buffer with bulk
//                    async copies (global -> shared once, shared -> each peer; 8 KB pieces through
//                    a small staging area beside the operand ring) and announces every few rows
//                    with a flag, so all SMs compute: they start on the local shard at once and
//                    pick up remote row blocks in the order they arrive.
//   GEMM->reduce-scatter  each output row block belongs to one rank.  The epilogue stores
//                    bf16 partial tiles straight into the owner's slot buffer over NVLink and
//                    counts them in; when a CTA runs out of tiles it reduces finished row
//                    blocks of its own shard in fixed rank order (deterministic).
//
// One CTA per SM, persistent over tiles of 128 x 256, K step 64, 4-stage TMA ring, one elected
// thread issues tcgen05.mma (kind::f16, M128 N256 K16) into one of two 256-column TMEM
// accumulators so the epilogue of tile i overlaps the main loop of tile i+1.  TMA loads never
// use cluster multicast and only ever read this GPU's own memory; peers are reached with plain
// or bulk stores.  Every wait is bounded and ends in an error status, not a hang.
//
// The plain and all-gather modes have two more forms, chosen per problem by the host (gemm_tall_pays,
// gemm_tail_slices): tiles of 256 x 256 (template parameter MT = 2: two 128-row accumulators fill
// all 512 TMEM columns and share one B tile, 3 stages of 64 KB, eight epilogue warps), and a
// split of the partly filled last wave of tiles along K (its CTAs park fp32 partial accumulators
// in a workspace, meet on a counter, and each sums one band of rows over all slices in slice
// order, fetching the bands with bulk copies into the idle operand ring).
#include <algorithm>
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include "../core/log.h"
#include "coll_device.cuh"
#include "gemm_sm100.h"
#include "sm100_prims.cuh"

namespace amem {
namespace gemmk {

using namespace sm100;

constexpr int BM = kGemmBM, BN_MAX = kGemmBN, BK = kGemmBK, STAGES = kGemmStages;
// A stage always reserves room for the widest tile; the tile width itself (p.bn, a multiple of
// 32 up to 256) is picked per problem so that the last wave of tiles is not nearly empty.
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN_MAX * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int UMMA_K = 16;
constexpr uint32_t TMEM_COLS = 512;
constexpr int COPY_PIECE = 32 * 1024;  // bytes per bulk copy when split-K partials are fetched into the ring
constexpr int EPI_CHUNK_BYTES = BM * 32 * 2;  // one 32-column chunk of a tile in bf16
// Staging beside the ring: two chunks for the reduce-scatter epilogue, or four pieces of the
// all-gather mover (the two modes never run in one launch).
constexpr int SIDE_BUFS = 4;   // a power of two
static_assert(kAgPieceBytes == EPI_CHUNK_BYTES, "the mover's pieces use the epilogue's staging buffers");
// A parked (split-K) accumulator: BN/4 column groups x (rows of every band padded to an odd
// count) x 4 floats; bands x padded rows <= BM + 2 * slices <= BM + 64.
constexpr int SK_MAX_SLICES = 32;
constexpr size_t SK_SLOT_FLOATS = (size_t)(BN_MAX / 4) * (BM + 2 * SK_MAX_SLICES) * 4;

struct __align__(8) SmemCtl {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  uint64_t tfull[2];
  uint64_t tempty[2];
  uint64_t copy_full[STAGES];   // all-gather mover: a piece has landed in side buffer s
  uint64_t sk_full;             // split-K fix-up: the bands of all slices have landed in the ring
  uint32_t tmem_base;
  int abort;
  int s_abort_coll;
  int mover_go;     // all-gather: the cross-launch guard has passed, peers may be written
  int next_unit;    // all-gather: next unit (in this CTA's sequence) a mover warp takes
};

struct Tile {
  int shard;      // owner rank of the rows (0 when not fused); grouped: the group
  int m_in;       // row-block index inside the shard / group
  int n_blk;
  int row0;       // grouped: first row of the tile in A and C
  int rows;       // grouped: rows of the tile that belong to its group
};

// Grouped mode: tiles of all groups in one sequence, group after group, row blocks fastest.
__device__ __forceinline__ int grouped_total_tiles(const GemmParams& p, int tiles_n) {
  int total = 0;
  for (int e = 0; e < p.groups; ++e) total += ((p.group_off[e + 1] - p.group_off[e] + BM - 1) / BM) * tiles_n;
  return total;
}
__device__ __forceinline__ Tile grouped_tile_of(const GemmParams& p, int t, int tiles_n) {
  Tile o;
  o.shard = o.m_in = o.n_blk = o.row0 = o.rows = 0;
  int acc = 0, first = p.group_off[0];
  for (int e = 0; e < p.groups; ++e) {
    const int next = p.group_off[e + 1];
    const int rows = next - first, tm = (rows + BM - 1) / BM, cnt = tm * tiles_n;
    if (t < acc + cnt) {
      const int v = t - acc;
      o.shard = e;
      o.m_in = v % tm;
      o.n_blk = v / tm;
      o.row0 = first + o.m_in * BM;
      o.rows = min(BM, rows - o.m_in * BM);
      return o;
    }
    acc += cnt;
    first = next;
  }
  return o;
}

// One unit of work of a compute CTA: a whole tile, or (tail split) a range of K blocks of one.
struct Work {
  int t, kb0, kb1;
  int slice;   // -1: whole tile
};
// CTA g of G runs `full_waves` whole tiles (t = g, g + G, ...) and then at most one item of the
// last wave: a whole tile when that wave is not split, else slice g % S of tail tile g / S.
__device__ __forceinline__ int work_count(int g, int G, int total_tiles, int S) {
  const int full = total_tiles / G, rem = total_tiles - full * G;
  return full + ((S > 1 ? g < rem * S : g < rem) ? 1 : 0);
}
__device__ __forceinline__ Work work_of(int i, int g, int G, int total_tiles, int S, int num_kb) {
  const int full = total_tiles / G;
  Work w;
  if (i < full || S <= 1) {
    w.t = g + i * G;
    w.kb0 = 0;
    w.kb1 = num_kb;
    w.slice = -1;
  } else {
    w.t = full * G + g / S;
    w.slice = g % S;
    w.kb0 = (int)((long)w.slice * num_kb / S);
    w.kb1 = (int)((long)(w.slice + 1) * num_kb / S);
  }
  return w;
}

// Tile order.  plain: row blocks fastest (CTAs that run together share the B tile in L2).
// all-gather: the local shard first, then row block by row block across the source ranks
// nearest-sender first, the order in which the movers deliver.  reduce-scatter: remote
// owners first (rank+1, rank+2, ...), my own rows last.
__device__ __forceinline__ Tile tile_of(const GemmParams& p, int t, int tiles_m, int tiles_n) {
  const int n = p.coll.nranks, r = p.coll.rank;
  if (p.mode == kGemmGrouped) return grouped_tile_of(p, t, tiles_n);
  Tile o;
  o.row0 = o.rows = 0;
  if (p.mode == kGemmAllGather && n > 1) {
    int own = tiles_m * tiles_n;
    if (t < own) {
      o.shard = r;
      o.m_in = t % tiles_m;
      o.n_blk = t / tiles_m;
    } else {
      // Remote rows: bands of a few row blocks (all sources, all column blocks per band), so the
      // tiles in flight share B tiles in L2 while the next band is still arriving.
      int u = t - own;
      const int GM2 = max(1, 16 / (n - 1));
      const int band_tiles = GM2 * (n - 1) * tiles_n;
      const int band = u / band_tiles;
      const int first_m = band * GM2;
      const int gm = min(GM2, tiles_m - first_m);
      const int w = u - band * band_tiles;
      o.m_in = first_m + w % gm;
      const int rest = w / gm;
      o.shard = (r - 1 - (rest % (n - 1)) + 2 * n) % n;
      o.n_blk = rest / (n - 1);
    }
  } else {
    int per_shard = tiles_m * tiles_n;
    int s = t / per_shard, v = t % per_shard;
    o.shard = (p.mode == kGemmReduceScatter && n > 1) ? (r + 1 + s) % n : s;
    // Bands of 16 row blocks: the ~148 tiles in flight then span 16 row blocks x ~9 column
    // blocks, so both operands are re-used out of L2 instead of streaming all of A from HBM
    // once per column block.
    const int GM = 16;
    const int band = v / (GM * tiles_n);
    const int first_m = band * GM;
    const int gm = min(GM, tiles_m - first_m);
    const int w = v - band * GM * tiles_n;
    o.m_in = first_m + w % gm;
    o.n_blk = w / gm;
  }
  return o;
}

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---- all-gather mover: one thread per CTA drives bulk copies through the side buffers; a unit
// = p.ag_unit_rows rows of my shard, contiguous in memory; CTA c moves units c, c + nctas, ... so
// the CTAs together deliver the shard roughly front to back.  Loads run two pieces ahead of the
// stores; a piece is read from HBM once and stored to every peer.
struct PieceIter {
  int u;        // current unit
  size_t o;     // byte offset inside the unit
  bool valid;
};
__device__ __forceinline__ size_t unit_bytes(const GemmParams& p, int u) {
  int rows = min(p.ag_unit_rows, p.rows_per_rank - u * p.ag_unit_rows);
  return (size_t)rows * (size_t)p.K * 2;
}
__device__ __forceinline__ void piece_next(const GemmParams& p, int units, int nctas, PieceIter& it) {
  it.o += kAgPieceBytes;
  if (it.o >= unit_bytes(p, it.u)) {
    it.o = 0;
    it.u += nctas;
    it.valid = it.u < units;
  }
}
__device__ void ag_mover(const GemmParams& p, char* bufs, SmemCtl* ctl, int cta, int nctas, uint32_t epoch) {
  const int n = p.coll.nranks, r = p.coll.rank;
  const size_t row_bytes = (size_t)p.K * 2;
  const size_t unit_stride = (size_t)p.ag_unit_rows * row_bytes;
  const int units = (p.rows_per_rank + p.ag_unit_rows - 1) / p.ag_unit_rows;
  const char* src = (const char*)p.a_local;
  const size_t shard_off = (size_t)r * p.rows_per_rank * row_bytes;
  uint32_t phase_bits = 0;  // parity of copy_full[s], one bit per buffer
  PieceIter ld{cta, 0, cta < units}, st = ld;
  auto issue_load = [&](const PieceIter& it, int k) {
    size_t ub = unit_bytes(p, it.u);
    uint32_t len = (uint32_t)min((size_t)kAgPieceBytes, ub - it.o);
    int s = k % SIDE_BUFS;
    mbar_expect_tx(&ctl->copy_full[s], len);
    bulk_g2s(bufs + (size_t)s * kAgPieceBytes, src + (size_t)it.u * unit_stride + it.o, len, &ctl->copy_full[s]);
  };
  int loaded = 0;
  for (; loaded < 2 && ld.valid; ++loaded) {
    issue_load(ld, loaded);
    piece_next(p, units, nctas, ld);
  }
  for (int k = 0; st.valid; ++k) {
    const int s = k % SIDE_BUFS;
    if (!mbar_wait(&ctl->copy_full[s], (phase_bits >> s) & 1u, p.coll.timeout_ns, &ctl->abort)) {
      // gave up: let the loads already in flight land before the CTA exits
      for (int k2 = k; k2 < loaded; ++k2) {
        const int s2 = k2 % SIDE_BUFS;
        for (int i = 0; i < 100000 && !mbar_try_wait(&ctl->copy_full[s2], (phase_bits >> s2) & 1u); ++i) {
        }
      }
      break;
    }
    phase_bits ^= 1u << s;
    const size_t ub = unit_bytes(p, st.u);
    const uint32_t len = (uint32_t)min((size_t)kAgPieceBytes, ub - st.o);
    const size_t dst_off = shard_off + (size_t)st.u * unit_stride + st.o;
    char* buf = bufs + (size_t)s * kAgPieceBytes;
    for (int q1 = 1; q1 < n; ++q1) bulk_s2g((char*)p.ag_buf[(r + q1) % n] + dst_off, buf, len);
    if (p.copy_own) bulk_s2g((char*)p.ag_buf[r] + dst_off, buf, len);
    bulk_commit();
    const bool unit_done = st.o + len >= ub;
    const int unit = st.u;
    piece_next(p, units, nctas, st);
    if (ld.valid) {
      // the buffer of piece k+2 was last read by the stores of piece k-2: let all but the
      // newest store group finish reading, then refill it
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      issue_load(ld, k + 2);
      loaded = k + 3;
      piece_next(p, units, nctas, ld);
    }
    if (unit_done) {
      bulk_wait_all();  // this unit's bytes have been written
      __threadfence_system();
      for (int q1 = 1; q1 < n; ++q1) dev::st_release_sys(&p.fflags[(r + q1) % n]->ag_ready[r][unit], epoch);
      if (p.copy_own) dev::st_release_sys(&p.fflags[r]->ag_ready[r][unit], epoch);
    }
  }
  bulk_wait_all();  // nothing of this CTA's shared memory is still being read when it exits
}

// One unit of the shard (p.ag_unit_rows rows) to every peer, by one warp; nothing is fenced or
// announced yet.
__device__ __forceinline__ void ag_copy_unit(const GemmParams& p, int u, int lane) {
  const int n = p.coll.nranks, r = p.coll.rank;
  const size_t row_bytes = (size_t)p.K * 2;
  const size_t unit_stride = (size_t)p.ag_unit_rows * row_bytes;
  const size_t shard_off = (size_t)r * p.rows_per_rank * row_bytes;
  const size_t nvec = unit_bytes(p, u) / 16;
  const uint4* src = (const uint4*)((const char*)p.a_local + (size_t)u * unit_stride);
  const size_t dst_off = shard_off + (size_t)u * unit_stride;
  for (size_t i0 = 0; i0 < nvec; i0 += 256) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const size_t i = i0 + (size_t)j * 32 + lane;
      if (i < nvec) v[j] = __ldg(src + i);
    }
    if (p.ag_mc) {
      // one store per 16 bytes, replicated into every rank's gathered buffer by the switch
      char* dst = (char*)p.ag_mc + dst_off;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const size_t i = i0 + (size_t)j * 32 + lane;
        if (i < nvec)
          asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dst + i * 16), "r"(v[j].x), "r"(v[j].y), "r"(v[j].z), "r"(v[j].w) : "memory");
      }
    } else {
      for (int q1 = p.copy_own ? 0 : 1; q1 < n; ++q1) {
        uint4* dst = (uint4*)((char*)p.ag_buf[(r + q1) % n] + dst_off);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const size_t i = i0 + (size_t)j * 32 + lane;
          if (i < nvec) dst[i] = v[j];
        }
      }
    }
  }
}
// Announces unit u to every peer: each lane first makes its own stores visible system-wide.
__device__ __forceinline__ void ag_flag_unit(const GemmParams& p, int u, uint32_t epoch, int lane) {
  const int n = p.coll.nranks, r = p.coll.rank;
  __threadfence_system();
  __syncwarp();
  if (lane < n && (lane != 0 || p.copy_own)) dev::st_release_sys(&p.fflags[(r + lane) % n]->ag_ready[r][u], epoch);
}
// The CTA's warps that move data share its sequence of units (cta, cta + nctas, ...): each takes
// the next one.  Returns -1 when none is left.
__device__ __forceinline__ int ag_take_unit(const GemmParams& p, SmemCtl* ctl, int cta, int nctas, int lane) {
  const int units = (p.rows_per_rank + p.ag_unit_rows - 1) / p.ag_unit_rows;
  int k = 0;
  if (lane == 0) k = atomicAdd(&ctl->next_unit, 1);
  k = __shfl_sync(0xffffffffu, k, 0);
  const int u = cta + k * nctas;
  return u < units ? u : -1;
}
// The same job as ag_mover with plain loads and stores by whole warps (several per CTA, so that
// enough bytes are in flight to cover the link's latency): nothing of it goes through the SM's
// bulk-copy engine, which the operand loads of the main loop depend on.
__device__ void ag_mover_lsu(const GemmParams& p, SmemCtl* ctl, int cta, int nctas, uint32_t epoch, int lane) {
  for (int u; (u = ag_take_unit(p, ctl, cta, nctas, lane)) >= 0;) {
    ag_copy_unit(p, u, lane);
    ag_flag_unit(p, u, epoch, lane);
  }
}

// ---- reduce phase of GEMM -> reduce-scatter: out = sum over source slots, fixed order.
// Partials sit tile-major: [slot][row block][column block][32-column chunk][128 rows][32 cols],
// which is what lets the epilogue ship each 8 KB chunk with one bulk store.
__device__ void rs_reduce(const GemmParams& p, SmemCtl* ctl, int cta, int nctas, int tiles_m, int tiles_n) {
  const int n = p.coll.nranks, r = p.coll.rank;
  const int tid = threadIdx.x;
  const FusedFlags* mine = p.fflags[r];
  const __nv_bfloat16* slots = (const __nv_bfloat16*)p.rs_buf[r];
  __nv_bfloat16* out = (__nv_bfloat16*)p.rs_out;
  const int BN = p.bn;
  const size_t tile_elems = (size_t)BM * BN;
  const size_t slot_elems = (size_t)tiles_m * tiles_n * tile_elems;
  const uint32_t per_call = (uint32_t)tiles_n;  // one count per delivered tile
  volatile int* abort = &ctl->abort;
  for (int item = cta; item < tiles_m * tiles_n; item += nctas) {
    int m_in = item % tiles_m, n_blk = item / tiles_m;
    if (tid < n) {
      uint32_t want = dev::ld_volatile(&mine->rs_expect[tid][m_in]) + per_call;
      if (!*abort && !dev::wait_flag_ge(&mine->rs_done[tid][m_in], want, p.coll.timeout_ns)) {
        dev::report_error(p.coll.status, kDevGemmTimeout, r, tid, m_in, want);
        *abort = 1;
      }
    }
    __syncthreads();
    int row0 = m_in * BM, col0 = n_blk * BN;
    int rows = min(BM, p.rows_per_rank - row0);
    int cols = min(BN, p.N - col0);
    int vec_per_row = cols / 8;  // N % 8 == 0
    const size_t tile_base = ((size_t)m_in * tiles_n + n_blk) * tile_elems;
    for (int i = tid; i < rows * vec_per_row; i += blockDim.x) {
      int rr = i / vec_per_row, cv = i % vec_per_row;
      // inside a 64-byte row the four 16-byte pieces are rotated by the row number (the
      // epilogue does that to spread its shared-memory stores over the banks)
      size_t e_in = tile_base + (size_t)(cv / 4) * (BM * 32) + (size_t)rr * 32 + (size_t)(((cv % 4) + rr) & 3) * 8;
      float acc[8];
      uint4 raw[kMaxRanks];
#pragma unroll
      for (int s2 = 0; s2 < kMaxRanks; ++s2)
        if (s2 < n) raw[s2] = *(const uint4*)(slots + (size_t)s2 * slot_elems + e_in);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
      for (int s2 = 0; s2 < kMaxRanks; ++s2) {
        if (s2 < n) {
          const __nv_bfloat16* h = (const __nv_bfloat16*)&raw[s2];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += __bfloat162float(h[j]);
        }
      }
      alignas(16) __nv_bfloat16 res[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) res[j] = __float2bfloat16_rn(acc[j]);
      *(uint4*)(out + (size_t)(row0 + rr) * p.N + col0 + cv * 8) = *(const uint4*)res;
    }
    __syncthreads();
  }
}

// ---- the kernel body, shared by the one-rank-per-GPU kernel and the emulation kernel -------
template <int MT>  // accumulators (128-row halves) per tile: 1, or 2 for the tall tiles of the plain and all-gather modes
__device__ void gemm_body(const GemmParams& p, const CUtensorMap* map_a, const CUtensorMap* map_a_local, const CUtensorMap* map_b,
                          int cta, int nctas, char* smem_raw) {
  // operand ring first (1024-byte aligned for the 128-byte swizzle), control words after it
  char* ring = (char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  char* epi_stage = ring + (size_t)STAGES * STAGE_BYTES;  // 4 x 8 KB: reduce-scatter epilogue (2) or all-gather mover (4)
  SmemCtl* ctl = (SmemCtl*)(epi_stage + SIDE_BUFS * EPI_CHUNK_BYTES);
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int n = p.coll.nranks, r = p.coll.rank;
  const bool fused = n > 1 && p.mode != kGemmPlain;
  volatile int* abort = &ctl->abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
      mbar_init(&ctl->copy_full[s], 1);
    }
    mbar_init(&ctl->sk_full, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ctl->tfull[b], 1);
      mbar_init(&ctl->tempty[b], 4 * MT);  // one arrival per epilogue warp
    }
    ctl->abort = 0;
    ctl->mover_go = 0;
    ctl->next_unit = 0;
    mbar_fence_init();
    tma_prefetch_desc(map_a);
    tma_prefetch_desc(map_b);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  // protocol state of this launch (epochs, operation counter)
  dev::Proto proto;
  dev::proto_begin(proto, p.coll, cta, nctas, &ctl->s_abort_coll);  // contains a __syncthreads
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t epoch = proto.opseq + 1u;  // value of this launch's all-gather ready flags

  // Cross-launch guard: before anything of this launch lands in a peer's buffer, the peer must
  // have left the previous launch (it signals this barrier only after starting this one).  The
  // reduce-scatter epilogue writes to peers from every warp: the whole CTA waits.  In the all-gather
  // mode only the mover warp writes to peers: it alone exchanges the flags (mover_barrier below,
  // same flag words and epoch as block_barrier) and the compute warps start at once.
  const bool ag = p.mode == kGemmAllGather && fused;
  constexpr int MOVER_WARP = 2 + 4 * MT;   // the first mover warp; the warps behind it are movers too
  if (fused && p.mode == kGemmReduceScatter) dev::block_barrier(proto);
  if (ag) proto.epoch += 1;

  // Tall tiles (plain and all-gather modes): MT = 2 accumulators of 128 rows share one B tile; the
  // ring then holds 3 stages of 64 KB (A 32 KB + B 32 KB) instead of 4 of 48 KB.
  constexpr int TM = BM * MT;                                   // rows of a tile
  constexpr int n_stages = MT == 2 ? 3 : STAGES;
  constexpr int a_bytes = A_BYTES * MT;
  constexpr size_t stage_bytes = MT == 2 ? (size_t)(2 * A_BYTES + B_BYTES) : (size_t)STAGE_BYTES;
  const int tiles_m = (p.rows_per_rank + TM - 1) / TM;
  const int BN = p.bn;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int shards = (p.mode == kGemmPlain || n == 1) ? 1 : n;
  const int total_tiles = p.mode == kGemmGrouped ? grouped_total_tiles(p, tiles_n) : tiles_m * tiles_n * shards;
  const int num_kb = (p.K + BK - 1) / BK;
  const int g = cta, G = nctas;  // every CTA computes
  const uint32_t idesc = make_idesc_bf16(BM, BN);
  const int S = ((p.mode == kGemmPlain || p.mode == kGemmAllGather) && p.sk_slices > 1 && p.sk_ws && p.sk_ctr) ? p.sk_slices : 1;
  const int n_items = work_count(g, G, total_tiles, S);

  if (warp >= MOVER_WARP) {
    // ------------------------------------------------------------ all-gather movers
    if (ag) {
      bool go = true;
      if (warp == MOVER_WARP) {
        // the cross-launch guard, by this warp alone: lane t talks to rank t
        if (lane < n && lane != r) {
          __threadfence_system();
          dev::st_release_sys(&p.coll.ctrl[lane]->flags[cta][r], proto.epoch);
          if (!dev::wait_flag_ge(&proto.me->flags[cta][lane], proto.epoch, p.coll.timeout_ns)) {
            dev::report_error(p.coll.status, kDevBarrierTimeout, r, lane, cta, proto.epoch);
            *abort = 1;
            go = false;
          }
        }
        go = __all_sync(0xffffffffu, go);
        if (lane == 0) {
          *(volatile int*)&ctl->mover_go = go ? 1 : -1;
          __threadfence_block();
        }
      } else {
        // the other mover warps start when the first one has passed the guard
        const unsigned long long t0 = dev::globaltimer_ns();
        int st = 0;
        while ((st = *(volatile int*)&ctl->mover_go) == 0 && !*abort && dev::globaltimer_ns() - t0 < p.coll.timeout_ns) {
        }
        go = st == 1;
      }
      const bool by_warps = p.ag_mover == 1 || p.ag_mc;
      if (go && by_warps && warp - MOVER_WARP < p.ag_mover_warps) ag_mover_lsu(p, ctl, cta, nctas, epoch, lane);
      else if (go && warp == MOVER_WARP && lane == 0) ag_mover(p, epi_stage, ctl, cta, nctas, epoch);
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (lane 0 issues;
    // the whole warp polls the ready flags of a remote tile's rows)
    int stage = 0;
    uint32_t phase = 0, issued = 0, issued_phase = 0;
    bool ok = true;
    for (int i = 0; i < n_items && ok; ++i) {
      const Work wk = work_of(i, g, G, total_tiles, S, num_kb);
      Tile tl = tile_of(p, wk.t, tiles_m, tiles_n);
      const bool remote = ag && tl.shard != r;
      if (remote) {
        const int ur = p.ag_unit_rows;
        const int r0 = tl.m_in * TM, r1 = min(r0 + TM, p.rows_per_rank);
        const int u0 = r0 / ur, u1 = (r1 + ur - 1) / ur;
        // Up to eight flags per lane, all loaded before any is looked at (one trip to L2 when the
        // rows are already here, which is the common case); relaxed loads, one fence at the end.
        const uint32_t* fl = &p.fflags[r]->ag_ready[tl.shard][0];
        bool mine = true;
        for (int base = u0; base < u1 && mine; base += 256) {
          unsigned long long t0 = 0;
          for (;;) {
            uint32_t v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int u = base + j * 32 + lane;
              v[j] = u < u1 ? dev::ld_relaxed_sys(fl + u) : epoch;
            }
            bool all = true;
#pragma unroll
            for (int j = 0; j < 8; ++j) all = all && (int32_t)(v[j] - epoch) >= 0;
            if (all) break;
            const unsigned long long now = dev::globaltimer_ns();
            if (t0 == 0) t0 = now;
            if (*abort || now - t0 > p.coll.timeout_ns) {
              dev::report_error(p.coll.status, kDevGemmTimeout, r, tl.shard, base + lane, epoch);
              *abort = 1;
              mine = false;
              break;
            }
          }
        }
        __threadfence_system();  // the relaxed loads that saw the flags + this fence = acquire
        ok = __all_sync(0xffffffffu, mine);
        if (lane == 0) {
          __threadfence_system();  // what the other lanes acquired is ordered before this lane's reads
          fence_proxy_async();     // peers' stores -> my TMA reads
        }
      }
      if (lane == 0 && ok) {
        const CUtensorMap* ma = (ag && !remote) ? map_a_local : map_a;
        int row0 = tl.m_in * TM + ((ag && !remote) ? 0 : tl.shard * p.rows_per_rank);
        int b_row0 = tl.n_blk * BN;
        if (p.mode == kGemmGrouped) {
          row0 = tl.row0;
          b_row0 += tl.shard * p.N;   // group e's matrix starts at row e * N of the stacked B
        }
        for (int kb = wk.kb0; kb < wk.kb1 && ok; ++kb) {
          ok = mbar_wait(&ctl->empty[stage], phase ^ 1u, p.coll.timeout_ns, abort);
          if (!ok) break;
          mbar_expect_tx(&ctl->full[stage], (uint32_t)(a_bytes + BN * BK * 2));
          tma_load_2d(ring + (size_t)stage * stage_bytes, ma, &ctl->full[stage], kb * BK, row0);  // box of TM rows
          tma_load_2d(ring + (size_t)stage * stage_bytes + a_bytes, map_b, &ctl->full[stage], kb * BK, b_row0);
          issued |= 1u << stage;
          issued_phase = (issued_phase & ~(1u << stage)) | (phase << stage);
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (lane == 0 && !ok) {
      // gave up: let the copies already in flight land before the CTA exits
      dev::report_error(p.coll.status, kDevGemmTimeout, r, r, cta, 0xdead0001u);
      for (int s = 0; s < STAGES; ++s) {
        if (!(issued & (1u << s))) continue;
        for (int i = 0; i < 100000 && !mbar_try_wait(&ctl->full[s], (issued_phase >> s) & 1u); ++i) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (; it < n_items && ok; ++it) {
        const Work wk = work_of(it, g, G, total_tiles, S, num_kb);
        // one accumulator per tile and two buffers in turn, or (tall) both used by one tile
        const int buf = MT == 2 ? 0 : (it & 1);
        const uint32_t acc_phase = MT == 2 ? ((uint32_t)it & 1u) : ((uint32_t)(it >> 1) & 1u);
        ok = mbar_wait(&ctl->tempty[buf], acc_phase ^ 1u, p.coll.timeout_ns, abort);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN_MAX);
        for (int kb = wk.kb0; kb < wk.kb1; ++kb) {
          ok = mbar_wait(&ctl->full[stage], phase, p.coll.timeout_ns, abort);
          if (!ok) break;
          tc_fence_after_sync();
          const uint64_t da = make_smem_desc_sw128(ring + (size_t)stage * stage_bytes);
          const uint64_t da2 = make_smem_desc_sw128(ring + (size_t)stage * stage_bytes + A_BYTES);
          const uint64_t db = make_smem_desc_sw128(ring + (size_t)stage * stage_bytes + a_bytes);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // 16 bf16 = 32 bytes further along K inside the 128-byte swizzled row
            const uint32_t acc = (kb > wk.kb0 || kk) ? 1u : 0u;
            tc_mma_f16(d_tmem, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, acc);
            if (MT == 2) tc_mma_f16(d_tmem + (uint32_t)BN_MAX, da2 + (uint64_t)(kk * 2), db + (uint64_t)(kk * 2), idesc, acc);
          }
          tc_commit(&ctl->empty[stage]);  // frees the stage when these MMAs have read it
          if (++stage == n_stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(&ctl->tfull[buf]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (4 warps)
    const int lane_grp = warp % 4;  // TMEM lanes [32 * lane_grp, +32) belong to this warp
    // tall tiles: eight epilogue warps, warps 2-5 drain the first accumulator, 6-9 the second
    const int my_h = MT == 2 ? (warp - 2) / 4 : 0;
    constexpr int EPI_THREADS = 128 * MT;
    int it = 0;
    bool ok = true;
    const bool epi_help = ag && p.ag_epi_help && (p.ag_mover == 1 || p.ag_mc);
    int help_pending = -1;     // unit this warp copied but has not announced yet
    bool help_done = false;    // the CTA's units are all taken
    for (; it < n_items && ok; ++it) {
      const Work wk = work_of(it, g, G, total_tiles, S, num_kb);
      Tile tl = tile_of(p, wk.t, tiles_m, tiles_n);
      const int buf = MT == 2 ? 0 : (it & 1);
      const uint32_t acc_phase = MT == 2 ? ((uint32_t)it & 1u) : ((uint32_t)(it >> 1) & 1u);
      if (epi_help) {
        // No accumulator to drain yet: move units of the shard meanwhile, one at a time, looking at
        // the accumulator's barrier between units (a unit that was copied is announced first).
        for (;;) {
          const bool ready = __shfl_sync(0xffffffffu, mbar_try_wait(&ctl->tfull[buf], acc_phase) ? 1 : 0, 0) != 0;
          if (help_pending >= 0) {
            ag_flag_unit(p, help_pending, epoch, lane);
            help_pending = -1;
          }
          if (ready || help_done || *(volatile int*)&ctl->mover_go != 1) break;
          const int u = ag_take_unit(p, ctl, cta, nctas, lane);
          if (u < 0) {
            help_done = true;
            break;
          }
          ag_copy_unit(p, u, lane);
          help_pending = u;
        }
      }
      ok = mbar_wait(&ctl->tfull[buf], acc_phase, p.coll.timeout_ns, abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (uint32_t)(buf * BN_MAX) + ((uint32_t)(lane_grp * 32) << 16);
      if (p.mode == kGemmReduceScatter && fused) {
        // Partial tile -> the owner's slot number r.  Each 32-column chunk (128 rows x 64 bytes
        // = 8 KB, contiguous at the destination) is staged in shared memory and shipped with
        // ONE bulk store over NVLink; four staging buffers take turns.
        const bool issuer = warp == 2 && lane == 0;
        const size_t tile_elems = (size_t)BM * BN;
        __nv_bfloat16* dst_tile = (__nv_bfloat16*)p.rs_buf[tl.shard] +
                                  (((size_t)r * tiles_m + tl.m_in) * tiles_n + tl.n_blk) * tile_elems;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          char* sbuf = epi_stage + (c & (SIDE_BUFS - 1)) * EPI_CHUNK_BYTES;
          if (issuer) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");  // store c-4 has read sbuf
          asm volatile("bar.sync 1, 128;" ::: "memory");
          uint32_t v[32];
          tmem_ld_32x32(t_row + (uint32_t)(c * 32), v);
          tmem_ld_wait();
          uint4* srow = (uint4*)(sbuf + (size_t)(lane_grp * 32 + lane) * 64);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            alignas(16) __nv_bfloat162 h[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              h[q] = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 2 * q]), __uint_as_float(v[j * 8 + 2 * q + 1]));
            srow[(j + lane) & 3] = *(const uint4*)h;  // rotated so a warp's stores spread over the banks
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (issuer) {
            bulk_s2g(dst_tile + (size_t)c * (BM * 32), sbuf, EPI_CHUNK_BYTES);
            bulk_commit();
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->tempty[buf]);
        if (issuer) {
          bulk_wait_all();  // the whole tile has been written at the owner
          __threadfence_system();
          red_release_sys_add(&p.fflags[tl.shard]->rs_done[r][tl.m_in], 1u);
        }
      } else if (wk.slice >= 0) {
        // Slice of a tail tile: park the fp32 accumulator, meet the tile's other slices, then
        // sum one band of its rows over all slices (in slice order) and store that band.
        // A parked accumulator (one per 128-row half of the tile) is laid out [band][4-column
        // group][row in band, padded to an odd count][4 floats]: a band of one slice is one
        // contiguous piece, fetched with bulk copies into the (now idle) operand ring, so every
        // slice's band is in flight at once; the odd row count keeps the shared-memory reads that
        // follow free of bank conflicts.
        const int j = wk.t - (total_tiles / G) * G;
        const size_t part_elems = SK_SLOT_FLOATS;  // one parked accumulator, padding included
        const int groups = BN / 4;
        const int rows_per = (BM + S - 1) / S, rows_pad = rows_per | 1;
        const size_t band_vecs = (size_t)groups * rows_pad;
        const int row = lane_grp * 32 + lane;
        {
          const int h = my_h;
          float4* mine = (float4*)(p.sk_ws + (((size_t)j * S + wk.slice) * MT + h) * part_elems);
          float4* my_row = mine + (size_t)(row / rows_per) * band_vecs + (row % rows_per);
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(t_row + (uint32_t)(h * BN_MAX + c * 32), v);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 8; ++q)
              my_row[(size_t)(c * 8 + q) * rows_pad] =
                  make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->tempty[buf]);
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        uint32_t* ctr = p.sk_ctr + 2 * j;
        const int r0 = wk.slice * rows_per, r1 = min(BM, r0 + rows_per);
        const uint32_t band_bytes = (uint32_t)(band_vecs * sizeof(float4));
        if (warp == 2 && lane == 0) {
          atomicAdd(ctr, 1u);
          if (*abort || !dev::wait_flag_ge(ctr, (uint32_t)S, p.coll.timeout_ns)) {
            dev::report_error(p.coll.status, kDevGemmTimeout, r, wk.slice, j, 0xdead0003u);
            *abort = 1;
          }
          __threadfence();
        }
        for (int h = 0; h < MT; ++h) {
          asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");  // the ring is free: MMAs done (h = 0), sums of the first half done (h = 1)
          if (warp == 2 && lane == 0 && !*abort && r1 > r0) {
            fence_proxy_async();
            mbar_expect_tx(&ctl->sk_full, band_bytes * (uint32_t)S);
            for (int s2 = 0; s2 < S; ++s2) {
              const char* src = (const char*)(p.sk_ws + (((size_t)j * S + s2) * MT + h) * part_elems + (size_t)wk.slice * band_vecs * 4);
              for (uint32_t o = 0; o < band_bytes; o += COPY_PIECE)
                bulk_g2s(ring + (size_t)s2 * band_bytes + o, src + o, min((uint32_t)COPY_PIECE, band_bytes - o), &ctl->sk_full);
            }
          }
          asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
          if (!*abort && r1 > r0 && mbar_wait(&ctl->sk_full, (uint32_t)h & 1u, p.coll.timeout_ns, abort)) {
            const float4* sm = (const float4*)ring;
            const int total = (r1 - r0) * groups;
            for (int e = my_h * 128 + row; e < total; e += EPI_THREADS) {
              const int rr = e / groups, c4 = e % groups;
              const float4* sp = sm + (size_t)c4 * rows_pad + rr;
              float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int s2 = 0; s2 < S; ++s2) {
                const float4 x = sp[(size_t)s2 * band_vecs];
                acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
              }
              const int grow = tl.m_in * TM + h * BM + r0 + rr, gcol = tl.n_blk * BN + c4 * 4;
              if (grow < p.rows_per_rank && gcol < p.N) {
                alignas(8) __nv_bfloat162 hh[2];
                hh[0] = __floats2bfloat162_rn(acc.x, acc.y);
                hh[1] = __floats2bfloat162_rn(acc.z, acc.w);
                *(uint2*)((__nv_bfloat16*)p.C + ((size_t)tl.shard * p.rows_per_rank + grow) * p.ldc + gcol) = *(const uint2*)hh;
              }
            }
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
        if (warp == 2 && lane == 0) {
          __threadfence();
          if (atomicAdd(ctr + 1, 1u) == (uint32_t)S - 1u) {  // last reader: leave the counters at zero
            ctr[0] = 0;
            ctr[1] = 0;
            __threadfence();
          }
        }
      } else {
        {
          const int h = my_h;
          const bool grouped = p.mode == kGemmGrouped;
          const int row_local = h * BM + lane_grp * 32 + lane;
          const int row_in = tl.m_in * TM + row_local;  // row inside the shard
          const bool row_ok = grouped ? row_local < tl.rows : row_in < p.rows_per_rank;
          __nv_bfloat16* dst_row = (__nv_bfloat16*)p.C + (grouped ? (size_t)(tl.row0 + row_local) : (size_t)tl.shard * p.rows_per_rank + row_in) * p.ldc;
          const bool swiglu = grouped && p.epilogue == kEpiSwiGLU;
          // SwiGLU: chunk c holds 32 gate columns, chunk c + 1 the matching 32 up columns
          auto store_swiglu = [&](const uint32_t* gate, const uint32_t* up, int c) {
            const int col = (tl.n_blk * BN + c * 32) / 2;   // output column of the pair's first element
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (col + j * 8 < p.N / 2) {
                  alignas(16) __nv_bfloat162 h2[4];
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    const float g0 = __uint_as_float(gate[j * 8 + 2 * q]), g1 = __uint_as_float(gate[j * 8 + 2 * q + 1]);
                    const float u0 = __uint_as_float(up[j * 8 + 2 * q]), u1 = __uint_as_float(up[j * 8 + 2 * q + 1]);
                    h2[q] = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                  }
                  *(uint4*)(dst_row + col + j * 8) = *(const uint4*)h2;
                }
              }
            }
          };
          // two register buffers: the TMEM load of the next 32 columns is in flight while the
          // current ones are converted and stored
          auto store_chunk = [&](const uint32_t* v, int c) {
            const int col = tl.n_blk * BN + c * 32;
            if (row_ok) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                if (col + j * 8 < p.N) {
                  alignas(16) __nv_bfloat162 h2[4];
#pragma unroll
                  for (int q = 0; q < 4; ++q)
                    h2[q] = __floats2bfloat162_rn(__uint_as_float(v[j * 8 + 2 * q]), __uint_as_float(v[j * 8 + 2 * q + 1]));
                  *(uint4*)(dst_row + col + j * 8) = *(const uint4*)h2;
                }
              }
            }
          };
          const uint32_t t_half = t_row + (uint32_t)(h * BN_MAX);
          const int nchunks = BN / 32;
          uint32_t va[32], vb[32];
          tmem_ld_32x32(t_half, va);
#pragma unroll 1
          for (int c = 0; c < nchunks; c += 2) {
            tmem_ld_wait();
            if (c + 1 < nchunks) tmem_ld_32x32(t_half + (uint32_t)((c + 1) * 32), vb);
            if (swiglu) {   // the tile width is a multiple of 64 in this mode: chunks come in pairs
              tmem_ld_wait();
              store_swiglu(va, vb, c);
              if (c + 2 < nchunks) tmem_ld_32x32(t_half + (uint32_t)((c + 2) * 32), va);
              continue;
            }
            store_chunk(va, c);
            if (c + 1 < nchunks) {
              tmem_ld_wait();
              if (c + 2 < nchunks) tmem_ld_32x32(t_half + (uint32_t)((c + 2) * 32), va);
              store_chunk(vb, c + 1);
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->tempty[buf]);
      }
    }
    if (epi_help) {
      // out of tiles: announce what is still pending and keep moving until the CTA's units are gone
      if (help_pending >= 0) ag_flag_unit(p, help_pending, epoch, lane);
      if (!*abort && *(volatile int*)&ctl->mover_go == 1) ag_mover_lsu(p, ctl, cta, nctas, epoch, lane);
    }
  }

  __syncthreads();
  if (p.mode == kGemmReduceScatter && fused) rs_reduce(p, ctl, cta, nctas, tiles_m, tiles_n);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0) {
    if (*abort) dev::report_error(p.coll.status, kDevGemmTimeout, r, r, cta, 0xdead0002u);
  }
  // A single-rank launch keeps no protocol state (launches on different streams may overlap).
  if (threadIdx.x == 0 && n > 1) {
    CtrlBlock* me = p.coll.ctrl[r];
    me->epoch[cta] = proto.epoch;
    __threadfence();
    uint32_t ticket = atomicAdd(&me->done_blocks, 1u);
    if (ticket == (uint32_t)nctas - 1) {  // last CTA of this rank: close the operation
      me->done_blocks = 0;
      if (p.mode == kGemmReduceScatter && fused) {
        FusedFlags* f = p.fflags[r];
        for (int s = 0; s < n; ++s)
          for (int m = 0; m < tiles_m; ++m) f->rs_expect[s][m] += (uint32_t)tiles_n;
      }
      me->opseq = proto.opseq + 1u;
      __threadfence();
    }
  }
}

template <int MT>
__global__ void __launch_bounds__(MT == 2 ? kGemmThreadsTall : kGemmThreads, 1)  // TMA warp, MMA warp, 4 * MT epilogue warps, mover warps
gemm_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ CUtensorMap map_a,
            const __grid_constant__ CUtensorMap map_a_local, const __grid_constant__ CUtensorMap map_b) {
  extern __shared__ char smem_raw[];
  gemm_body<MT>(p, &map_a, &map_a_local, &map_b, blockIdx.x, gridDim.x, smem_raw);
}

struct EmuGemmParams {
  GemmLaunch rank[kMaxRanks];
};
template <int MT>
__global__ void __launch_bounds__(MT == 2 ? kGemmThreadsTall : kGemmThreads, 1) gemm_kernel_emu(const __grid_constant__ EmuGemmParams all) {
  extern __shared__ char smem_raw[];
  const GemmLaunch& g = all.rank[blockIdx.y];
  gemm_body<MT>(g.p, &g.map_a, &g.map_a_local, &g.map_b, blockIdx.x, gridDim.x, smem_raw);
}

}  // namespace gemmk

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      p = nullptr;
    }
    return (EncodeTiledFn)p;
  }();
  return fn;
}

Status make_tensor_map_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(kCudaError, "cuTensorMapEncodeTiled is not available in this driver");
  if (((uintptr_t)base & 15) || (ld_elems * 2) % 16) return fail(kInvalidArgument, "TMA needs a 16-byte aligned base and row pitch");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {(cuuint32_t)kGemmBK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kCudaError, "cuTensorMapEncodeTiled failed: %d (rows %llu cols %llu ld %llu)", (int)r,
                                     (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld_elems);
  return kSuccess;
}

size_t gemm_smem_bytes() { return (size_t)kGemmStages * gemmk::STAGE_BYTES + gemmk::SIDE_BUFS * gemmk::EPI_CHUNK_BYTES + sizeof(gemmk::SmemCtl) + 1024 + 64; }

bool gemm_ag_uses_mover_warps(int nranks) {
  const long d = env_long("AMEM_AG_DESIGN", 0);
  return d == 1 ? true : d == 2 ? false : nranks <= 4;
}

int gemm_ag_unit_rows(int rows_per_rank, int K) {
  const int by_flags = (rows_per_rank + kMaxAgUnits - 1) / kMaxAgUnits;      // at most kMaxAgUnits flags per source
  const int by_piece = (kAgPieceBytes + K * 2 - 1) / (K * 2);                // a unit is at least one piece of the mover
  return std::max(1, std::max(by_flags, by_piece));
}

static double splitk_fixup_blocks() {
  const long v = env_long("AMEM_GEMM_SPLITK_COST", 24);  // in K blocks of main loop (measured: 20-35)
  return (double)v;
}

int gemm_tail_slices(long tiles, int ctas, int k_blocks) {
  long rem = tiles % ctas;
  if (rem == 0 || k_blocks <= 0) return 1;
  long s = std::min<long>(ctas / rem, k_blocks / 8);
  if (s > gemmk::SK_MAX_SLICES) s = gemmk::SK_MAX_SLICES;
  if (s < 2) return 1;
  // the fix-up (park the accumulator, wait, re-read a band of every slice) costs about as much
  // as two dozen K blocks of main loop; split only when the shortened wave plus that clearly
  // wins (with two or three slices it measured no better than the unsplit wave)
  double tail = 1.0 / (double)s + splitk_fixup_blocks() / (double)k_blocks;
  return tail < 0.75 ? (int)s : 1;
}

size_t gemm_splitk_ws_bytes(int ctas) { return (size_t)ctas * 2 * gemmk::SK_SLOT_FLOATS * sizeof(float); }  // two halves of a tall tile
size_t gemm_splitk_ctr_words(int ctas) { return (size_t)2 * ctas; }

int gemm_pick_bn(int row_tiles, int N, int ctas, int k_blocks, int* slices) {
  int best = kGemmBN, best_s = 1;
  double best_cost = -1;
  for (int bn = kGemmBN; bn >= 128; bn -= 32) {
    long tiles = (long)row_tiles * ((N + bn - 1) / bn);
    long full = tiles / ctas, rem = tiles % ctas;
    int s = gemm_tail_slices(tiles, ctas, k_blocks);
    double tail = rem == 0 ? 0.0 : (s > 1 ? 1.0 / s + splitk_fixup_blocks() / k_blocks : 1.0);
    // measured: a tile's time depends only weakly on its width (the main loop is bound by
    // filling shared memory, not by the tensor pipe), so count waves first, width second
    double cost = ((double)full + tail) * (bn + 600);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
      best_s = s;
    }
  }
  if (slices) *slices = best_s;
  return best;
}

// Cost of a tiling in units of "one K block of a 128-row tile's main loop": waves x (K blocks
// + exposed epilogue), with the partly filled last wave priced as in gemm_pick_bn.
static double tiling_cost(int row_tiles, int N, int bn, int slices, int k_blocks, int ctas, double per_block, double epilogue) {
  long tiles = (long)row_tiles * ((N + bn - 1) / bn);
  long full = tiles / ctas, rem = tiles % ctas;
  double tail = rem == 0 ? 0.0 : (slices > 1 ? 1.0 / slices + splitk_fixup_blocks() / k_blocks : 1.0);
  return ((double)full + tail) * ((double)k_blocks * per_block + epilogue);
}

bool gemm_tall_pays(int M, int N, int k_blocks, int ctas, int bn_flat, int slices_flat, int bn_tall, int slices_tall) {
  // measured (8192^3 and 4096^3, both forms in one run): a tall tile does twice the work per K
  // block in about 1.65x the time of a flat one (its main loop is bound by the tensor pipe, the
  // flat one by filling shared memory) and exposes an epilogue worth about 17 flat K blocks
  const double flat = tiling_cost((M + kGemmBM - 1) / kGemmBM, N, bn_flat, slices_flat, k_blocks, ctas, 1.0, 0.0);
  const double tall = tiling_cost((M + 2 * kGemmBM - 1) / (2 * kGemmBM), N, bn_tall, slices_tall, k_blocks, ctas, 1.65, 17.0);
  return tall < flat;
}

int gemm_default_grid(int device) {
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  return sms > 0 ? sms : 148;
}

static Status prepare_kernel(const void* fn) {
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_smem_bytes());
  if (e != cudaSuccess) return fail(kCudaError, "cudaFuncSetAttribute(%zu bytes of shared memory): %s", gemm_smem_bytes(), cudaGetErrorString(e));
  return kSuccess;
}

Status launch_gemm(const GemmLaunch& g, cudaStream_t stream) {
  static Status ready = prepare_kernel((const void*)gemmk::gemm_kernel<1>);
  static Status ready_tall = prepare_kernel((const void*)gemmk::gemm_kernel<2>);
  const bool tall = (g.p.mode == kGemmPlain || g.p.mode == kGemmAllGather) && g.p.tall;
  if ((tall ? ready_tall : ready) != kSuccess) return tall ? ready_tall : ready;
  if (tall) gemmk::gemm_kernel<2><<<g.grid, kGemmThreadsTall, gemm_smem_bytes(), stream>>>(g.p, g.map_a, g.map_a_local, g.map_b);
  else gemmk::gemm_kernel<1><<<g.grid, kGemmThreads, gemm_smem_bytes(), stream>>>(g.p, g.map_a, g.map_a_local, g.map_b);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kCudaError, "gemm launch failed: %s", cudaGetErrorString(e));
  return kSuccess;
}

Status launch_gemm_emu(const GemmLaunch* ranks, int nranks, cudaStream_t stream) {
  static Status ready = prepare_kernel((const void*)gemmk::gemm_kernel_emu<1>);
  static Status ready_tall = prepare_kernel((const void*)gemmk::gemm_kernel_emu<2>);
  const bool tall = ranks[0].p.mode == kGemmAllGather && ranks[0].p.tall;
  if ((tall ? ready_tall : ready) != kSuccess) return tall ? ready_tall : ready;
  static gemmk::EmuGemmParams all;  // launches are serialised by the emulation rendez-vous
  for (int r = 0; r < nranks; ++r) all.rank[r] = ranks[r];
  void* params[] = {(void*)&all};
  dim3 grid(ranks[0].grid, nranks), block(tall ? kGemmThreadsTall : kGemmThreads);
  const void* fn = tall ? (const void*)gemmk::gemm_kernel_emu<2> : (const void*)gemmk::gemm_kernel_emu<1>;
  cudaError_t e = cudaLaunchCooperativeKernel(fn, grid, block, params, gemm_smem_bytes(), stream);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(kCudaError, "emulated gemm cooperative launch (%d x %d CTAs) failed: %s", ranks[0].grid, nranks, cudaGetErrorString(e));
  }
  return kSuccess;
}

}  // namespace amem
