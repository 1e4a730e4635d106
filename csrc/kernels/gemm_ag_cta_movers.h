// All-gather -> GEMM with DEDICATED MOVER CTAs: the schedule used from five ranks up, where the
// transfer takes about as long as the GEMM and movers that share an SM with the main loop fall
// behind it (measured on 8 GPUs: 0.476 ms with 16 mover CTAs against 0.543 ms with mover warps in
// every CTA; on 4 GPUs the mover-warp form of gemm_sm100.cu is the faster one).  Same tcgen05 /
// TMEM / TMA tile pipeline as gemm_sm100.cu, kept as a translation unit of its own with its own
// parameter block and flag layout (namespace amem::agcta); only its all-gather mode is called.
// Host-visible description of the tcgen05 GEMM kernels (plain, all-gather -> GEMM,
// GEMM -> reduce-scatter).  C[M,N] = A[M,K] * B[N,K]^T, bf16 operands (both K-major, i.e. the
// layout of activations [tokens, features] and of torch Linear weights [out, in]), fp32
// accumulation in tensor memory, bf16 output.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "../core/status.h"
#include "coll_args.h"

namespace amem {
namespace agcta {

static const int kGemmBM = 128, kGemmBN = 256, kGemmBK = 64, kGemmStages = 4;
static const int kGemmThreads = 192;       // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue
static const int kAgUnitRows = 32;         // rows of A announced by one all-gather ready flag
static const int kMaxUnits = 256;          // flag slots per source rank

// kGemmGrouped: A [rows, K] holds `groups` runs of rows, run e = [group_off[e], group_off[e+1]) with
// group_off in DEVICE memory (the MoE dispatch produces it there, nothing comes back to the host);
// B stacks one [N, K] matrix per group as [groups * N, K]; C has A's rows.  Row tiles start at the
// group's first row, whatever its alignment (TMA has no alignment rule on the row coordinate), and
// the rows a tile has beyond its group are computed and not stored.
enum GemmMode : int { kGemmPlain = 0, kGemmAllGather = 1, kGemmReduceScatter = 2, kGemmGrouped = 3 };
// Epilogue of the grouped mode: plain store, or SwiGLU of column pairs — B's rows are then laid out
// in alternating blocks of 32 gate rows and 32 up rows, the output has N / 2 columns and
// out[:, 32 j + i] = silu(acc[:, 64 j + i]) * acc[:, 64 j + 32 + i].
enum GemmEpilogue : int { kEpiStore = 0, kEpiSwiGLU = 1 };

// Flags of the fused kernels; lives in every rank's control segment right after CtrlBlock,
// so it is saved and restored by pause/resume like the rest of the protocol state.
struct FusedFlags {
  uint32_t ag_ready[kMaxRanks][kMaxUnits];   // written by source rank s: unit u of its shard has landed (value = epoch)
  uint32_t rs_done[kMaxRanks][kMaxUnits];    // incremented by source rank s: partial tiles of row block u delivered
  uint32_t rs_expect[kMaxRanks][kMaxUnits];  // my running total of deliveries to expect per (source, row block)
};

struct GemmParams {
  int M, N, K;              // problem of this rank (M = all rows, gathered or to be scattered)
  int bn;                   // tile width in columns: multiple of 32, <= kGemmBN (see gemm_pick_bn)
  int tall;                 // plain mode: 1 = tiles of 256 rows (two accumulators side by side in TMEM, one B tile
                            // feeds both: a third less shared-memory fill per FLOP; the epilogue is then not overlapped)
  int mode;
  void* C;                  // plain / all-gather: bf16 [M, N] row-major, leading dimension ldc
  int ldc;
  int rows_per_rank;        // M / nranks (M when nranks == 1)
  int comm_ctas;            // all-gather: CTAs [0, comm_ctas) move data, the rest compute
  int copy_own;             // all-gather: also place my own shard in the gathered buffer
  const void* a_local;      // all-gather: my shard, bf16 [rows_per_rank, K]
  void* ag_buf[kMaxRanks];  // all-gather: every rank's gathered-A buffer [M, K]; [rank] is mine
  void* rs_buf[kMaxRanks];  // reduce-scatter: every rank's partial buffer, tile-major [nranks][row blocks][col blocks][128 x 256]
  void* rs_out;             // reduce-scatter: bf16 [rows_per_rank, N]
  FusedFlags* fflags[kMaxRanks];
  const int* group_off;     // grouped: device array of groups + 1 row offsets
  int groups;               // grouped: number of groups (<= 256)
  int epilogue;             // grouped: GemmEpilogue
  // Split-K of the last, partly filled wave of tiles (plain mode): each of its tiles is cut in
  // sk_slices ranges of K that run on different CTAs; partial accumulators meet in sk_ws
  // (fp32, [tile][slice][32-column chunk][128 rows][32]) and are summed in slice order.
  int sk_slices;            // 0 or 1: off
  float* sk_ws;
  uint32_t* sk_ctr;         // two counters per tail tile (arrived, finished), zero between launches
  CollArgs coll;            // rank, nranks, control blocks, status words, timeout
};

struct GemmLaunch {
  GemmParams p;
  CUtensorMap map_a;        // plain/RS: A [M, K]; all-gather: the gathered buffer [M, K]
  CUtensorMap map_a_local;  // all-gather: my own shard [rows_per_rank, K]
  CUtensorMap map_b;        // B [N, K]
  int grid;                 // CTAs (per rank)
};

// Encodes a 2-D bf16 row-major tensor map with a [box_rows, 64] box and the 128-byte swizzle.
Status make_tensor_map_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld_elems, uint32_t box_rows);

size_t gemm_smem_bytes();
Status launch_gemm(const GemmLaunch& g, cudaStream_t stream);
// All ranks of an emulated communicator in one cooperative grid (blockIdx.y = rank).
Status launch_gemm_emu(const GemmLaunch* ranks, int nranks, cudaStream_t stream);
int gemm_default_grid(int device);
// Tile width that minimises (waves of tiles) x (tile width) for `ctas` compute CTAs.  With
// `k_blocks` > 0 the last wave may be split along K (see GemmParams::sk_slices): its cost is
// then 1/slices of a wave plus the fix-up, and *slices receives the split to use (1 = none).
int gemm_pick_bn(int row_tiles, int N, int ctas, int k_blocks = 0, int* slices = nullptr);
// Whether 256-row tiles (GemmParams::tall) are expected to beat 128-row tiles for this problem.
bool gemm_tall_pays(int M, int N, int k_blocks, int ctas, int bn_flat, int slices_flat, int bn_tall, int slices_tall);
// Slices of the tail split for a given tiling, 1 when splitting does not pay.
int gemm_tail_slices(long tiles, int ctas, int k_blocks);
// Bytes of split-K workspace / number of counters that a launch on `ctas` CTAs may touch.
size_t gemm_splitk_ws_bytes(int ctas);
size_t gemm_splitk_ctr_words(int ctas);

}  // namespace agcta
}  // namespace amem
