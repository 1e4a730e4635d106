// Structures shared by the host launcher, the CUDA kernels and the host (mock) executor.
//
// Protocol in one paragraph.  Every rank owns a control segment (CtrlBlock, STATEFUL: it is
// saved and restored by pause/resume) and a staging segment (SCRATCH: dropped on pause),
// both mapped by every peer.  Collectives are "push" style: a rank stores its contribution
// straight into the consumer's staging slot over NVLink, block b then raises flag
// flags[b][my_rank] in the consumer's CtrlBlock to the block's current epoch and waits for
// the same flag from every peer in its own CtrlBlock.  Epoch counters live on the device
// (CtrlBlock::epoch[b]), so a captured CUDA graph replays correctly and nothing but the
// control segment has to survive a pause.  Staging is split in two halves used by
// alternate operations (CtrlBlock::opseq parity) and each half in two quarters used by
// alternate chunks, which removes every trailing barrier.  All waits are bounded: on expiry
// the block records {code, rank, peer, block, epoch} in a host-mapped status word and the
// kernel runs to completion without faulting.
// Reference parity: the reference has no device code of its own (amem_nccl_plugin/Makefile:36); its
// collectives are NCCL 2.27.5's kernels, whose buffers it re-creates on resume.
#pragma once
#include <cstddef>
#include <cstdint>

namespace amem {

static const int kMaxRanks = 8;        // one NVLink/NVSwitch domain
static const int kMaxBlocks = 512;     // flag rows available to one launch
static const int kP2PBlocks = 32;      // blocks of a send/recv launch, per peer
static const int kStatusWords = 16;
static const int kLLBlocks = 8;        // blocks of a flag-in-data (small message) launch

// Collective kinds (values are part of the host<->kernel contract only).
enum CollKind : int {
  kCollAllReduce = 0,
  kCollAllGather = 1,
  kCollReduceScatter = 2,
  kCollBroadcast = 3,
  kCollReduce = 4,
  kCollAllToAll = 5,
  kCollSendRecv = 6,
};

// Allreduce variants chosen by the tuner.
// kAlgoWindow: both buffers lie in registered windows, the all-reduce works on them in place
// (through the windows' multicast mapping when there is one, by peer loads and stores otherwise).
// kAlgoLL: small messages travel as 8-byte packets {4 bytes of data, 4-byte flag}; the receiver polls
// the packets themselves, so there is no barrier and no fence between the data and its signal.
enum Algo : int { kAlgoAuto = 0, kAlgoOneShot = 1, kAlgoTwoShot = 2, kAlgoNvls = 3, kAlgoWindow = 4, kAlgoLL = 5 };

// ncclDataType_t / ncclRedOp_t numbering.
// 8-bit floats are carried by the copy collectives (all-gather, all-to-all, broadcast, send/recv);
// reductions on them are refused (NCCL numbering: ncclFloat8e4m3 = 10, ncclFloat8e5m2 = 11).
enum DType : int { kI8 = 0, kU8 = 1, kI32 = 2, kU32 = 3, kI64 = 4, kU64 = 5, kF16 = 6, kF32 = 7, kF64 = 8, kBF16 = 9, kF8E4M3 = 10, kF8E5M2 = 11 };
enum RedOp : int { kSum = 0, kProd = 1, kMax = 2, kMin = 3, kAvg = 4 };

inline size_t dtype_size(int dt) {
  switch (dt) {
    case kI8: case kU8: case kF8E4M3: case kF8E5M2: return 1;
    case kF16: case kBF16: return 2;
    case kI32: case kU32: case kF32: return 4;
    case kI64: case kU64: case kF64: return 8;
    default: return 0;
  }
}

struct alignas(128) CtrlBlock {
  uint32_t opseq;                       // operations completed on this communicator (device side)
  uint32_t done_blocks;                 // ticket counter used to bump opseq once per launch
  uint32_t reserved[30];
  uint32_t epoch[kMaxBlocks];           // my barrier epoch, per block index
  uint32_t flags[kMaxBlocks][kMaxRanks];          // written by peers: flags[block][source rank]
  // point-to-point credit protocol, indexed [peer][block]
  uint32_t p2p_ready[kMaxRanks][kP2PBlocks];      // written by the sender: chunk sequence available
  uint32_t p2p_taken[kMaxRanks][kP2PBlocks];      // written by the receiver: chunk sequence consumed
  uint32_t p2p_sent[kMaxRanks][kP2PBlocks];       // my local count of chunks sent to peer
  uint32_t p2p_rcvd[kMaxRanks][kP2PBlocks];       // my local count of chunks received from peer
  // small all-to-all scratch for counts (MoE routing): xchg[source rank][i]
  uint32_t xchg[kMaxRanks][256];
  // chunk credits of the pipelined collectives, per block: cseq = chunks this block has moved so
  // far (mine); ready[b][s] = written by rank s: its chunk number N has landed in my staging;
  // freed[b][s] = written by rank s: it has drained my chunk number N from its staging
  uint32_t cseq[kMaxBlocks];
  uint32_t ready[kMaxBlocks][kMaxRanks];
  uint32_t freed[kMaxBlocks][kMaxRanks];
  // flag-in-data protocol, per block: ll_seq = such operations this block has done (mine, also the
  // flag value of the next one); ll_ack[b][s] = written by rank s: it has consumed my operation N.
  // A slot is rewritten two operations later, after the receiver's ack for the earlier one.
  uint32_t ll_seq[kLLBlocks];
  uint32_t ll_ack[kLLBlocks][kMaxRanks];
};

enum DeviceError : uint32_t { kDevOk = 0, kDevBarrierTimeout = 1, kDevP2PTimeout = 2, kDevBadArgs = 3, kDevGemmTimeout = 4 };

struct CollArgs {
  int kind, algo;
  int rank, nranks;
  int dtype, redop;
  int out_dtype;           // differs from dtype only for the fused scale+cast reduce-scatter
  int root;
  const void* send;
  void* recv;
  size_t count;            // elements: allreduce/bcast/reduce total; allgather/reducescatter/alltoall per rank
  float scale;             // multiplies the reduced value (1/n for avg, user scale for fused RS)
  int has_scale;
  CtrlBlock* ctrl[kMaxRanks];   // ctrl[rank] is mine, others are peers' blocks mapped here
  char* stage[kMaxRanks];       // staging segments, same indexing
  char* mc_stage;               // multicast mapping of the staging segments (NVLS) or null
  size_t stage_bytes;           // bytes of one staging segment
  size_t p2p_slot_bytes;        // bytes of one (peer, block) slot in the p2p area at the end of staging
  // registered windows (algo == kAlgoWindow): the operands as every rank maps them, already
  // offset to the first element, and their multicast views (null without NVLS)
  const char* win_send[kMaxRanks];
  char* win_recv[kMaxRanks];
  const char* mc_send;
  char* mc_recv;
  uint32_t* status;             // host-mapped, kStatusWords words
  unsigned long long timeout_ns;
  // send/recv lists for grouped point-to-point (kind == kCollSendRecv)
  int n_p2p;
  int p2p_max_lanes;       // blocks one transfer may use (<= kP2PBlocks; small on emulated comms)
  int nvls_split;          // sixteenths of a block's warps on the switch job of the pipelined NVLS all-reduce (0 = 4)
  struct P2P {
    int peer;
    int is_send;
    const void* src;
    void* dst;
    size_t bytes;
  } p2p[2 * kMaxRanks];
};

// Plan computed identically on every rank from (kind, bytes, nranks).
struct LaunchPlan {
  int algo;
  int blocks;
  int threads;
  size_t chunk_elems;   // elements of the per-chunk unit (meaning depends on kind)
};

// ---- staging layout, computed the same way on host and device --------------------------
// [ half 0 | half 1 | p2p area ]; a half is two quarters.
#if defined(__CUDACC__)
#define AMEM_HD __host__ __device__ inline
#else
#define AMEM_HD inline
#endif
// [ half 0 | half 1 | p2p slots | flag-in-data slots ]: the last two form the reserved tail.
// A flag-in-data slot holds one source rank's packets of one operation (two parities alternate):
// twice the bytes of a p2p slot, i.e. p2p_slot_bytes of payload per peer.
AMEM_HD size_t ll_slot_bytes(size_t p2p_slot_bytes) { return 2 * p2p_slot_bytes; }
AMEM_HD size_t ll_area_bytes(size_t p2p_slot_bytes) { return (size_t)kMaxRanks * 2 * ll_slot_bytes(p2p_slot_bytes); }
AMEM_HD size_t p2p_area_bytes(size_t p2p_slot_bytes) { return (size_t)kMaxRanks * 2 * kP2PBlocks * p2p_slot_bytes + ll_area_bytes(p2p_slot_bytes); }
AMEM_HD size_t ll_slot_offset(size_t stage_bytes, size_t p2p_slot_bytes, int src, uint32_t parity) {
  return stage_bytes - ll_area_bytes(p2p_slot_bytes) + (size_t)(src * 2 + (int)(parity & 1u)) * ll_slot_bytes(p2p_slot_bytes);
}
AMEM_HD size_t quarter_bytes(size_t stage_bytes, size_t p2p_slot_bytes) {
  size_t q = (stage_bytes - p2p_area_bytes(p2p_slot_bytes)) / 4;
  return q & ~(size_t)4095;
}
AMEM_HD size_t quarter_offset(size_t stage_bytes, size_t p2p_slot_bytes, uint32_t opseq, uint32_t chunk) {
  return (size_t)((opseq & 1u) * 2u + (chunk & 1u)) * quarter_bytes(stage_bytes, p2p_slot_bytes);
}
AMEM_HD size_t half_offset(size_t stage_bytes, size_t p2p_slot_bytes, uint32_t opseq) {
  return (size_t)(opseq & 1u) * 2u * quarter_bytes(stage_bytes, p2p_slot_bytes);
}
AMEM_HD size_t p2p_slot_offset(size_t stage_bytes, size_t p2p_slot_bytes, int src, uint32_t parity, int block) {
  return stage_bytes - p2p_area_bytes(p2p_slot_bytes) + ((size_t)(src * 2 + (int)(parity & 1u)) * kP2PBlocks + block) * p2p_slot_bytes;
}
// Bytes one rank may put in its slot of a quarter (or of half a half, for two-shot).
AMEM_HD size_t slot_bytes_of(size_t region_bytes, int nranks) { return (region_bytes / nranks) & ~(size_t)255; }

// Blocks ("lanes") that carry one point-to-point transfer; depends only on its size, so both
// ends agree.
AMEM_HD int p2p_lanes(size_t bytes, size_t slot_bytes, int max_lanes) {
  size_t l = (bytes + slot_bytes - 1) / slot_bytes;
  return l < 1 ? 1 : (l > (size_t)max_lanes ? max_lanes : (int)l);
}

// Host executor for the mock backend (same protocol, runs on the calling thread).
int host_run_collective(const CollArgs& a, const LaunchPlan& plan);

}  // namespace amem
