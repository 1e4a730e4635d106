/* NCCL-compatible C API of the B200-native pausable collective library.
 *
 * Function names, argument order, enum values and the 128-byte ncclUniqueId follow NCCL 2.27 so
 * that code written against nccl.h (including ctypes loaders that look symbols up by name)
 * works unchanged.  On top of that come the five AMem entry points the reference adds to
 * nccl.h (nccl_patch/nccl_2.27.5-1.diff:329-355) -- ncclPause, ncclResume, ncclMemStats,
 * ncclSetGroupID, ncclGetGroupID -- and a small set of amem* extensions for the fused
 * operations and for observability.
 */
#ifndef AMEM_B200_NCCL_H_
#define AMEM_B200_NCCL_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NCCL_MAJOR 2
#define NCCL_MINOR 27
#define NCCL_PATCH 5
#define NCCL_SUFFIX "+amem.b200"
#define NCCL_VERSION_CODE 22705
#define NCCL_VERSION(X, Y, Z) (((X) <= 2 && (Y) <= 8) ? (X) * 1000 + (Y) * 100 + (Z) : (X) * 10000 + (Y) * 100 + (Z))

typedef struct CUstream_st* cudaStream_t;
typedef struct ncclComm* ncclComm_t;
typedef struct ncclWindow* ncclWindow_t;
#define NCCL_COMM_NULL NULL

#define NCCL_UNIQUE_ID_BYTES 128
typedef struct { char internal[NCCL_UNIQUE_ID_BYTES]; } ncclUniqueId;

typedef enum {
  ncclSuccess = 0,
  ncclUnhandledCudaError = 1,
  ncclSystemError = 2,
  ncclInternalError = 3,
  ncclInvalidArgument = 4,
  ncclInvalidUsage = 5,
  ncclRemoteError = 6,
  ncclInProgress = 7,
  ncclNumResults = 8
} ncclResult_t;

#define NCCL_CONFIG_UNDEF_INT INT32_MIN
#define NCCL_CONFIG_UNDEF_PTR NULL
#define NCCL_SPLIT_NOCOLOR -1

typedef struct ncclConfig_v22700 {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int blocking;
  int cgaClusterSize;
  int minCTAs;
  int maxCTAs;
  const char* netName;
  int splitShare;
  int trafficClass;
  const char* commName;
  int collnetEnable;
  int CTAPolicy;
  int shrinkShare;
  int nvlsCTAs;
} ncclConfig_t;

#define NCCL_CONFIG_INITIALIZER {                                   \
  sizeof(ncclConfig_t), 0xcafebeef, NCCL_VERSION_CODE,              \
  NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, \
  NCCL_CONFIG_UNDEF_PTR, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_PTR, \
  NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT, NCCL_CONFIG_UNDEF_INT }

typedef enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3, ncclAvg = 4, ncclNumOps = 5, ncclMaxRedOp = 0x7fffffff } ncclRedOp_t;

typedef enum {
  ncclInt8 = 0, ncclChar = 0,
  ncclUint8 = 1,
  ncclInt32 = 2, ncclInt = 2,
  ncclUint32 = 3,
  ncclInt64 = 4,
  ncclUint64 = 5,
  ncclFloat16 = 6, ncclHalf = 6,
  ncclFloat32 = 7, ncclFloat = 7,
  ncclFloat64 = 8, ncclDouble = 8,
  ncclBfloat16 = 9,
  ncclFloat8e4m3 = 10, /* copy collectives only: all-gather, all-to-all, broadcast, send/recv */
  ncclFloat8e5m2 = 11,
  ncclNumTypes = 12
} ncclDataType_t;

/* ---- memory ------------------------------------------------------------------------- */
/* VMM allocation on the current device, tracked by the registry and therefore pausable:
 * its contents are saved on ncclPause and restored at the same address on ncclResume. */
ncclResult_t ncclMemAlloc(void** ptr, size_t size);
ncclResult_t ncclMemFree(void* ptr);

/* ---- communicator ------------------------------------------------------------------- */
ncclResult_t ncclGetVersion(int* version);
ncclResult_t ncclGetUniqueId(ncclUniqueId* uniqueId);
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank);
ncclResult_t ncclCommInitRankConfig(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank, ncclConfig_t* config);
ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist);
ncclResult_t ncclCommFinalize(ncclComm_t comm);
ncclResult_t ncclCommDestroy(ncclComm_t comm);
ncclResult_t ncclCommAbort(ncclComm_t comm);
ncclResult_t ncclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm, ncclConfig_t* config);
const char* ncclGetErrorString(ncclResult_t result);
const char* ncclGetLastError(ncclComm_t comm);
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError);
ncclResult_t ncclCommCount(const ncclComm_t comm, int* count);
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device);
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank);
/* Buffer registration is accepted for source compatibility; the push protocol needs none. */
ncclResult_t ncclCommRegister(const ncclComm_t comm, void* buff, size_t size, void** handle);
ncclResult_t ncclCommDeregister(const ncclComm_t comm, void* handle);
ncclResult_t ncclCommWindowRegister(ncclComm_t comm, void* buff, size_t size, ncclWindow_t* win, int winFlags);
ncclResult_t ncclCommWindowDeregister(ncclComm_t comm, ncclWindow_t win);
/* Several unique ids may be passed for source compatibility; the first one is the meeting point. */
ncclResult_t ncclCommInitRankScalable(ncclComm_t* newcomm, int nranks, int myrank, int nId, ncclUniqueId* commIds, ncclConfig_t* config);
/* Not supported (returns ncclInvalidUsage): a communicator cannot lose ranks; create a new one. */
ncclResult_t ncclCommShrink(ncclComm_t comm, int* excludeRanksList, int excludeRanksCount, ncclComm_t* newcomm, ncclConfig_t* config, int shrinkFlags);

/* Pre-multiplied sum: sum_r (scalar * x_r).  The scalar is read when the operator is created. */
typedef enum { ncclScalarDevice = 0, ncclScalarHostImmediate = 1 } ncclScalarResidence_t;
ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype, ncclScalarResidence_t residence, ncclComm_t comm);
ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm);

/* ---- collectives -------------------------------------------------------------------- */
ncclResult_t ncclReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, int root, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclBroadcast(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
/* count = elements exchanged with EACH peer; block j of sendbuff goes to rank j. */
ncclResult_t ncclAlltoAll(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclSend(const void* sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclRecv(void* recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm, cudaStream_t stream);
ncclResult_t ncclGroupStart(void);
ncclResult_t ncclGroupEnd(void);

/* Filled by ncclGroupSimulateEnd: the group is closed without being launched and its duration
 * (microseconds) is estimated. */
typedef struct ncclSimInfo_v22200 {
  size_t size;
  unsigned int magic;
  unsigned int version;
  float estimatedTime;
} ncclSimInfo_t;
#define NCCL_UNDEF_FLOAT -1.0f
#define NCCL_SIM_INFO_INITIALIZER { sizeof(ncclSimInfo_t), 0x74685283, NCCL_VERSION_CODE, NCCL_UNDEF_FLOAT }
ncclResult_t ncclGroupSimulateEnd(ncclSimInfo_t* simInfo);
/* Re-reads the logging environment (GMM_LOG). */
void ncclResetDebugInit(void);

/* ---- AMem: pause / resume ------------------------------------------------------------ */
/* comm == NULL (or *comm == NULL): every communicator of the process plus ncclMemAlloc
 * memory.  Otherwise only that communicator.  Synchronous; every rank of the communicator
 * must call; idempotent.  After ncclPause returns, the physical memory behind the
 * communicator (this rank's and its mappings of the peers') has been returned to the driver
 * while all virtual addresses stay reserved.  Collectives issued while paused fail with
 * ncclInvalidUsage. */
ncclResult_t ncclPause(ncclComm_t* comm);
ncclResult_t ncclResume(ncclComm_t* comm);
ncclResult_t ncclMemStats(void);
/* Only before the first tracked allocation of the process; distinguishes co-located groups
 * (for instance training = 100, inference = 200). */
ncclResult_t ncclSetGroupID(int id);
ncclResult_t ncclGetGroupID(int* id);

/* ---- amem extensions ------------------------------------------------------------------ */
typedef struct {
  uint64_t bytes_by_tag[16];
  uint64_t stateful_bytes, scratch_bytes, imported_bytes, multicast_bytes;
  uint64_t live_bytes, paused_bytes, shadow_bytes;
  uint64_t n_local, n_imported;
  uint64_t pause_count, resume_count;
  int group_id;
  int paused;
} amemMemStats_t;

typedef struct {
  double quiesce_us, offload_us, release_import_us, release_local_us, pause_barrier_us, pause_total_us;
  double create_map_us, agree_us, exchange_us, import_us, preload_us, resume_barrier_us, resume_total_us;
  uint64_t bytes_offloaded, bytes_preloaded;
  uint64_t bytes_released_local, bytes_released_peer;
  uint64_t n_offload, n_release_local, n_release_peer;
  uint64_t free_before_pause, free_after_pause, free_after_resume;
} amemPauseResumeStats_t;

ncclResult_t amemMemStatsGet(amemMemStats_t* out);
/* Phase timings and byte counts of the most recent pause and resume (comm NULL: process). */
ncclResult_t amemPauseResumeStatsGet(ncclComm_t comm, amemPauseResumeStats_t* out);

/* Reduce-scatter fused with a scale and an output type cast: recv[i] = (out_type)(scale *
 * sum_r send_r[rank*recvcount + i]).  fp32 <-> bf16/fp16 and same-type are supported. */
ncclResult_t amemReduceScatterScaleCast(const void* sendbuff, void* recvbuff, size_t recvcount, ncclDataType_t in_type,
                                        ncclDataType_t out_type, float scale, ncclComm_t comm, cudaStream_t stream);
/* All-reduce with a forced variant: 1 one-shot, 2 two-shot, 3 NVLS (0 lets the tuner pick). */
ncclResult_t amemAllReduceAlgo(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                               int algo, ncclComm_t comm, cudaStream_t stream);
/* tcgen05 GEMM, bf16 in / fp32 accumulate / bf16 out: C[M,N] = A[M,K] * B[N,K]^T (both operands
 * row-major with K contiguous, the layout of activations and of Linear weights).  N and K must
 * be multiples of 8. */
ncclResult_t amemGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, cudaStream_t stream);
/* The tiling amemGemmBf16 picks for a problem on a GPU with `sms` SMs: tile rows (128 or 256), tile
 * columns, K-slices of the last wave (1 = not split).  Host arithmetic only; outputs may be NULL. */
/* Variant (1 one-shot, 2 two-shot, 3 NVLS, 0 n/a), grid and chunk the library picks for a collective
 * (kind: 0 all-reduce, 1 all-gather, 2 reduce-scatter, 3 broadcast, 4 reduce, 5 all-to-all) on `nranks`
 * GPUs; stage_bytes 0 = default staging.  Host arithmetic only. */
ncclResult_t amemTunerPlan(int kind, size_t count, ncclDataType_t dtype, int nranks, int nvls, size_t stage_bytes, int* algo,
                           int* blocks, size_t* chunk_elems);
/* Debug guard behind the staging layout (AMEM_CANARY=1): ncclInternalError if a kernel wrote past it. */
/* Variable-size all-to-all; counts and displacements in elements, MPI_Alltoallv convention. */
ncclResult_t amemAlltoAllv(const void* sendbuff, const size_t* sendcounts, const size_t* sdispls, void* recvbuff,
                           const size_t* recvcounts, const size_t* rdispls, ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);
ncclResult_t amemCheckCanary(ncclComm_t comm);
ncclResult_t amemDebugDirtyCanary(ncclComm_t comm); /* test hook: dirties the guard */
/* Grouped GEMM (one launch for all experts of a rank): for every group e,
 * C[group_off[e] .. group_off[e+1], :] = A[same rows, :] * B[e]^T.  group_off is a DEVICE array of
 * groups + 1 int32 row offsets (amemMoeDispatch's expert_offsets), B is bf16 [groups, N, K].
 * epilogue 0: C is bf16 [rows_cap, N]; epilogue 1 (SwiGLU): B[e]'s rows alternate in blocks of 32
 * gate rows and 32 up rows and C is bf16 [rows_cap, N / 2] = silu(gate) * up. */
ncclResult_t amemGroupedGemmBf16(const void* A, const void* B, void* C, const int* group_off, int groups, int rows_cap, int rows_hint,
                                 int N, int K, int epilogue, cudaStream_t stream);
ncclResult_t amemGemmPlan(int M, int N, int K, int sms, int* tile_rows, int* tile_cols, int* tail_slices);
/* Schedule of amemAllGatherGemm for nranks ranks (1 = mover warps in every CTA, 0 = dedicated mover CTAs), rows of a
   shard per ready flag and ready flags per source rank.  Host arithmetic, no GPU needed. */
ncclResult_t amemAllGatherGemmPlan(int nranks, int rows_per_rank, int K, int* mover_warps, int* rows_per_flag, int* flags_per_rank);
/* One kernel: C[M,N] = allgather_rows(a_shard)[M,K] * B[N,K]^T.  a_shard holds this rank's
 * M/nranks rows; the transfer of the other ranks' rows overlaps the tensor-core work. */
ncclResult_t amemAllGatherGemm(const void* a_shard, const void* B, void* C, int M, int N, int K, ncclComm_t comm, cudaStream_t stream);
/* One kernel: out[M/nranks,N] = reduce_scatter_rows(A[M,K] * B[N,K]^T); partial tiles travel
 * to their owner from the epilogue and are summed there in rank order. */
ncclResult_t amemGemmReduceScatter(const void* A, const void* B, void* out, int M, int N, int K, ncclComm_t comm, cudaStream_t stream);
/* MoE expert parallelism.  Experts are spread evenly over the communicator (expert e lives on
 * rank e / (E / nranks)).  amemMoeBuffers (collective) returns this rank's receive buffer and
 * expert-output buffer, both bf16 [capacity_rows, d] in symmetric scratch memory.
 * amemMoeDispatch writes every (token, choice) row into its expert's rank at its final
 * expert-sorted position (the permutation is fused into the all-to-all); amemMoeCombine pulls
 * the expert outputs back and applies the routing weights in one pass. */
ncclResult_t amemMoeBuffers(ncclComm_t comm, int capacity_rows, int d, void** recv_x, void** y);
ncclResult_t amemMoeDispatch(const void* x, const int* topk_idx, int T, int k, int d, int E, int capacity_rows, int* expert_counts,
                             int* expert_offsets, int* send_pos, ncclComm_t comm, cudaStream_t stream);
/* The same with one more output: *dropped_rows (device int, may be null) = rows routed to this rank
 * that did not fit capacity_rows.  Such rows are not sent (send_pos -1, weight zero in the combine),
 * the counts and offsets describe only stored rows, and the communicator stays usable. */
ncclResult_t amemMoeDispatchCounted(const void* x, const int* topk_idx, int T, int k, int d, int E, int capacity_rows, int* expert_counts,
                                    int* expert_offsets, int* send_pos, int* dropped_rows, ncclComm_t comm, cudaStream_t stream);
ncclResult_t amemMoeCombine(const int* topk_idx, const float* topk_w, const int* send_pos, void* out, int T, int k, int d, int E,
                            int capacity_rows, ncclComm_t comm, cudaStream_t stream);
/* 1 if the communicator's ranks share one GPU and run as one cooperative grid; 1 if NVLS is in use. */
ncclResult_t amemCommInfo(ncclComm_t comm, int* emulated, int* nvls, size_t* stage_bytes);
/* Host-side fault injection for tests: what = "uds:drop" | "uds:short" | "uds:nofd" |
 * "uds:delay" | "uds:clear" | "vmm:create" | "vmm:map" | "vmm:import" | "vmm:export" |
 * "vmm:host_alloc"; the nth next such call misbehaves. */
ncclResult_t amemInject(const char* what, int nth, int param);
/* Bytes of physical memory and number of mappings this process holds through the backend. */
ncclResult_t amemBackendUsage(size_t* physical_bytes, size_t* mappings, const char** backend_name);
/* Runs one device thread that waits, as the collective kernels wait for their peers, for a word that
 * is set beforehand (flag_is_set != 0) or never (0), for at most timeout_ms.  *code receives the
 * device error code written to host-visible status words (0 = the flag came, 1 = the wait ran out),
 * *waited_ms the kernel's duration.  The kernel always returns; the CUDA context stays usable. */
ncclResult_t amemDeviceWaitProbe(int timeout_ms, int flag_is_set, int* code, float* waited_ms);
/* 1 when the memory backend is CUDA device memory, 0 for the host-memory mock. */
int amemBackendIsDevice(void);
/* JSON with the time spent in every kind of VMM driver call (create, map, set_access, ...). */
ncclResult_t amemBackendTimings(char* buf, size_t len, int reset);
const char* amemLastError(void);

#ifdef __cplusplus
}
#endif
#endif /* AMEM_B200_NCCL_H_ */
