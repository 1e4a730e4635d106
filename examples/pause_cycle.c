/* A program written against nccl.h only: N ranks (forked processes, one GPU each, or host memory
 * with AMEM_BACKEND=mock) run  all-reduce -> ncclMemStats -> ncclPause -> ncclResume -> all-reduce
 * for a few message sizes, the way the reference's patched nccl-tests do between sizes
 * (nccl_patch/nccl-tests.diff:24-50: "ncclPause(NULL); sleep(6); ncclResume(NULL);"), and check
 * the sums.  Nothing in it is specific to this library except the three AMem calls the reference
 * adds to NCCL (nccl_patch/nccl_2.27.5-1.diff:329-355).
 *
 *   host memory, no GPU:   gcc -std=c11 -Icsrc/include examples/pause_cycle.c \
 *                              -Lasystem_amem_b200/lib -lamem_b200 -Wl,-rpath,$PWD/asystem_amem_b200/lib -o pause_cycle
 *                          AMEM_BACKEND=mock ./pause_cycle 2
 *   GPUs:                  nvcc -DWITH_CUDA -x cu ... (same flags), then ./pause_cycle 8
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#ifdef WITH_CUDA
#include <cuda_runtime.h>
#endif
#include "nccl.h"

#define CHECK(call)                                                                             \
  do {                                                                                          \
    ncclResult_t r_ = (call);                                                                   \
    if (r_ != ncclSuccess) {                                                                    \
      fprintf(stderr, "rank %d: %s failed: %s (%s)\n", rank, #call, ncclGetErrorString(r_), ncclGetLastError(NULL)); \
      return 1;                                                                                 \
    }                                                                                           \
  } while (0)

static void to_device(void* dst, const void* src, size_t bytes) {
#ifdef WITH_CUDA
  cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice);
#else
  memcpy(dst, src, bytes);
#endif
}
static void to_host(void* dst, const void* src, size_t bytes, cudaStream_t stream) {
#ifdef WITH_CUDA
  cudaStreamSynchronize(stream);
  cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost);
#else
  (void)stream;
  memcpy(dst, src, bytes);
#endif
}

static int run_rank(int rank, int nranks, const ncclUniqueId* id) {
#ifdef WITH_CUDA
  cudaSetDevice(rank);
#endif
  ncclComm_t comm;
  CHECK(ncclCommInitRank(&comm, nranks, *id, rank));
  const size_t sizes[] = {1 << 10, 1 << 20, 4 << 20};  /* elements */
  for (int s = 0; s < 3; ++s) {
    const size_t n = sizes[s];
    float* host = (float*)malloc(n * sizeof(float));
    void *send = NULL, *recv = NULL;
    CHECK(ncclMemAlloc(&send, n * sizeof(float)));   /* tracked: saved and restored across a pause */
    CHECK(ncclMemAlloc(&recv, n * sizeof(float)));
    for (size_t i = 0; i < n; ++i) host[i] = (float)(rank + 1) + (float)(i % 7);
    to_device(send, host, n * sizeof(float));
    for (int round = 0; round < 2; ++round) {
      CHECK(ncclAllReduce(send, recv, n, ncclFloat32, ncclSum, comm, NULL));
      to_host(host, recv, n * sizeof(float), NULL);
      for (size_t i = 0; i < n; i += 997) {
        float want = (float)nranks * (float)(i % 7) + (float)(nranks * (nranks + 1) / 2);
        if (host[i] != want) {
          fprintf(stderr, "rank %d: size %zu round %d element %zu is %f, expected %f\n", rank, n, round, i, host[i], want);
          return 1;
        }
      }
      if (round == 0) {
        if (rank == 0 && s == 0) CHECK(ncclMemStats());
        CHECK(ncclPause(NULL));    /* every rank: the communicator's memory is back with the driver */
        CHECK(ncclResume(NULL));   /* every rank: same addresses, same contents, no re-initialisation */
      }
    }
    CHECK(ncclMemFree(send));
    CHECK(ncclMemFree(recv));
    free(host);
  }
  CHECK(ncclCommDestroy(comm));
  return 0;
}

int main(int argc, char** argv) {
  int nranks = argc > 1 ? atoi(argv[1]) : 2;
  if (nranks < 1 || nranks > 8) {
    fprintf(stderr, "usage: %s [ranks 1..8]\n", argv[0]);
    return 2;
  }
  ncclUniqueId id;
  if (ncclGetUniqueId(&id) != ncclSuccess) {
    fprintf(stderr, "ncclGetUniqueId failed\n");
    return 2;
  }
  pid_t pids[8];
  for (int r = 0; r < nranks; ++r) {
    pids[r] = fork();
    if (pids[r] == 0) _exit(run_rank(r, nranks, &id));
  }
  int bad = 0;
  for (int r = 0; r < nranks; ++r) {
    int st = 0;
    waitpid(pids[r], &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) bad = 1;
  }
  printf(bad ? "FAILED\n" : "pause cycle ok: %d ranks\n", nranks);
  return bad;
}
