// Harness that drives the UNMODIFIED reference plugin (libamem_nccl.so.1) through its own
// public entry points, the way its NCCL patch does.
//
// The reference's product is the plugin; its NCCL patch only reports allocations to it:
//   * a local cuMem allocation:   amem_addAllocInfo(ptr, size, LOCAL_POSIX, dev, handle, -1, 0, NULL, P2P)
//                                 (nccl_patch/nccl_2.27.5-1.diff:278-280)
//   * an ncclMemAlloc buffer:     same with caller POSIX (nccl_patch/nccl_2.27.5-1.diff:41-47)
//   * a peer's buffer mapped here: amem_addAllocInfo(ptr, size, PEER_POSIX, dev, handle, peerDev,
//                                 exporterHandle, comm, P2P_PEER) (nccl_patch/nccl_2.27.5-1.diff:572-575)
// and ncclPause / ncclResume are amem_memPause(getpid(), 0) / amem_memResume(getpid(), 0)
// (nccl_patch/nccl_2.27.5-1.diff:69-88).  This file makes the same driver calls NCCL makes
// (cuMemCreate -> reserve -> map -> set access -> export; import -> reserve -> map -> set access,
// amem_nccl_plugin/amem_nccl.h:164-234 shows the shapes) and the same plugin calls; everything
// between those calls — registry, worker threads, socket protocol, offload, release, re-create,
// re-import — is the reference's stock code.  Nothing of this repository's library is linked.
//
// Exposed as plain C functions for a ctypes caller, one process per GPU; file descriptors travel
// between the processes on the caller's side.
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include "amem_nccl.h"  // the reference's own header, used unchanged

namespace {

char g_err[512];

int drv_fail(const char* what, CUresult r) {
  const char* s = nullptr;
  cuGetErrorString(r, &s);
  snprintf(g_err, sizeof(g_err), "%s failed: %d (%s)", what, (int)r, s ? s : "?");
  return -1;
}
#define DRV(call)                                  \
  do {                                             \
    CUresult _r = (call);                          \
    if (_r != CUDA_SUCCESS) return drv_fail(#call, _r); \
  } while (0)

int g_dev = 0;
size_t g_gran = 0;

CUmemAllocationProp dev_prop() {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = g_dev;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

int set_access(CUdeviceptr p, size_t size) {
  CUmemAccessDesc a;
  memset(&a, 0, sizeof(a));
  a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  a.location.id = g_dev;
  a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  DRV(cuMemSetAccess(p, size, &a, 1));
  return 0;
}

}  // namespace

extern "C" {

const char* rh_last_error() { return g_err; }

// Binds the process to `dev` (index among the visible devices) and creates its context.
int rh_init(int dev) {
  g_dev = dev;
  if (cudaSetDevice(dev) != cudaSuccess || cudaFree(0) != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "cudaSetDevice(%d) failed: %s", dev, cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  DRV(cuInit(0));
  CUmemAllocationProp p = dev_prop();
  DRV(cuMemGetAllocationGranularity(&g_gran, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
  return 0;
}

uint64_t rh_granularity() { return g_gran; }

// One local allocation, reported to the plugin with caller tag `caller` (1 = NCCL's own p2p
// buffers, 3 = ncclMemAlloc).  Returns the device address and the allocation handle's value
// (importers pass that value back to the plugin so that it can find the exporter's record).
int rh_alloc_local(uint64_t size, int caller, uint64_t* out_ptr, uint64_t* out_handle) {
  CUmemAllocationProp p = dev_prop();
  CUmemGenericAllocationHandle h = 0;
  CUdeviceptr va = 0;
  DRV(cuMemCreate(&h, size, &p, 0));
  DRV(cuMemAddressReserve(&va, size, g_gran, 0, 0));
  DRV(cuMemMap(va, size, 0, h, 0));
  if (set_access(va, size)) return -1;
  int rc = amem_addAllocInfo(va, size, AMEM_TYPE_CUMEM_LOCAL_POSIX, g_dev, h, -1, 0ULL, NULL, (amem_caller_type)caller);
  if (rc != 0) {
    snprintf(g_err, sizeof(g_err), "amem_addAllocInfo(local) returned %d", rc);
    return -1;
  }
  *out_ptr = (uint64_t)va;
  *out_handle = (uint64_t)h;
  return 0;
}

int rh_export(uint64_t handle, int* out_fd) {
  int fd = -1;
  DRV(cuMemExportToShareableHandle(&fd, (CUmemGenericAllocationHandle)handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *out_fd = fd;
  return 0;
}

// Maps a peer's allocation here and reports it the way ncclP2pImportShareableBuffer does.
// Closes `fd`.
int rh_import(int fd, uint64_t size, int peer_dev, uint64_t exporter_handle, uint64_t* out_ptr) {
  CUmemGenericAllocationHandle h = 0;
  CUdeviceptr va = 0;
  CUresult r = cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  if (r != CUDA_SUCCESS) return drv_fail("cuMemImportFromShareableHandle", r);
  DRV(cuMemAddressReserve(&va, size, g_gran, 0, 0));
  DRV(cuMemMap(va, size, 0, h, 0));
  if (set_access(va, size)) return -1;
  int rc = amem_addAllocInfo(va, size, AMEM_TYPE_CUMEM_PEER_POSIX, g_dev, h, peer_dev, exporter_handle, NULL,
                             AMEM_CALLER_NCCL_P2P_PEER);
  if (rc != 0) {
    snprintf(g_err, sizeof(g_err), "amem_addAllocInfo(peer) returned %d", rc);
    return -1;
  }
  *out_ptr = (uint64_t)va;
  return 0;
}

// Fills [ptr, ptr+size) with the 32-bit pattern `word` and waits for it.
int rh_fill(uint64_t ptr, uint64_t size, uint32_t word) {
  DRV(cuMemsetD32((CUdeviceptr)ptr, word, size / 4));
  DRV(cuCtxSynchronize());
  return 0;
}

// Reads 4 KiB at the start, the middle and the end of the range back and compares every word
// with `word`.  Returns the number of mismatching words, -1 on a driver error.
int rh_check(uint64_t ptr, uint64_t size, uint32_t word) {
  std::vector<uint32_t> host(1024);
  const uint64_t span = host.size() * 4;
  uint64_t offs[3] = {0, (size / 2) & ~(uint64_t)4095, size >= span ? size - span : 0};
  int bad = 0;
  for (uint64_t off : offs) {
    uint64_t n = size - off < span ? size - off : span;
    DRV(cuMemcpyDtoH(host.data(), (CUdeviceptr)(ptr + off), n));
    for (uint64_t i = 0; i < n / 4; ++i) bad += host[i] != word;
  }
  return bad;
}

int rh_copy_h2d(uint64_t dst, const void* src, uint64_t size) {
  DRV(cuMemcpyHtoD((CUdeviceptr)dst, src, size));
  return 0;
}
int rh_copy_d2h(void* dst, uint64_t src, uint64_t size) {
  DRV(cuMemcpyDtoH(dst, (CUdeviceptr)src, size));
  return 0;
}

int rh_mem_info(uint64_t* free_b, uint64_t* total_b) {
  size_t f = 0, t = 0;
  if (cudaMemGetInfo(&f, &t) != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "cudaMemGetInfo failed");
    return -1;
  }
  *free_b = f;
  *total_b = t;
  return 0;
}

// What the patched ncclPause / ncclResume / ncclMemStats do.
int rh_pause() { return amem_memPause(getpid(), 0); }
int rh_resume() { return amem_memResume(getpid(), 0); }
void rh_stats() { amem_dumpAllocStats(true); }
int rh_paused() { return amem_checkPaused(false) ? 1 : 0; }

}  // extern "C"
