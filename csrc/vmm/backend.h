// VmmBackend: the narrow interface through which the registry, the pause/resume engine
// and the communicator touch virtual-memory-managed device memory.
//
// Two implementations exist: the CUDA driver one (cuMem* / cuMulticast*), and an
// in-memory fake whose "physical allocations" are memfd files and whose mappings are
// host mmaps, so that export -> SCM_RIGHTS -> import -> remap-at-the-same-address runs
// for real between CPU-only processes.  The reference hard-wires the driver calls as
// inline helpers (amem_nccl_plugin/amem_nccl.h:141-327) and therefore has no way to be
// tested without GPUs.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

#include "../core/status.h"

namespace amem {

class VmmBackend {
 public:
  virtual ~VmmBackend() {}
  virtual const char* name() const = 0;
  // true: memory is device memory and collectives run as CUDA kernels;
  // false: memory is host shared memory and collectives run on the calling thread.
  virtual bool is_device() const = 0;

  virtual Status granularity(int dev, size_t* out) = 0;
  virtual Status mem_info(int dev, size_t* free_bytes, size_t* total_bytes) = 0;
  virtual Status device_sync(int dev) = 0;
  // Called once by a helper thread before it makes memory-management calls for device `dev`.
  virtual Status thread_init(int dev) { (void)dev; return kSuccess; }

  // Virtual address ranges.  A reserved range stays reserved across pause/resume.
  virtual Status reserve(size_t size, size_t align, uint64_t* va) = 0;
  virtual Status free_va(uint64_t va, size_t size) = 0;

  // Physical allocations (exportable as a POSIX file descriptor).
  virtual Status create(int dev, size_t size, uint64_t* handle) = 0;
  virtual Status release(uint64_t handle) = 0;
  virtual Status export_fd(uint64_t handle, int* fd) = 0;
  // Does not close `fd`; the caller owns it.
  virtual Status import_fd(int fd, size_t size, uint64_t* handle) = 0;

  // Map `handle` at `va` and give device `dev` read/write access.
  virtual Status map(uint64_t va, size_t size, uint64_t handle, int dev) = 0;
  virtual Status unmap(uint64_t va, size_t size) = 0;
  // Map now, grant access later: a backend whose access call is expensive maps only and sets
  // *needs_access; the caller then covers any number of adjacent mappings with ONE grant_access.
  // The default maps with access at once.
  virtual Status map_deferred(uint64_t va, size_t size, uint64_t handle, int dev, bool* needs_access) {
    *needs_access = false;
    return map(va, size, handle, dev);
  }
  // Read/write access for device `dev` to [va, va+size), all of which must be mapped.
  virtual Status grant_access(uint64_t va, size_t size, int dev) { (void)va; (void)size; (void)dev; return kSuccess; }

  // Pinned host shadows and the side-stream copies of pause/resume
  // (the reference's amem_launchOffload / amem_lauchPreload, amem_nccl.h:304-327).
  virtual Status host_alloc(size_t size, void** out) = 0;
  virtual Status host_free(void* p, size_t size) = 0;
  virtual Status copy_to_host_async(void* dst, uint64_t src_va, size_t size, int dev) = 0;
  virtual Status copy_to_device_async(uint64_t dst_va, const void* src, size_t size, int dev) = 0;
  virtual Status copies_sync(int dev) = 0;
  virtual Status memset_zero(uint64_t va, size_t size, int dev) = 0;

  // NVLink-switch multicast objects (NVLS).  Unsupported backends return false / error.
  virtual bool mc_supported(int dev) { (void)dev; return false; }
  virtual Status mc_granularity(int ndev, size_t size, size_t* out) { (void)ndev; (void)size; (void)out; return kInvalidUsage; }
  virtual Status mc_create(int ndev, size_t size, uint64_t* mc) { (void)ndev; (void)size; (void)mc; return kInvalidUsage; }
  virtual Status mc_add_device(uint64_t mc, int dev) { (void)mc; (void)dev; return kInvalidUsage; }
  virtual Status mc_bind(uint64_t mc, size_t mc_off, uint64_t handle, size_t size) { (void)mc; (void)mc_off; (void)handle; (void)size; return kInvalidUsage; }
  virtual Status mc_unbind(uint64_t mc, int dev, size_t mc_off, size_t size) { (void)mc; (void)dev; (void)mc_off; (void)size; return kInvalidUsage; }

  // Test hook: make the `nth` next call of the named primitive ("create", "map",
  // "import", "export", "host_alloc") fail with a system/CUDA error.  nth <= 0 clears.
  virtual void inject_failure(const char* op, int nth) { (void)op; (void)nth; }

  // Bytes of physical memory this process currently holds through this backend
  // (created or imported and not yet released).  Used by leak checks.
  virtual size_t live_physical_bytes() = 0;
  virtual size_t live_mappings() = 0;
  // JSON object with the wall time and call count of every kind of driver call so far.
  virtual std::string timings(bool reset) { (void)reset; return "{}"; }
};

// Process-wide backends.  `cuda_backend()` returns nullptr when no CUDA driver is usable.
VmmBackend* cuda_backend();
VmmBackend* mock_backend();
// Chooses by AMEM_BACKEND = cuda | mock | auto (auto: cuda when a device exists).
VmmBackend* default_backend();

}  // namespace amem
