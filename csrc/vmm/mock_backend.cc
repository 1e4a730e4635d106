// In-memory fake of the VMM backend for GPU-less machines.
//
// physical allocation = memfd file; export = dup(); import = dup() of the received fd;
// reserve = PROT_NONE anonymous mapping; map = MAP_FIXED|MAP_SHARED of the memfd over the
// reservation; unmap = put the PROT_NONE hole back (the address stays reserved, exactly
// like cuMemUnmap without cuMemAddressFree).  Two CPU processes that exchange such fds
// over a Unix socket really share the pages, so the host collectives and the whole
// pause/resume protocol are exercised without a GPU.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "../core/log.h"
#include "backend.h"

namespace amem {
namespace {

class MockBackend : public VmmBackend {
 public:
  const char* name() const override { return "mock"; }
  bool is_device() const override { return false; }

  Status granularity(int, size_t* out) override {
    *out = (size_t)env_long("AMEM_MOCK_GRANULARITY", 64 * 1024);
    return kSuccess;
  }
  Status mem_info(int, size_t* free_bytes, size_t* total_bytes) override {
    size_t total = (size_t)env_long("AMEM_MOCK_TOTAL_MB", 8192) << 20;
    std::lock_guard<std::mutex> g(mu_);
    *total_bytes = total;
    *free_bytes = total > live_bytes_ ? total - live_bytes_ : 0;
    return kSuccess;
  }
  Status device_sync(int) override { return kSuccess; }

  Status reserve(size_t size, size_t align, uint64_t* va) override {
    if (align < 4096) align = 4096;
    size_t span = size + align;
    void* p = mmap(nullptr, span, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (p == MAP_FAILED) return fail(kSystemError, "mock reserve mmap: %s", strerror(errno));
    uint64_t base = (uint64_t)p;
    uint64_t aligned = (base + align - 1) / align * align;
    if (aligned > base) munmap((void*)base, aligned - base);
    uint64_t end = base + span, aend = aligned + size;
    if (end > aend) munmap((void*)aend, end - aend);
    *va = aligned;
    return kSuccess;
  }
  Status free_va(uint64_t va, size_t size) override {
    if (munmap((void*)va, size) != 0) return fail(kSystemError, "mock free_va: %s", strerror(errno));
    return kSuccess;
  }

  Status create(int, size_t size, uint64_t* handle) override {
    if (should_fail("create")) return fail(kCudaError, "mock create: injected out-of-memory");
    int fd = (int)syscall(SYS_memfd_create, "amem_mock_phys", 0u);
    if (fd < 0) return fail(kSystemError, "memfd_create: %s", strerror(errno));
    if (ftruncate(fd, (off_t)size) != 0) {
      close(fd);
      return fail(kSystemError, "ftruncate: %s", strerror(errno));
    }
    std::lock_guard<std::mutex> g(mu_);
    uint64_t h = next_handle_++;
    phys_[h] = Phys{fd, size};
    live_bytes_ += size;
    *handle = h;
    return kSuccess;
  }
  Status release(uint64_t handle) override {
    std::lock_guard<std::mutex> g(mu_);
    auto it = phys_.find(handle);
    if (it == phys_.end()) return fail(kInvalidArgument, "mock release: unknown handle %llu", (unsigned long long)handle);
    close(it->second.fd);
    live_bytes_ -= it->second.size;
    phys_.erase(it);
    return kSuccess;
  }
  Status export_fd(uint64_t handle, int* fd) override {
    if (should_fail("export")) return fail(kCudaError, "mock export: injected failure");
    std::lock_guard<std::mutex> g(mu_);
    auto it = phys_.find(handle);
    if (it == phys_.end()) return fail(kInvalidArgument, "mock export: unknown handle");
    int d = dup(it->second.fd);
    if (d < 0) return fail(kSystemError, "dup: %s", strerror(errno));
    *fd = d;
    return kSuccess;
  }
  Status import_fd(int fd, size_t size, uint64_t* handle) override {
    if (should_fail("import")) return fail(kCudaError, "mock import: injected failure");
    int d = dup(fd);
    if (d < 0) return fail(kSystemError, "dup(import): %s", strerror(errno));
    std::lock_guard<std::mutex> g(mu_);
    uint64_t h = next_handle_++;
    phys_[h] = Phys{d, size};
    live_bytes_ += size;
    *handle = h;
    return kSuccess;
  }

  Status map(uint64_t va, size_t size, uint64_t handle, int) override {
    if (should_fail("map")) return fail(kCudaError, "mock map: injected failure");
    int fd;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = phys_.find(handle);
      if (it == phys_.end()) return fail(kInvalidArgument, "mock map: unknown handle");
      if (it->second.size < size) return fail(kInvalidArgument, "mock map: size beyond allocation");
      fd = it->second.fd;
    }
    void* p = mmap((void*)va, size, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0);
    if (p == MAP_FAILED) return fail(kSystemError, "mock map mmap: %s", strerror(errno));
    std::lock_guard<std::mutex> g(mu_);
    ++mappings_;
    return kSuccess;
  }
  Status unmap(uint64_t va, size_t size) override {
    void* p = mmap((void*)va, size, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_FIXED | MAP_NORESERVE, -1, 0);
    if (p == MAP_FAILED) return fail(kSystemError, "mock unmap mmap: %s", strerror(errno));
    std::lock_guard<std::mutex> g(mu_);
    --mappings_;
    return kSuccess;
  }

  Status host_alloc(size_t size, void** out) override {
    if (should_fail("host_alloc")) return fail(kSystemError, "mock host_alloc: injected failure");
    void* p = nullptr;
    if (posix_memalign(&p, 4096, size ? size : 1) != 0) return fail(kSystemError, "posix_memalign failed");
    *out = p;
    return kSuccess;
  }
  Status host_free(void* p, size_t) override {
    free(p);
    return kSuccess;
  }
  Status copy_to_host_async(void* dst, uint64_t src_va, size_t size, int) override {
    memcpy(dst, (const void*)src_va, size);
    return kSuccess;
  }
  Status copy_to_device_async(uint64_t dst_va, const void* src, size_t size, int) override {
    memcpy((void*)dst_va, src, size);
    return kSuccess;
  }
  Status copies_sync(int) override { return kSuccess; }
  Status memset_zero(uint64_t va, size_t size, int) override {
    memset((void*)va, 0, size);
    return kSuccess;
  }

  void inject_failure(const char* op, int nth) override {
    std::lock_guard<std::mutex> g(mu_);
    if (nth <= 0) inject_.erase(op);
    else inject_[op] = nth;
  }
  size_t live_physical_bytes() override {
    std::lock_guard<std::mutex> g(mu_);
    return live_bytes_;
  }
  size_t live_mappings() override {
    std::lock_guard<std::mutex> g(mu_);
    return (size_t)mappings_;
  }

 private:
  struct Phys {
    int fd;
    size_t size;
  };
  bool should_fail(const char* op) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = inject_.find(op);
    if (it == inject_.end()) return false;
    if (--it->second == 0) {
      inject_.erase(it);
      return true;
    }
    return false;
  }
  std::mutex mu_;
  std::map<uint64_t, Phys> phys_;
  std::map<std::string, int> inject_;
  uint64_t next_handle_ = 1;
  size_t live_bytes_ = 0;
  long mappings_ = 0;
};

}  // namespace

VmmBackend* mock_backend() {
  static MockBackend* b = new MockBackend();
  return b;
}

}  // namespace amem
