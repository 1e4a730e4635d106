// CUDA driver implementation of the VMM backend (cuMem* / cuMulticast*).
//
// Driver entry points are fetched through cudaGetDriverEntryPoint, so the library has no
// link-time dependency on libcuda and loads on machines without a driver (where only the
// mock backend is usable).  Physical allocations are pinned device memory with POSIX
// file-descriptor shareable handles, as in the reference (amem_nccl.h:164-193); virtual
// addresses are never freed by unmap, which is what lets resume put memory back at the
// same address.
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <string>

#include "../core/log.h"
#include "backend.h"

namespace amem {
namespace {

struct Drv {
  bool ok = false;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
};

template <typename F>
bool load_sym(const char* name, F* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<F>(fn);
  return true;
}

Drv& drv() {
  static Drv d;
  static std::once_flag once;
  std::call_once(once, [] {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
      cudaGetLastError();
      return;
    }
    bool ok = true;
    ok &= load_sym("cuMemGetAllocationGranularity", &d.MemGetAllocationGranularity);
    ok &= load_sym("cuMemAddressReserve", &d.MemAddressReserve);
    ok &= load_sym("cuMemAddressFree", &d.MemAddressFree);
    ok &= load_sym("cuMemCreate", &d.MemCreate);
    ok &= load_sym("cuMemRelease", &d.MemRelease);
    ok &= load_sym("cuMemMap", &d.MemMap);
    ok &= load_sym("cuMemUnmap", &d.MemUnmap);
    ok &= load_sym("cuMemSetAccess", &d.MemSetAccess);
    ok &= load_sym("cuMemExportToShareableHandle", &d.MemExportToShareableHandle);
    ok &= load_sym("cuMemImportFromShareableHandle", &d.MemImportFromShareableHandle);
    ok &= load_sym("cuGetErrorString", &d.GetErrorString);
    ok &= load_sym("cuDeviceGetAttribute", &d.DeviceGetAttribute);
    // Multicast is optional (absent on old drivers).
    load_sym("cuMulticastCreate", &d.MulticastCreate);
    load_sym("cuMulticastAddDevice", &d.MulticastAddDevice);
    load_sym("cuMulticastBindMem", &d.MulticastBindMem);
    load_sym("cuMulticastUnbind", &d.MulticastUnbind);
    load_sym("cuMulticastGetGranularity", &d.MulticastGetGranularity);
    d.ok = ok;
  });
  return d;
}

Status drv_fail(const char* what, CUresult r) {
  const char* s = nullptr;
  if (drv().GetErrorString) drv().GetErrorString(r, &s);
  return fail(kCudaError, "%s failed: %d (%s)", what, (int)r, s ? s : "?");
}
Status rt_fail(const char* what, cudaError_t e) {
  return fail(kCudaError, "%s failed: %s", what, cudaGetErrorString(e));
}
#define DRV(call, what)                         \
  do {                                          \
    CUresult _r = (call);                       \
    if (_r != CUDA_SUCCESS) return drv_fail(what, _r); \
  } while (0)
#define RT(call, what)                          \
  do {                                          \
    cudaError_t _e = (call);                    \
    if (_e != cudaSuccess) return rt_fail(what, _e);  \
  } while (0)

CUmemAllocationProp device_prop(int dev) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = dev;
  p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return p;
}

// Wall time spent in each kind of driver call (AMEM tooling: amemBackendTimings).
struct CallTimer {
  std::atomic<uint64_t> ns{0}, calls{0};
};
enum { kTCreate, kTRelease, kTMap, kTAccess, kTUnmap, kTImport, kTExport, kTBind, kTUnbind, kTCount };
static CallTimer g_timers[kTCount];
static const char* kTimerNames[kTCount] = {"create", "release", "map", "set_access", "unmap", "import", "export", "mc_bind", "mc_unbind"};
struct Timed {
  int which;
  double t0;
  explicit Timed(int w) : which(w), t0(now_ms()) {}
  ~Timed() {
    g_timers[which].ns.fetch_add((uint64_t)((now_ms() - t0) * 1e6));
    g_timers[which].calls.fetch_add(1);
  }
};

class CudaBackend : public VmmBackend {
 public:
  std::string timings(bool reset) override {
    char buf[64];
    std::string out = "{";
    for (int i = 0; i < kTCount; ++i) {
      snprintf(buf, sizeof(buf), "%s\"%s_us\": %.1f, \"%s_calls\": %llu", i ? ", " : "", kTimerNames[i], g_timers[i].ns.load() / 1e3,
               kTimerNames[i], (unsigned long long)g_timers[i].calls.load());
      out += buf;
      if (reset) {
        g_timers[i].ns = 0;
        g_timers[i].calls = 0;
      }
    }
    return out + "}";
  }
  const char* name() const override { return "cuda"; }
  bool is_device() const override { return true; }

  Status granularity(int dev, size_t* out) override {
    CUmemAllocationProp p = device_prop(dev);
    // The recommended granularity (2 MiB on current parts) also satisfies multicast binding.
    DRV(drv().MemGetAllocationGranularity(out, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    return kSuccess;
  }
  Status mem_info(int dev, size_t* free_bytes, size_t* total_bytes) override {
    int cur = 0;
    RT(cudaGetDevice(&cur), "cudaGetDevice");
    if (cur != dev) RT(cudaSetDevice(dev), "cudaSetDevice");
    cudaError_t e = cudaMemGetInfo(free_bytes, total_bytes);
    if (cur != dev) cudaSetDevice(cur);
    RT(e, "cudaMemGetInfo");
    return kSuccess;
  }
  Status thread_init(int dev) override {
    RT(cudaSetDevice(dev), "cudaSetDevice");  // binds the device's primary context to this thread
    return kSuccess;
  }
  Status device_sync(int dev) override {
    int cur = 0;
    RT(cudaGetDevice(&cur), "cudaGetDevice");
    if (cur != dev) RT(cudaSetDevice(dev), "cudaSetDevice");
    cudaError_t e = cudaDeviceSynchronize();
    if (cur != dev) cudaSetDevice(cur);
    RT(e, "cudaDeviceSynchronize");
    return kSuccess;
  }

  Status reserve(size_t size, size_t align, uint64_t* va) override {
    CUdeviceptr p = 0;
    DRV(drv().MemAddressReserve(&p, size, align, 0, 0), "cuMemAddressReserve");
    *va = (uint64_t)p;
    return kSuccess;
  }
  Status free_va(uint64_t va, size_t size) override {
    DRV(drv().MemAddressFree((CUdeviceptr)va, size), "cuMemAddressFree");
    return kSuccess;
  }

  Status create(int dev, size_t size, uint64_t* handle) override {
    if (should_fail("create")) return fail(kCudaError, "cuMemCreate: injected out-of-memory");
    CUmemAllocationProp p = device_prop(dev);
    CUmemGenericAllocationHandle h = 0;
    {
      Timed t(kTCreate);
      DRV(drv().MemCreate(&h, size, &p, 0), "cuMemCreate");
    }
    *handle = (uint64_t)h;
    note_phys(h, size, +1);
    return kSuccess;
  }
  Status release(uint64_t handle) override {
    {
      Timed t(kTRelease);
      DRV(drv().MemRelease((CUmemGenericAllocationHandle)handle), "cuMemRelease");
    }
    note_phys(handle, 0, -1);
    return kSuccess;
  }
  Status export_fd(uint64_t handle, int* fd) override {
    if (should_fail("export")) return fail(kCudaError, "cuMemExportToShareableHandle: injected failure");
    int out = -1;
    Timed t(kTExport);
    DRV(drv().MemExportToShareableHandle(&out, (CUmemGenericAllocationHandle)handle,
                                         CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
        "cuMemExportToShareableHandle");
    *fd = out;
    return kSuccess;
  }
  Status import_fd(int fd, size_t size, uint64_t* handle) override {
    if (should_fail("import")) return fail(kCudaError, "cuMemImportFromShareableHandle: injected failure");
    CUmemGenericAllocationHandle h = 0;
    Timed t(kTImport);
    DRV(drv().MemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
        "cuMemImportFromShareableHandle");
    *handle = (uint64_t)h;
    // (An import inside the exporting process yields a handle with a reference of its own,
    // so emulated ranks release imports exactly like ranks in other processes do.)
    note_phys(h, size, +1);
    return kSuccess;
  }

  Status map(uint64_t va, size_t size, uint64_t handle, int dev) override {
    if (should_fail("map")) return fail(kCudaError, "cuMemMap: injected failure");
    {
      Timed t(kTMap);
      DRV(drv().MemMap((CUdeviceptr)va, size, 0, (CUmemGenericAllocationHandle)handle, 0), "cuMemMap");
    }
    Timed t2(kTAccess);
    CUmemAccessDesc a;
    memset(&a, 0, sizeof(a));
    a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    a.location.id = dev;
    a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CUresult r = drv().MemSetAccess((CUdeviceptr)va, size, &a, 1);
    if (r != CUDA_SUCCESS) {
      drv().MemUnmap((CUdeviceptr)va, size);
      return drv_fail("cuMemSetAccess", r);
    }
    mappings_.fetch_add(1);
    return kSuccess;
  }
  Status map_deferred(uint64_t va, size_t size, uint64_t handle, int dev, bool* needs_access) override {
    (void)dev;
    if (should_fail("map")) return fail(kCudaError, "cuMemMap: injected failure");
    static const long defer = env_long("AMEM_DEFER_ACCESS", 1);
    if (!defer) {
      *needs_access = false;
      return map(va, size, handle, dev);
    }
    Timed t(kTMap);
    DRV(drv().MemMap((CUdeviceptr)va, size, 0, (CUmemGenericAllocationHandle)handle, 0), "cuMemMap");
    mappings_.fetch_add(1);
    *needs_access = true;
    return kSuccess;
  }
  Status grant_access(uint64_t va, size_t size, int dev) override {
    Timed t(kTAccess);
    CUmemAccessDesc a;
    memset(&a, 0, sizeof(a));
    a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    a.location.id = dev;
    a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    DRV(drv().MemSetAccess((CUdeviceptr)va, size, &a, 1), "cuMemSetAccess");
    return kSuccess;
  }
  Status unmap(uint64_t va, size_t size) override {
    {
      Timed t(kTUnmap);
      DRV(drv().MemUnmap((CUdeviceptr)va, size), "cuMemUnmap");
    }
    mappings_.fetch_sub(1);
    return kSuccess;
  }

  // Host shadows.  First choice: a VMM allocation of pinned host memory on the NUMA node the GPU
  // hangs off (CU_MEM_LOCATION_TYPE_HOST_NUMA), mapped for the device and for the CPU, so the
  // save / restore copies stay on the local socket's memory controller — what the reference does
  // (amem_nccl_plugin/amem_nccl.h:237-283, with its fallback to node 0).  Where the driver or
  // the machine refuses that (no NUMA id, old driver, cgroup limits), plain cudaHostAlloc.
  // AMEM_HOST_NUMA=0 goes straight to cudaHostAlloc.
  Status host_alloc(size_t size, void** out) override {
    if (should_fail("host_alloc")) return fail(kSystemError, "cudaHostAlloc: injected failure");
    if (size == 0) size = 1;
    static const long want_numa = env_long("AMEM_HOST_NUMA", 1);
    if (want_numa && numa_host_alloc(size, out)) return kSuccess;
    RT(cudaHostAlloc(out, size, cudaHostAllocPortable), "cudaHostAlloc");
    return kSuccess;
  }
  Status host_free(void* p, size_t) override {
    HostVmm hv;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = host_vmm_.find(p);
      if (it == host_vmm_.end()) hv.handle = 0;
      else {
        hv = it->second;
        host_vmm_.erase(it);
      }
    }
    if (hv.handle) {
      drv().MemUnmap((CUdeviceptr)p, hv.size);
      drv().MemRelease((CUmemGenericAllocationHandle)hv.handle);
      drv().MemAddressFree((CUdeviceptr)p, hv.size);
      return kSuccess;
    }
    RT(cudaFreeHost(p), "cudaFreeHost");
    return kSuccess;
  }
  Status copy_to_host_async(void* dst, uint64_t src_va, size_t size, int dev) override {
    cudaStream_t s;
    AMEM_TRY(side_stream(dev, &s));
    RT(cudaMemcpyAsync(dst, (const void*)src_va, size, cudaMemcpyDefault, s), "cudaMemcpyAsync(D2H)");
    return kSuccess;
  }
  Status copy_to_device_async(uint64_t dst_va, const void* src, size_t size, int dev) override {
    cudaStream_t s;
    AMEM_TRY(side_stream(dev, &s));
    RT(cudaMemcpyAsync((void*)dst_va, src, size, cudaMemcpyDefault, s), "cudaMemcpyAsync(H2D)");
    return kSuccess;
  }
  Status copies_sync(int dev) override {
    cudaStream_t s;
    AMEM_TRY(side_stream(dev, &s));
    RT(cudaStreamSynchronize(s), "cudaStreamSynchronize(side)");
    return kSuccess;
  }
  Status memset_zero(uint64_t va, size_t size, int dev) override {
    cudaStream_t s;
    AMEM_TRY(side_stream(dev, &s));
    RT(cudaMemsetAsync((void*)va, 0, size, s), "cudaMemsetAsync");
    return kSuccess;
  }

  bool mc_supported(int dev) override {
    if (!drv().MulticastCreate) return false;
    int v = 0;
    if (drv().DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) != CUDA_SUCCESS) return false;
    return v != 0;
  }
  static CUmulticastObjectProp mc_prop(int ndev, size_t size) {
    CUmulticastObjectProp p;
    memset(&p, 0, sizeof(p));
    p.numDevices = (unsigned)ndev;
    p.size = size;
    p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return p;
  }
  Status mc_granularity(int ndev, size_t size, size_t* out) override {
    CUmulticastObjectProp p = mc_prop(ndev, size);
    // The recommended granularity is 512 MiB on B200; the minimum (2 MiB) is what binding needs.
    DRV(drv().MulticastGetGranularity(out, &p, CU_MULTICAST_GRANULARITY_MINIMUM), "cuMulticastGetGranularity");
    return kSuccess;
  }
  Status mc_create(int ndev, size_t size, uint64_t* mc) override {
    CUmulticastObjectProp p = mc_prop(ndev, size);
    CUmemGenericAllocationHandle h = 0;
    DRV(drv().MulticastCreate(&h, &p), "cuMulticastCreate");
    *mc = (uint64_t)h;
    return kSuccess;
  }
  Status mc_add_device(uint64_t mc, int dev) override {
    DRV(drv().MulticastAddDevice((CUmemGenericAllocationHandle)mc, (CUdevice)dev), "cuMulticastAddDevice");
    return kSuccess;
  }
  Status mc_bind(uint64_t mc, size_t mc_off, uint64_t handle, size_t size) override {
    Timed t(kTBind);
    DRV(drv().MulticastBindMem((CUmemGenericAllocationHandle)mc, mc_off, (CUmemGenericAllocationHandle)handle, 0, size, 0),
        "cuMulticastBindMem");
    return kSuccess;
  }
  Status mc_unbind(uint64_t mc, int dev, size_t mc_off, size_t size) override {
    Timed t(kTUnbind);
    DRV(drv().MulticastUnbind((CUmemGenericAllocationHandle)mc, (CUdevice)dev, mc_off, size), "cuMulticastUnbind");
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
  size_t live_mappings() override { return (size_t)mappings_.load(); }

 private:
  struct HostVmm {
    uint64_t handle = 0;
    size_t size = 0;
  };
  // Pinned host memory from the VMM allocator on the current device's NUMA node (node 0 as the
  // second try).  Any failure leaves nothing behind and returns false.
  bool numa_host_alloc(size_t size, void** out) {
    int dev = 0, node = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    if (drv().DeviceGetAttribute(&node, CU_DEVICE_ATTRIBUTE_HOST_NUMA_ID, dev) != CUDA_SUCCESS || node < 0) node = 0;
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_HOST_NUMA;
    prop.location.id = node;
    size_t gran = 0;
    if (drv().MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) != CUDA_SUCCESS || gran == 0) return false;
    size_t sz = (size + gran - 1) / gran * gran;
    CUmemGenericAllocationHandle h = 0;
    if (drv().MemCreate(&h, sz, &prop, 0) != CUDA_SUCCESS) {
      if (node == 0) return false;
      prop.location.id = node = 0;
      if (drv().MemCreate(&h, sz, &prop, 0) != CUDA_SUCCESS) return false;
    }
    CUdeviceptr va = 0;
    if (drv().MemAddressReserve(&va, sz, gran, 0, 0) != CUDA_SUCCESS) {
      drv().MemRelease(h);
      return false;
    }
    if (drv().MemMap(va, sz, 0, h, 0) != CUDA_SUCCESS) {
      drv().MemAddressFree(va, sz);
      drv().MemRelease(h);
      return false;
    }
    CUmemAccessDesc acc[2];
    memset(acc, 0, sizeof(acc));
    acc[0].location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc[0].location.id = dev;
    acc[0].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    acc[1].location.type = CU_MEM_LOCATION_TYPE_HOST_NUMA;
    acc[1].location.id = node;
    acc[1].flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if (drv().MemSetAccess(va, sz, acc, 2) != CUDA_SUCCESS) {
      drv().MemUnmap(va, sz);
      drv().MemAddressFree(va, sz);
      drv().MemRelease(h);
      return false;
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      HostVmm hv;
      hv.handle = (uint64_t)h;
      hv.size = sz;
      host_vmm_[(void*)va] = hv;
    }
    *out = (void*)va;
    return true;
  }
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
  void note_phys(uint64_t h, size_t size, int dir) {
    std::lock_guard<std::mutex> g(mu_);
    if (dir > 0) {
      sizes_[h] = size;
      live_bytes_ += size;
    } else {
      auto it = sizes_.find(h);
      if (it != sizes_.end()) {
        live_bytes_ -= it->second;
        sizes_.erase(it);
      }
    }
  }
  Status side_stream(int dev, cudaStream_t* out) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = streams_.find(dev);
    if (it == streams_.end()) {
      int cur = 0;
      RT(cudaGetDevice(&cur), "cudaGetDevice");
      if (cur != dev) RT(cudaSetDevice(dev), "cudaSetDevice");
      cudaStream_t s;
      cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
      if (cur != dev) cudaSetDevice(cur);
      RT(e, "cudaStreamCreate(side)");
      it = streams_.emplace(dev, s).first;
    }
    *out = it->second;
    return kSuccess;
  }
  std::mutex mu_;
  std::map<int, cudaStream_t> streams_;
  std::map<uint64_t, size_t> sizes_;
  std::map<std::string, int> inject_;
  std::map<void*, HostVmm> host_vmm_;
  size_t live_bytes_ = 0;
  std::atomic<long> mappings_{0};
};

}  // namespace

VmmBackend* cuda_backend() {
  if (!drv().ok) return nullptr;
  static CudaBackend* b = new CudaBackend();
  return b;
}

VmmBackend* default_backend() {
  std::string want = env_str("AMEM_BACKEND", "auto");
  if (want == "mock") return mock_backend();
  VmmBackend* c = cuda_backend();
  if (want == "cuda") return c;
  return c ? c : mock_backend();
}

}  // namespace amem
