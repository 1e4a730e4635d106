#include "tracked.h"

namespace amem {

Status tracked_alloc(VmmBackend* be, uint64_t owner, int dev, size_t bytes, int category, int tag, uint64_t* va_out, size_t* rounded) {
  if (!be) return fail(kInvalidUsage, "no usable memory backend");
  if (bytes == 0) return fail(kInvalidArgument, "empty allocation");
  Registry& reg = Registry::instance();
  if (reg.is_paused(owner)) return fail(kInvalidUsage, "allocation while the owner's memory is paused");
  size_t gran = 0;
  AMEM_TRY(be->granularity(dev, &gran));
  size_t sz = (bytes + gran - 1) / gran * gran;
  uint64_t va = 0, h = 0;
  AMEM_TRY(be->reserve(sz, gran, &va));
  Status s = be->create(dev, sz, &h);
  if (s != kSuccess) {
    be->free_va(va, sz);
    return s;
  }
  if ((s = be->map(va, sz, h, dev)) != kSuccess) {
    be->release(h);
    be->free_va(va, sz);
    return s;
  }
  Allocation rec;
  rec.va = va;
  rec.size = sz;
  rec.handle = h;
  rec.dev = dev;
  rec.type = kLocalPosix;
  rec.category = category;
  rec.tag = tag;
  rec.owner = owner;
  if ((s = reg.add(rec)) != kSuccess) {
    be->unmap(va, sz);
    be->release(h);
    be->free_va(va, sz);
    return s;
  }
  *va_out = va;
  if (rounded) *rounded = sz;
  return kSuccess;
}

Status tracked_free(VmmBackend* be, uint64_t va) {
  Allocation a;
  if (!Registry::instance().find(va, &a) || from_peer(a.type)) return fail(kInvalidArgument, "%#llx is not a tracked local allocation", (unsigned long long)va);
  if (a.state != kMemHole) {
    if (be->is_device()) be->device_sync(a.dev);
    be->unmap(a.va, a.size);
    be->release(a.handle);
  }
  if (a.shadow) be->host_free(a.shadow, a.size);
  be->free_va(a.va, a.size);
  Registry::instance().remove(a.va);
  return kSuccess;
}

}  // namespace amem
