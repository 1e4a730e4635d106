#include "registry.h"

#include <algorithm>
#include <cstring>

#include "../core/log.h"

namespace amem {

Registry::Registry() { group_id_ = (int)env_long("AMEM_GROUPID", 0); }

Registry& Registry::instance() {
  static Registry* r = new Registry();
  return *r;
}

Status Registry::add(const Allocation& a) {
  std::lock_guard<std::mutex> g(mu_);
  auto os = owner_state_.find(a.owner);
  bool owner_paused = os != owner_state_.end() && (os->second == kRunPaused || os->second == kRunPausing);
  if (process_paused_ || owner_paused)
    return fail(kInvalidUsage, "allocation of %zu bytes refused: memory of this scope is paused", a.size);
  if (a.va == 0 || a.size == 0) return fail(kInvalidArgument, "registry add: empty allocation");
  auto it = by_va_.find(a.va);
  if (it != by_va_.end()) {
    LOGW("registry: address %#llx registered twice; replacing the %zu-byte record", (unsigned long long)a.va, it->second.size);
    if (it->second.handle) by_handle_.erase(it->second.handle);
    by_va_.erase(it);
  }
  Allocation rec = a;
  if (rec.state == kMemInvalid) rec.state = kMemAlloc;
  by_va_[rec.va] = rec;
  if (rec.handle && !from_peer(rec.type)) by_handle_[rec.handle] = rec.va;
  ever_added_ = true;
  return kSuccess;
}

Status Registry::remove(uint64_t va) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_va_.find(va);
  if (it == by_va_.end()) return fail(kInvalidArgument, "registry remove: %#llx is not tracked", (unsigned long long)va);
  if (it->second.handle) {
    auto h = by_handle_.find(it->second.handle);
    if (h != by_handle_.end() && h->second == va) by_handle_.erase(h);
  }
  by_va_.erase(it);
  return kSuccess;
}

bool Registry::find(uint64_t va, Allocation* out) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_va_.find(va);
  if (it == by_va_.end()) return false;
  if (out) *out = it->second;
  return true;
}

bool Registry::find_by_handle(uint64_t handle, Allocation* out) {
  std::lock_guard<std::mutex> g(mu_);
  auto h = by_handle_.find(handle);
  if (h == by_handle_.end()) return false;
  auto it = by_va_.find(h->second);
  if (it == by_va_.end()) return false;
  if (out) *out = it->second;
  return true;
}

bool Registry::find_containing(uint64_t addr, Allocation* out) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_va_.upper_bound(addr);
  if (it == by_va_.begin()) return false;
  --it;
  if (addr >= it->second.va + it->second.size) return false;
  if (out) *out = it->second;
  return true;
}

Status Registry::add_importer(uint64_t va, int rank) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_va_.find(va);
  if (it == by_va_.end()) return fail(kInvalidArgument, "add_importer: %#llx is not tracked", (unsigned long long)va);
  if (rank < 0 || rank >= 32) return fail(kInvalidArgument, "add_importer: rank %d out of range", rank);
  it->second.importers |= 1u << rank;
  return kSuccess;
}

Status Registry::update(const Allocation& a) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = by_va_.find(a.va);
  if (it == by_va_.end()) return fail(kInvalidArgument, "registry update: %#llx is not tracked", (unsigned long long)a.va);
  if (it->second.handle && !from_peer(it->second.type)) {
    auto h = by_handle_.find(it->second.handle);
    if (h != by_handle_.end() && h->second == a.va) by_handle_.erase(h);
  }
  it->second = a;
  if (a.handle && !from_peer(a.type)) by_handle_[a.handle] = a.va;
  return kSuccess;
}

std::vector<Allocation> Registry::snapshot(uint64_t owner, bool any_owner) {
  std::vector<Allocation> v;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : by_va_)
      if (any_owner || kv.second.owner == owner) v.push_back(kv.second);
  }
  std::sort(v.begin(), v.end(), [](const Allocation& x, const Allocation& y) {
    if (x.owner != y.owner) return x.owner < y.owner;
    if (x.sym_id != y.sym_id) return x.sym_id < y.sym_id;
    if (x.exporter_rank != y.exporter_rank) return x.exporter_rank < y.exporter_rank;
    return x.va < y.va;
  });
  return v;
}

void Registry::stats(MemStats* out) {
  memset(out, 0, sizeof(*out));
  std::lock_guard<std::mutex> g(mu_);
  for (auto& kv : by_va_) {
    const Allocation& a = kv.second;
    int tag = a.tag >= 0 && a.tag < kMaxCaller ? a.tag : 0;
    out->bytes_by_tag[tag] += a.size;
    if (from_peer(a.type)) {
      out->imported_bytes += a.size;
      out->n_imported++;
    } else {
      out->n_local++;
      if (a.category == kScratch) out->scratch_bytes += a.size;
      else out->stateful_bytes += a.size;  // saved-on-pause and resident protocol state
      if (a.mc_handle) out->multicast_bytes += a.size;
    }
    if (a.state == kMemHole) out->paused_bytes += a.size;
    else out->live_bytes += a.size;
    if (a.shadow) out->shadow_bytes += a.size;
  }
  out->pause_count = pause_count_.load();
  out->resume_count = resume_count_.load();
  out->group_id = group_id_;
  out->paused = process_paused_ ? 1 : 0;
}

void Registry::dump_stats(bool verbose) {
  MemStats s;
  stats(&s);
  // Same shape as the reference's ncclMemStats lines: "caller_N allocBytes" and a total.
  uint64_t total = 0;
  for (int i = 0; i < kMaxCaller; ++i) {
    if (!s.bytes_by_tag[i]) continue;
    total += s.bytes_by_tag[i];
    LOGI("group:%d caller_%d allocBytes:%llu", s.group_id, i, (unsigned long long)s.bytes_by_tag[i]);
  }
  LOGI("group:%d total allocBytes:%llu (%llu MB) stateful:%llu scratch:%llu imported:%llu multicast:%llu live:%llu paused:%llu shadows:%llu pauses:%llu resumes:%llu",
       s.group_id, (unsigned long long)total, (unsigned long long)(total >> 20), (unsigned long long)s.stateful_bytes,
       (unsigned long long)s.scratch_bytes, (unsigned long long)s.imported_bytes, (unsigned long long)s.multicast_bytes,
       (unsigned long long)s.live_bytes, (unsigned long long)s.paused_bytes, (unsigned long long)s.shadow_bytes,
       (unsigned long long)s.pause_count, (unsigned long long)s.resume_count);
  if (verbose) {
    for (auto& a : snapshot(0, true))
      LOGI("  va:%#llx size:%zu type:%d tag:%d cat:%d owner:%#llx sym:%u exporter:%d importers:%#x state:%d",
           (unsigned long long)a.va, a.size, a.type, a.tag, a.category, (unsigned long long)a.owner, a.sym_id,
           a.exporter_rank, a.importers, a.state);
  }
}

Status Registry::set_group_id(int id) {
  std::lock_guard<std::mutex> g(mu_);
  if (ever_added_) return fail(kInvalidUsage, "group id can only be set before the first tracked allocation");
  group_id_ = id;
  return kSuccess;
}

int Registry::group_id() {
  std::lock_guard<std::mutex> g(mu_);
  return group_id_;
}

void Registry::set_owner_state(uint64_t owner, int run_state) {
  std::lock_guard<std::mutex> g(mu_);
  owner_state_[owner] = run_state;
}

int Registry::owner_state(uint64_t owner) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = owner_state_.find(owner);
  return it == owner_state_.end() ? kRunInit : it->second;
}

void Registry::set_process_paused(bool p) {
  std::lock_guard<std::mutex> g(mu_);
  process_paused_ = p;
}

bool Registry::process_paused() {
  std::lock_guard<std::mutex> g(mu_);
  return process_paused_;
}

void Registry::forget_owner(uint64_t owner) {
  std::lock_guard<std::mutex> g(mu_);
  owner_state_.erase(owner);
}

size_t Registry::size() {
  std::lock_guard<std::mutex> g(mu_);
  return by_va_.size();
}

}  // namespace amem
