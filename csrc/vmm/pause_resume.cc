#include "pause_resume.h"

#include <unistd.h>

#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../core/log.h"

#if defined(AMEM_WITH_NVTX)
#include <nvtx3/nvToolsExt.h>
#define RANGE_PUSH(name) nvtxRangePushA(name)
#define RANGE_POP() nvtxRangePop()
#else
#define RANGE_PUSH(name) ((void)0)
#define RANGE_POP() ((void)0)
#endif

namespace amem {
namespace {

struct Phase {
  double t0;
  double* slot;
  Phase(const char* name, double* s) : t0(now_ms()), slot(s) { RANGE_PUSH(name); (void)name; }
  ~Phase() {
    RANGE_POP();
    if (slot) *slot += (now_ms() - t0) * 1000.0;
  }
};

bool is_local(const Allocation& a) { return !from_peer(a.type); }

// Runs fn(0) .. fn(n-1), one thread per index (the calling thread takes index 0).  The driver
// calls that pause and resume make per peer (unmap, release, import, map, set-access) are
// independent of one another, and with eight ranks they are most of the latency.
// AMEM_PR_THREADS=0 runs them in turn.
template <typename F>
void parallel_each(size_t n, F fn) {
  static const long on = env_long("AMEM_PR_THREADS", 1);
  if (n <= 1 || !on) {
    for (size_t i = 0; i < n; ++i) fn(i);
    return;
  }
  std::vector<std::thread> th;
  th.reserve(n - 1);
  for (size_t i = 1; i < n; ++i) th.emplace_back([&fn, i] { fn(i); });
  fn(0);
  for (auto& t : th) t.join();
}

// Result of one per-peer job; the error text lives in a thread-local slot, so it is carried
// back to the calling thread by hand.
struct JobResult {
  Status st = kSuccess;
  std::string err;
};
Status first_error(const std::vector<JobResult>& res) {
  for (const auto& r : res)
    if (r.st != kSuccess) {
      last_error_slot() = r.err;
      return r.st;
    }
  return kSuccess;
}

// Undo what one resume attempt built, so the scope is back in the PAUSED state.
void rollback_locals(Registry& reg, VmmBackend* be, std::vector<Allocation>& made) {
  for (auto& a : made) {
    if (a.mc_handle) be->mc_unbind(a.mc_handle, a.dev, a.mc_offset, a.size);
    be->unmap(a.va, a.size);
    be->release(a.handle);
    a.handle = 0;
    a.state = kMemHole;
    reg.update(a);
  }
  be->copies_sync(made.empty() ? 0 : made[0].dev);
  made.clear();
}

}  // namespace

Status pause_scope(Registry& reg, VmmBackend* be, uint64_t owner, int dev, PeerExchange* px,
                   const EngineOptions& opt, PauseResumeStats* st) {
  PauseResumeStats local;
  if (!st) st = &local;
  int rs = reg.owner_state(owner);
  if (rs == kRunPaused) return kSuccess;  // idempotent, like the reference (amem_nccl.cpp:481-488)
  st->quiesce_us = st->offload_us = st->release_import_us = st->release_local_us = st->pause_barrier_us = 0;
  st->bytes_offloaded = st->bytes_released_local = st->bytes_released_peer = 0;
  st->n_offload = st->n_release_local = st->n_release_peer = 0;
  double t_begin = now_ms();
  reg.set_owner_state(owner, kRunPausing);

  size_t free_b = 0, total_b = 0;
  be->mem_info(dev, &free_b, &total_b);
  st->free_before_pause = free_b;
  {
    Phase p("amem.pause.quiesce", &st->quiesce_us);
    AMEM_TRY(be->device_sync(dev));
  }
  std::vector<Allocation> recs = reg.snapshot(owner, false);

  {  // 1. start every host save; they run back to back on the side stream
    Phase p("amem.pause.offload", &st->offload_us);
    for (auto& a : recs) {
      if (!is_local(a) || a.state != kMemAlloc || a.category == kResident) continue;
      bool keep = a.category == kStateful && a.tag != opt.offload_free_tag;
      if (!keep) continue;
      if (!a.shadow) AMEM_TRY(be->host_alloc(a.size, &a.shadow));
      AMEM_TRY(be->copy_to_host_async(a.shadow, a.va, a.size, a.dev));
      a.state = kMemOffloading;
      reg.update(a);
      st->bytes_offloaded += a.size;
      st->n_offload++;
    }
  }
  {  // 2. let go of the peers' memory while the copies run (no data to save: the owner has it)
    Phase p("amem.pause.release_import", &st->release_import_us);
    std::vector<Allocation*> peers;
    for (auto& a : recs)
      if (!is_local(a) && a.state == kMemAlloc && a.category != kResident) peers.push_back(&a);
    std::vector<JobResult> res(peers.size());
    parallel_each(peers.size(), [&](size_t i) {
      Allocation& a = *peers[i];
      Status s = i ? be->thread_init(dev) : kSuccess;
      if (s == kSuccess) s = be->unmap(a.va, a.size);
      if (s == kSuccess) s = be->release(a.handle);
      res[i].st = s;
      if (s != kSuccess) res[i].err = last_error_slot();
    });
    for (size_t i = 0; i < peers.size(); ++i) {
      if (res[i].st != kSuccess) continue;
      Allocation& a = *peers[i];
      a.handle = 0;
      a.state = kMemHole;
      reg.update(a);
      st->bytes_released_peer += a.size;
      st->n_release_peer++;
    }
    AMEM_TRY(first_error(res));
  }
  {  // 3. saves done -> drop the local physical memory, keep the addresses
    Phase p("amem.pause.release_local", &st->release_local_us);
    AMEM_TRY(be->copies_sync(dev));
    for (auto& a : recs) {
      if (!is_local(a) || (a.state != kMemAlloc && a.state != kMemOffloading) || a.category == kResident) continue;
      if (a.mc_handle) AMEM_TRY(be->mc_unbind(a.mc_handle, a.dev, a.mc_offset, a.size));
      AMEM_TRY(be->unmap(a.va, a.size));
      AMEM_TRY(be->release(a.handle));
      a.handle = 0;
      a.state = kMemHole;
      reg.update(a);
      st->bytes_released_local += a.size;
      st->n_release_local++;
    }
  }
  if (px && opt.barrier) {  // 4. pages return to the driver only after the last importer released
    Phase p("amem.pause.barrier", &st->pause_barrier_us);
    AMEM_TRY(px->barrier());
  }
  reg.set_owner_state(owner, kRunPaused);
  if (st->n_release_local + st->n_release_peer > 0) reg.count_pause();  // empty scopes do not count
  be->mem_info(dev, &free_b, &total_b);
  st->free_after_pause = free_b;
  st->pause_total_us = (now_ms() - t_begin) * 1000.0;
  LOGD("pause owner:%#llx offloaded:%llu B in %llu copies, released local:%llu B (%llu) peer:%llu B (%llu), %.0f us",
       (unsigned long long)owner, (unsigned long long)st->bytes_offloaded, (unsigned long long)st->n_offload,
       (unsigned long long)st->bytes_released_local, (unsigned long long)st->n_release_local,
       (unsigned long long)st->bytes_released_peer, (unsigned long long)st->n_release_peer, st->pause_total_us);
  return kSuccess;
}

Status resume_scope(Registry& reg, VmmBackend* be, uint64_t owner, int dev, PeerExchange* px,
                    const EngineOptions& opt, PauseResumeStats* st) {
  PauseResumeStats local;
  if (!st) st = &local;
  if (reg.owner_state(owner) != kRunPaused) return kSuccess;  // idempotent
  st->create_map_us = st->agree_us = st->exchange_us = st->import_us = st->preload_us = st->resume_barrier_us = 0;
  st->bytes_preloaded = 0;
  double t_begin = now_ms();
  reg.set_owner_state(owner, kRunResuming);
  std::vector<Allocation> recs = reg.snapshot(owner, false);
  std::vector<Allocation> made;
  Status mine = kSuccess;

  {  // 1. new physical memory at the old addresses, restores queued behind it
    Phase p("amem.resume.create_map", &st->create_map_us);
    for (auto& a : recs) {
      if (!is_local(a) || a.state != kMemHole) continue;
      uint64_t h = 0;
      mine = be->create(a.dev, a.size, &h);
      if (mine != kSuccess) break;
      mine = be->map(a.va, a.size, h, a.dev);
      if (mine != kSuccess) {
        be->release(h);
        break;
      }
      if (a.mc_handle) {
        mine = be->mc_bind(a.mc_handle, a.mc_offset, h, a.size);
        if (mine != kSuccess) {
          be->unmap(a.va, a.size);
          be->release(h);
          break;
        }
      }
      a.handle = h;
      a.state = kMemPreloading;
      reg.update(a);
      made.push_back(a);
      bool restore = a.shadow && a.category == kStateful && a.tag != opt.offload_free_tag;
      if (restore) {
        mine = be->copy_to_device_async(a.va, a.shadow, a.size, a.dev);
        if (mine != kSuccess) break;
        st->bytes_preloaded += a.size;
      }
    }
  }
  std::string my_error = last_error_slot();
  {  // 2. either every rank got its memory or nobody resumes
    Phase p("amem.resume.agree", &st->agree_us);
    bool all = mine == kSuccess;
    if (px) {
      Status s = px->all_ok(mine == kSuccess, &all);
      if (s != kSuccess) all = false;
    }
    if (!all) {
      rollback_locals(reg, be, made);
      reg.set_owner_state(owner, kRunPaused);
      if (mine != kSuccess) {
        last_error_slot() = my_error;
        return mine;
      }
      return fail(kRemoteError, "resume rolled back: a peer could not re-create its memory");
    }
  }
  if (px) {
    {  // 3a. all sends first (small messages, they fit the socket buffers) ...
      Phase p("amem.resume.exchange", &st->exchange_us);
      int me = px->rank();
      for (auto& a : made) {
        uint32_t others = a.importers & ~(1u << me);
        if (!others) continue;
        int fd = -1;
        AMEM_TRY(be->export_fd(a.handle, &fd));
        Status s = kSuccess;
        for (int r = 0; r < px->nranks() && s == kSuccess; ++r)
          if (others & (1u << r)) s = px->send_fd(r, a.sym_id, a.size, fd);
        close(fd);
        AMEM_TRY(s);
      }
    }
    {  // 3b. ... then all receives, mapping each peer's memory where it used to be
      Phase p("amem.resume.import", &st->import_us);
      // the descriptors first, in record order (the peers sent them in that order) ...
      std::vector<Allocation*> holes;
      std::vector<int> fds;
      for (auto& a : recs) {
        if (is_local(a) || a.state != kMemHole) continue;
        uint32_t sym = 0;
        uint64_t sz = 0;
        int fd = -1;
        Status s = px->recv_fd(a.exporter_rank, &sym, &sz, &fd);
        if (s == kSuccess && (sym != a.sym_id || sz != a.size)) {
          if (fd >= 0) close(fd);
          fd = -1;
          s = fail(kInternalError, "resume: expected segment %u (%zu B) from rank %d, got %u (%llu B)", a.sym_id, a.size,
                   a.exporter_rank, sym, (unsigned long long)sz);
        }
        if (s != kSuccess) {
          for (int f : fds) close(f);
          return s;
        }
        holes.push_back(&a);
        fds.push_back(fd);
      }
      // ... then every peer's memory goes back where it used to be, side by side
      std::vector<JobResult> res(holes.size());
      parallel_each(holes.size(), [&](size_t i) {
        Allocation& a = *holes[i];
        uint64_t h = 0;
        Status s = i ? be->thread_init(dev) : kSuccess;
        if (s == kSuccess) s = be->import_fd(fds[i], a.size, &h);
        close(fds[i]);
        if (s == kSuccess) {
          s = be->map(a.va, a.size, h, a.dev);
          if (s != kSuccess) {
            std::string keep = last_error_slot();
            be->release(h);
            last_error_slot() = keep;
          }
        }
        res[i].st = s;
        if (s != kSuccess) res[i].err = last_error_slot();
        else a.handle = h;
      });
      for (size_t i = 0; i < holes.size(); ++i) {
        if (res[i].st != kSuccess) continue;
        holes[i]->state = kMemAlloc;
        reg.update(*holes[i]);
      }
      AMEM_TRY(first_error(res));
    }
  }
  {  // 4. contents are back
    Phase p("amem.resume.preload", &st->preload_us);
    AMEM_TRY(be->copies_sync(dev));
    for (auto& a : made) {
      a.state = kMemAlloc;
      reg.update(a);
    }
  }
  if (px && opt.barrier) {  // 5. nobody may signal into a peer whose restore is still running
    Phase p("amem.resume.barrier", &st->resume_barrier_us);
    AMEM_TRY(px->barrier());
  }
  reg.set_owner_state(owner, kRunResumed);
  if (!made.empty() || st->bytes_preloaded > 0) reg.count_resume();
  size_t free_b = 0, total_b = 0;
  be->mem_info(dev, &free_b, &total_b);
  st->free_after_resume = free_b;
  st->resume_total_us = (now_ms() - t_begin) * 1000.0;
  LOGD("resume owner:%#llx restored:%llu B, %.0f us", (unsigned long long)owner,
       (unsigned long long)st->bytes_preloaded, st->resume_total_us);
  return kSuccess;
}

}  // namespace amem
