#include "pause_resume.h"

#include <unistd.h>

#include <algorithm>
#include <atomic>
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

// Times one phase of the pass; the figure goes into every scope of the pass (the phases run
// once for all of them).
struct Phase {
  double t0;
  std::vector<double*> slots;
  explicit Phase(const char* name) : t0(now_ms()) { RANGE_PUSH(name); (void)name; }
  ~Phase() {
    RANGE_POP();
    double us = (now_ms() - t0) * 1000.0;
    for (double* s : slots)
      if (s) *s += us;
  }
};

bool is_local(const Allocation& a) { return !from_peer(a.type); }

// Runs fn(i, on_helper) for i in [0, n) on the calling thread plus up to seven helpers that take
// the next index from a shared counter.  The driver calls that pause and resume make per peer
// (unmap, release, import, map) are independent of one another.  AMEM_PR_THREADS=0 runs them in
// turn; any other value is the largest number of threads used (default 8).
template <typename F>
void parallel_each(size_t n, F fn) {
  static const long knob = env_long("AMEM_PR_THREADS", 8);
  size_t threads = knob <= 0 ? 1 : (knob == 1 ? 8 : (size_t)knob);
  if (threads > n) threads = n;
  if (threads <= 1) {
    for (size_t i = 0; i < n; ++i) fn(i, false);
    return;
  }
  std::atomic<size_t> next{0};
  auto worker = [&](bool helper) {
    for (;;) {
      size_t i = next.fetch_add(1);
      if (i >= n) break;
      fn(i, helper);
    }
  };
  std::vector<std::thread> th;
  th.reserve(threads - 1);
  for (size_t t = 1; t < threads; ++t) th.emplace_back([&worker] { worker(true); });
  worker(false);
  for (auto& t : th) t.join();
}

// Per-scope working state of one pass.
struct Work {
  EngineScope* sc = nullptr;
  std::vector<Allocation> recs;
  std::vector<Allocation> made;      // locals re-created by this resume attempt
  std::vector<size_t> mapped;        // indices into recs: imports mapped by this resume attempt
  Status st = kSuccess;              // first error of this scope
  std::string err;
  int prev_state = kRunInit;
  bool go = false;                   // resume: passed the first vote

  void note(Status s) {
    if (s != kSuccess && st == kSuccess) {
      st = s;
      err = last_error_slot();
    }
  }
  PauseResumeStats* stats() { return sc->stats; }
};

// Ring distance from this rank to the rank that owns an imported record (1 = right-hand neighbour).
int peer_distance(const Work& w, const Allocation& a) {
  if (!w.sc->px || a.exporter_rank < 0) return 0;
  const int n = w.sc->px->nranks();
  return (a.exporter_rank - w.sc->px->rank() + n) % n;
}

void add_slot(Phase& p, std::vector<Work>& ws, double PauseResumeStats::*field) {
  for (auto& w : ws)
    if (w.sc->stats) p.slots.push_back(&(w.sc->stats->*field));
}

std::vector<int> devices_of(const std::vector<Work>& ws) {
  std::vector<int> devs;
  for (auto& w : ws) {
    if (std::find(devs.begin(), devs.end(), w.sc->dev) == devs.end()) devs.push_back(w.sc->dev);
    for (auto& a : w.recs)
      if (std::find(devs.begin(), devs.end(), a.dev) == devs.end()) devs.push_back(a.dev);
  }
  return devs;
}

// Undo what one resume attempt built for a scope, so it is back in the PAUSED state.
void rollback(Registry& reg, VmmBackend* be, Work& w) {
  for (size_t i : w.mapped) {
    Allocation& a = w.recs[i];
    be->unmap(a.va, a.size);
    if (a.handle) be->release(a.handle);
    a.handle = 0;
    a.state = kMemHole;
    reg.update(a);
  }
  w.mapped.clear();
  if (!w.made.empty()) be->copies_sync(w.made[0].dev);  // no restore may still be writing into memory about to go
  for (auto& a : w.made) {
    if (a.mc_handle) be->mc_unbind(a.mc_handle, a.dev, a.mc_offset, a.size);
    be->unmap(a.va, a.size);
    be->release(a.handle);
    a.handle = 0;
    a.state = kMemHole;
    reg.update(a);
  }
  w.made.clear();
  reg.set_owner_state(w.sc->owner, kRunPaused);
}

Status finish(std::vector<Work>& ws) {
  for (auto& w : ws) w.sc->result = w.st;
  for (auto& w : ws)
    if (w.st != kSuccess) {
      last_error_slot() = w.err;
      return w.st;
    }
  return kSuccess;
}

}  // namespace

Status pause_scopes(Registry& reg, VmmBackend* be, std::vector<EngineScope>& scopes) {
  double t_begin = now_ms();
  std::vector<Work> ws;
  for (auto& sc : scopes) {
    sc.result = kSuccess;
    int rs = reg.owner_state(sc.owner);
    if (rs == kRunPaused) continue;  // idempotent, like the reference (amem_nccl.cpp:481-488)
    Work w;
    w.sc = &sc;
    w.prev_state = rs == kRunPausing || rs == kRunResuming ? kRunResumed : rs;
    if (sc.stats) {
      PauseResumeStats* st = sc.stats;
      st->quiesce_us = st->offload_us = st->release_import_us = st->release_local_us = st->pause_barrier_us = 0;
      st->bytes_offloaded = st->bytes_released_local = st->bytes_released_peer = 0;
      st->n_offload = st->n_release_local = st->n_release_peer = 0;
    }
    reg.set_owner_state(sc.owner, kRunPausing);
    if (sc.px) sc.px->begin_attempt();
    ws.push_back(std::move(w));
  }
  if (ws.empty()) return kSuccess;

  size_t free_b = 0, total_b = 0;
  be->mem_info(ws[0].sc->dev, &free_b, &total_b);
  for (auto& w : ws)
    if (w.stats()) w.stats()->free_before_pause = free_b;
  for (auto& w : ws) w.recs = reg.snapshot(w.sc->owner, false);
  std::vector<int> devs = devices_of(ws);

  Status early = kSuccess;
  {
    Phase p("amem.pause.quiesce");
    add_slot(p, ws, &PauseResumeStats::quiesce_us);
    for (int d : devs)
      if (early == kSuccess) early = be->device_sync(d);
  }
  if (early == kSuccess) {  // 1. start every host save; they run back to back on the side stream
    Phase p("amem.pause.offload");
    add_slot(p, ws, &PauseResumeStats::offload_us);
    for (auto& w : ws) {
      for (auto& a : w.recs) {
        if (early != kSuccess) break;
        if (!is_local(a) || a.state != kMemAlloc || a.category == kResident) continue;
        bool keep = a.category == kStateful && a.tag != w.sc->opt.offload_free_tag;
        if (!keep) continue;
        if (!a.shadow) early = be->host_alloc(a.size, &a.shadow);
        if (early == kSuccess) early = be->copy_to_host_async(a.shadow, a.va, a.size, a.dev);
        if (early != kSuccess) break;
        a.state = kMemOffloading;
        reg.update(a);
        if (w.stats()) {
          w.stats()->bytes_offloaded += a.size;
          w.stats()->n_offload++;
        }
      }
    }
  }
  if (early != kSuccess) {
    // Nothing has been released yet: put every record and every scope back as it was, so the
    // communicators stay usable and a later pause starts from a clean state.
    std::string why = last_error_slot();
    for (int d : devs) be->copies_sync(d);
    for (auto& w : ws) {
      for (auto& a : w.recs)
        if (a.state == kMemOffloading) {
          a.state = kMemAlloc;
          reg.update(a);
        }
      reg.set_owner_state(w.sc->owner, w.prev_state);
      w.st = early;
      w.err = why;
    }
    return finish(ws);
  }

  // From here on the pass goes to the end whatever fails: a scope that is half released is of
  // no use, one that is fully PAUSED (with the failure reported) can be resumed.
  {  // 2. let go of the peers' memory while the copies run (no data to save: the owner has it)
    Phase p("amem.pause.release_import");
    add_slot(p, ws, &PauseResumeStats::release_import_us);
    struct Job {
      Work* w;
      Allocation* a;
      Status st;
      std::string err;
    };
    std::vector<Job> jobs;
    for (auto& w : ws)
      for (auto& a : w.recs)
        if (!is_local(a) && a.state == kMemAlloc && a.category != kResident) jobs.push_back({&w, &a, kSuccess, ""});
    // every rank starts with a different peer (its right-hand neighbour), so that at any moment
    // the ranks' driver calls concern different GPUs' memory instead of all queueing on one
    std::stable_sort(jobs.begin(), jobs.end(), [](const Job& x, const Job& y) { return peer_distance(*x.w, *x.a) < peer_distance(*y.w, *y.a); });
    parallel_each(jobs.size(), [&](size_t i, bool helper) {
      Job& j = jobs[i];
      Status s = helper ? be->thread_init(j.a->dev) : kSuccess;
      if (s == kSuccess) s = be->unmap(j.a->va, j.a->size);
      if (s == kSuccess && j.a->handle) s = be->release(j.a->handle);   // (imports normally gave their handle back right after mapping)
      j.st = s;
      if (s != kSuccess) j.err = last_error_slot();
    });
    for (auto& j : jobs) {
      if (j.st != kSuccess) {
        last_error_slot() = j.err;
        j.w->note(j.st);
        continue;
      }
      j.a->handle = 0;
      j.a->state = kMemHole;
      reg.update(*j.a);
      if (j.w->stats()) {
        j.w->stats()->bytes_released_peer += j.a->size;
        j.w->stats()->n_release_peer++;
      }
    }
  }
  {  // 3. drop the local physical memory, keep the addresses: first what needs no save (it goes
     //    while the copies of the rest still run), then, once the saves are done, the rest
    Phase p("amem.pause.release_local");
    add_slot(p, ws, &PauseResumeStats::release_local_us);
    auto release_one = [&](Work& w, Allocation& a) {
      Status s = kSuccess;
      if (a.mc_handle) s = be->mc_unbind(a.mc_handle, a.dev, a.mc_offset, a.size);
      if (s == kSuccess) s = be->unmap(a.va, a.size);
      if (s == kSuccess) s = be->release(a.handle);
      if (s != kSuccess) {
        w.note(s);
        a.state = kMemAlloc;
        reg.update(a);
        return;
      }
      a.handle = 0;
      a.state = kMemHole;
      reg.update(a);
      if (w.stats()) {
        w.stats()->bytes_released_local += a.size;
        w.stats()->n_release_local++;
      }
    };
    for (auto& w : ws)
      for (auto& a : w.recs)
        if (is_local(a) && a.state == kMemAlloc && a.category != kResident) release_one(w, a);
    Status copies = kSuccess;
    std::string copies_err;
    for (int d : devs) {
      Status s = be->copies_sync(d);
      if (s != kSuccess && copies == kSuccess) {
        copies = s;
        copies_err = last_error_slot();
      }
    }
    for (auto& w : ws) {
      if (copies != kSuccess) {
        last_error_slot() = copies_err;
        w.note(copies);
      }
      for (auto& a : w.recs) {
        if (!is_local(a) || a.state != kMemOffloading) continue;
        if (copies != kSuccess) {  // its save did not finish: the memory stays
          a.state = kMemAlloc;
          reg.update(a);
          continue;
        }
        release_one(w, a);
      }
    }
  }
  {  // 4. pages return to the driver only after the last importer released
    Phase p("amem.pause.barrier");
    add_slot(p, ws, &PauseResumeStats::pause_barrier_us);
    for (auto& w : ws)
      if (w.sc->px && w.sc->opt.barrier) w.note(w.sc->px->barrier_begin());
    for (auto& w : ws)
      if (w.sc->px && w.sc->opt.barrier) w.note(w.sc->px->barrier_end());
  }
  be->mem_info(ws[0].sc->dev, &free_b, &total_b);
  bool counted = false;
  for (auto& w : ws) {
    reg.set_owner_state(w.sc->owner, kRunPaused);
    if (PauseResumeStats* st = w.stats()) {
      st->free_after_pause = free_b;
      st->pause_total_us = (now_ms() - t_begin) * 1000.0;
      if (!counted && st->n_release_local + st->n_release_peer > 0) {  // empty passes do not count
        reg.count_pause();
        counted = true;
      }
      LOGD("pause owner:%#llx offloaded:%llu B in %llu copies, released local:%llu B (%llu) peer:%llu B (%llu), %.0f us",
           (unsigned long long)w.sc->owner, (unsigned long long)st->bytes_offloaded, (unsigned long long)st->n_offload,
           (unsigned long long)st->bytes_released_local, (unsigned long long)st->n_release_local,
           (unsigned long long)st->bytes_released_peer, (unsigned long long)st->n_release_peer, st->pause_total_us);
    }
  }
  return finish(ws);
}

Status resume_scopes(Registry& reg, VmmBackend* be, std::vector<EngineScope>& scopes) {
  double t_begin = now_ms();
  std::vector<Work> ws;
  for (auto& sc : scopes) {
    sc.result = kSuccess;
    if (reg.owner_state(sc.owner) != kRunPaused) continue;  // idempotent
    Work w;
    w.sc = &sc;
    if (sc.stats) {
      PauseResumeStats* st = sc.stats;
      st->create_map_us = st->agree_us = st->exchange_us = st->import_us = st->preload_us = st->resume_barrier_us = 0;
      st->bytes_preloaded = 0;
    }
    reg.set_owner_state(sc.owner, kRunResuming);
    if (sc.px) sc.px->begin_attempt();
    w.recs = reg.snapshot(sc.owner, false);
    ws.push_back(std::move(w));
  }
  if (ws.empty()) return kSuccess;
  std::vector<int> devs = devices_of(ws);

  {  // 1. new physical memory at the old addresses, restores queued behind it
    Phase p("amem.resume.create_map");
    add_slot(p, ws, &PauseResumeStats::create_map_us);
    for (auto& w : ws) {
      Status mine = kSuccess;
      for (auto& a : w.recs) {
        if (!is_local(a) || a.state != kMemHole) continue;
        uint64_t h = 0;
        mine = be->create(a.dev, a.size, &h);
        if (mine != kSuccess) break;
        mine = be->map(a.va, a.size, h, a.dev);
        if (mine != kSuccess) {
          std::string keep = last_error_slot();
          be->release(h);
          last_error_slot() = keep;
          break;
        }
        if (a.mc_handle) {
          mine = be->mc_bind(a.mc_handle, a.mc_offset, h, a.size);
          if (mine != kSuccess) {
            std::string keep = last_error_slot();
            be->unmap(a.va, a.size);
            be->release(h);
            last_error_slot() = keep;
            break;
          }
        }
        a.handle = h;
        a.state = kMemPreloading;
        reg.update(a);
        w.made.push_back(a);
        if (a.clear_bytes) {  // queued on the side stream, finished before this rank votes in step 5
          mine = be->memset_zero(a.va + a.clear_offset, a.clear_bytes, a.dev);
          if (mine != kSuccess) break;
        }
        bool restore = a.shadow && a.category == kStateful && a.tag != w.sc->opt.offload_free_tag;
        if (restore) {
          mine = be->copy_to_device_async(a.va, a.shadow, a.size, a.dev);
          if (mine != kSuccess) break;
          if (w.stats()) w.stats()->bytes_preloaded += a.size;
        }
      }
      w.note(mine);
    }
  }
  {  // 2. per communicator: either every rank got its memory or nobody resumes
    Phase p("amem.resume.agree");
    add_slot(p, ws, &PauseResumeStats::agree_us);
    for (auto& w : ws)
      if (w.sc->px) w.sc->px->vote_begin(w.st == kSuccess);
    for (auto& w : ws) {
      bool all = w.st == kSuccess;
      if (w.sc->px) {
        Status s = w.sc->px->vote_end(&all);
        if (s != kSuccess) {
          all = false;
          w.note(s);
        }
      }
      w.go = all;
      if (!all) {
        if (w.st == kSuccess) {
          w.st = kRemoteError;
          w.err = "resume rolled back: a peer could not re-create its memory";
        }
        rollback(reg, be, w);
      }
    }
  }
  {  // 3a. all sends first (small messages, they fit the socket buffers) ...
    Phase p("amem.resume.exchange");
    add_slot(p, ws, &PauseResumeStats::exchange_us);
    for (auto& w : ws) {
      if (!w.go || !w.sc->px) continue;
      PeerExchange* px = w.sc->px;
      int me = px->rank();
      for (auto& a : w.made) {
        uint32_t others = a.importers & ~(1u << me);
        if (!others) continue;
        int fd = -1;
        Status s = be->export_fd(a.handle, &fd);
        w.note(s);
        for (int r = 0; r < px->nranks(); ++r) {
          if (!(others & (1u << r))) continue;
          // a peer always gets its message, so that the streams stay in step
          w.note(s == kSuccess ? px->send_fd(r, a.sym_id, a.size, fd) : px->send_no_fd(r, a.sym_id));
        }
        if (fd >= 0) close(fd);
      }
    }
  }
  {  // 3b. ... then all receives, mapping each peer's memory where it used to be
    Phase p("amem.resume.import");
    add_slot(p, ws, &PauseResumeStats::import_us);
    struct Job {
      Work* w;
      size_t idx;
      int fd;
      Status st;
      std::string err;
      uint64_t handle;
      bool needs_access;
    };
    std::vector<Job> jobs;
    // the descriptors first, in record order (the peers sent them in that order); every
    // expected message is taken off the socket even when an earlier one was bad
    for (auto& w : ws) {
      if (!w.go || !w.sc->px) continue;
      for (size_t i = 0; i < w.recs.size(); ++i) {
        Allocation& a = w.recs[i];
        if (is_local(a) || a.state != kMemHole) continue;
        uint32_t sym = 0;
        uint64_t sz = 0;
        int fd = -1;
        Status s = w.sc->px->recv_fd(a.exporter_rank, &sym, &sz, &fd);
        if (s == kSuccess && (sym != a.sym_id || sz != a.size)) {
          close(fd);
          fd = -1;
          s = fail(kInternalError, "resume: expected segment %u (%zu B) from rank %d, got %u (%llu B)", a.sym_id, a.size,
                   a.exporter_rank, sym, (unsigned long long)sz);
        }
        w.note(s);
        if (s == kSuccess) jobs.push_back({&w, i, fd, kSuccess, "", 0, false});
      }
    }
    // ... then every peer's memory goes back where it used to be; every rank starts with a
    // different peer (see pause)
    std::stable_sort(jobs.begin(), jobs.end(), [](const Job& x, const Job& y) {
      return peer_distance(*x.w, x.w->recs[x.idx]) < peer_distance(*y.w, y.w->recs[y.idx]);
    });
    parallel_each(jobs.size(), [&](size_t k, bool helper) {
      Job& j = jobs[k];
      Allocation& a = j.w->recs[j.idx];
      Status s = j.w->st;   // a scope that already failed only closes its descriptors
      if (s == kSuccess) {
        s = helper ? be->thread_init(a.dev) : kSuccess;
        if (s == kSuccess) s = be->import_fd(j.fd, a.size, &j.handle);
        if (s == kSuccess) {
          s = be->map_deferred(a.va, a.size, j.handle, a.dev, &j.needs_access);
          std::string keep = last_error_slot();
          be->release(j.handle);   // mapped or not, the handle is not needed again: the mapping holds the memory
          j.handle = 0;
          last_error_slot() = keep;
        }
        j.st = s;
        if (s != kSuccess) j.err = last_error_slot();
      } else {
        j.st = kInProgress;  // skipped
      }
      close(j.fd);
    });
    for (auto& j : jobs) {
      if (j.st == kInProgress) continue;
      if (j.st != kSuccess) {
        last_error_slot() = j.err;
        j.w->note(j.st);
        continue;
      }
      Allocation& a = j.w->recs[j.idx];
      a.handle = j.handle;
      a.state = kMemAlloc;
      reg.update(a);
      j.w->mapped.push_back(j.idx);
    }
    // access to everything just mapped: one call per run of adjacent mappings (a segment's
    // window is contiguous, so usually one call per segment instead of one per peer)
    for (auto& w : ws) {
      if (!w.go) continue;
      struct Run {
        uint64_t lo, hi;
        int dev;
        bool wanted;
      };
      std::vector<Run> runs;
      std::vector<const Allocation*> parts;
      for (auto& j : jobs)
        if (j.w == &w && j.st == kSuccess && j.needs_access) parts.push_back(&w.recs[j.idx]);
      if (parts.empty()) continue;
      std::vector<Run> all;
      for (const Allocation* a : parts) all.push_back({a->va, a->va + a->size, a->dev, true});
      for (auto& a : w.made) all.push_back({a.va, a.va + a.size, a.dev, false});  // already accessible; may bridge two runs
      std::sort(all.begin(), all.end(), [](const Run& x, const Run& y) { return x.lo < y.lo; });
      for (auto& r : all) {
        if (!runs.empty() && runs.back().hi == r.lo && runs.back().dev == r.dev) {
          runs.back().hi = r.hi;
          runs.back().wanted = runs.back().wanted || r.wanted;
        } else {
          runs.push_back(r);
        }
      }
      for (auto& r : runs)
        if (r.wanted) w.note(be->grant_access(r.lo, r.hi - r.lo, r.dev));
    }
  }
  {  // 4. contents are back
    Phase p("amem.resume.preload");
    add_slot(p, ws, &PauseResumeStats::preload_us);
    for (int d : devs) {
      Status s = be->copies_sync(d);
      if (s != kSuccess)
        for (auto& w : ws)
          if (w.go && w.sc->dev == d) w.note(s);
    }
  }
  {  // 5. second agreement: everybody's imports and restores went through, or everybody goes back to
     //    PAUSED.  It is also the closing barrier: a rank votes only once its restores have finished,
     //    so nobody signals into a peer whose memory is still being filled.
    Phase p("amem.resume.barrier");
    add_slot(p, ws, &PauseResumeStats::resume_barrier_us);
    // (a scope that failed the first agreement votes too: its peers, who may have gone on, then
    // learn of it at once instead of running into their deadline)
    for (auto& w : ws)
      if (w.sc->px) w.sc->px->vote_begin(w.go && w.st == kSuccess);
    for (auto& w : ws) {
      bool all = w.go && w.st == kSuccess;
      if (w.sc->px) {
        Status s = w.sc->px->vote_end(&all);
        if (s != kSuccess) {
          all = false;
          w.note(s);
        }
      }
      if (!w.go) continue;   // already rolled back
      if (!all) {
        if (w.st == kSuccess) {
          w.st = kRemoteError;
          w.err = "resume rolled back: a peer could not map or restore its memory";
        }
        rollback(reg, be, w);
        w.go = false;
      }
    }
  }
  size_t free_b = 0, total_b = 0;
  be->mem_info(ws[0].sc->dev, &free_b, &total_b);
  bool counted = false;
  for (auto& w : ws) {
    if (!w.go) continue;
    for (auto& a : w.made) {
      a.state = kMemAlloc;
      reg.update(a);
    }
    reg.set_owner_state(w.sc->owner, kRunResumed);
    if (!counted && (!w.made.empty() || (w.stats() && w.stats()->bytes_preloaded > 0))) {
      reg.count_resume();
      counted = true;
    }
    if (PauseResumeStats* st = w.stats()) {
      st->free_after_resume = free_b;
      st->resume_total_us = (now_ms() - t_begin) * 1000.0;
      LOGD("resume owner:%#llx restored:%llu B, %.0f us", (unsigned long long)w.sc->owner, (unsigned long long)st->bytes_preloaded,
           st->resume_total_us);
    }
  }
  return finish(ws);
}

Status pause_scope(Registry& reg, VmmBackend* be, uint64_t owner, int dev, PeerExchange* px, const EngineOptions& opt,
                   PauseResumeStats* st) {
  std::vector<EngineScope> one(1);
  one[0].owner = owner;
  one[0].dev = dev;
  one[0].px = px;
  one[0].opt = opt;
  one[0].stats = st;
  return pause_scopes(reg, be, one);
}

Status resume_scope(Registry& reg, VmmBackend* be, uint64_t owner, int dev, PeerExchange* px, const EngineOptions& opt,
                    PauseResumeStats* st) {
  std::vector<EngineScope> one(1);
  one[0].owner = owner;
  one[0].dev = dev;
  one[0].px = px;
  one[0].opt = opt;
  one[0].stats = st;
  return resume_scopes(reg, be, one);
}

}  // namespace amem
