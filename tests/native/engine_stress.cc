// Host-only stress driver for the pause / resume engine, built with -fsanitize=thread or
// -fsanitize=address,undefined by tests/test_cpu_sanitizers.py (no CUDA needed: it links the
// registry, the mock VMM backend, the Unix-socket mesh and the engine only).
//
// N ranks run as threads of one process.  Each rank owns a "control" segment (STATEFUL) and a
// "staging" segment (SCRATCH), hands both to every peer as file descriptors over the mesh, maps
// the peers' segments, and then cycles: write a pattern, pause (everything is unmapped and
// released, stateful contents go to a host shadow), check that the memory is gone, resume
// (same addresses, peers re-import), check the contents and write through a peer mapping.
// The reference has no such test: its tables are mutated from a worker thread without a lock
// (amem_nccl_plugin/amem_nccl.cpp:303,365,391), which is exactly what this run is meant to catch
// in the rebuild.
#include <unistd.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "../../csrc/core/log.h"
#include "../../csrc/ipc/rendezvous.h"
#include "../../csrc/vmm/backend.h"
#include "../../csrc/vmm/pause_resume.h"
#include "../../csrc/vmm/registry.h"

namespace amem {
// The CUDA backend is not linked into this binary.
VmmBackend* cuda_backend() { return nullptr; }
VmmBackend* default_backend() { return mock_backend(); }
}  // namespace amem

using namespace amem;

static std::atomic<int> g_failures{0};
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) {                                         \
      fprintf(stderr, "CHECK failed %s:%d: ", __FILE__, __LINE__); \
      fprintf(stderr, __VA_ARGS__);                        \
      fprintf(stderr, " (%s)\n", last_error_slot().c_str()); \
      g_failures.fetch_add(1);                             \
      return;                                              \
    }                                                      \
  } while (0)

static const size_t kCtrlBytes = 2u << 20, kStageBytes = 8u << 20;

struct Segment {
  uint64_t va[8];  // va[r]: where rank r's segment is mapped in this rank
};

static void rank_main(const UniqueId& uid, int rank, int n, int cycles) {
  VmmBackend* be = mock_backend();
  Registry& reg = Registry::instance();
  Mesh* mesh = nullptr;
  CHECK(Mesh::connect(uid, rank, n, &mesh) == kSuccess, "rank %d: mesh", rank);
  const uint64_t owner = mesh->comm_id() + 2 * (uint64_t)rank + 1;
  Segment seg[2];
  const size_t bytes[2] = {kCtrlBytes, kStageBytes};
  const int category[2] = {kStateful, kScratch};
  for (int s = 0; s < 2; ++s) {
    // my own memory
    uint64_t h = 0;
    CHECK(be->reserve(bytes[s], 0, &seg[s].va[rank]) == kSuccess, "reserve");
    CHECK(be->create(0, bytes[s], &h) == kSuccess, "create");
    CHECK(be->map(seg[s].va[rank], bytes[s], h, 0) == kSuccess, "map");
    Allocation a;
    a.va = seg[s].va[rank];
    a.size = bytes[s];
    a.handle = h;
    a.type = kLocalPosix;
    a.category = category[s];
    a.tag = kTagP2P;
    a.owner = owner;
    a.sym_id = (uint32_t)s;
    a.exporter_rank = rank;
    a.importers = (1u << n) - 1;
    a.state = kMemAlloc;
    CHECK(reg.add(a) == kSuccess, "registry add");
    // hand it to every peer, take theirs
    int fd = -1;
    CHECK(be->export_fd(h, &fd) == kSuccess, "export");
    for (int p = 0; p < n; ++p)
      if (p != rank) CHECK(mesh->send_fd(p, (uint32_t)s, bytes[s], fd) == kSuccess, "send fd");
    close(fd);
    for (int p = 0; p < n; ++p) {
      if (p == rank) continue;
      uint32_t sym = 0;
      uint64_t sz = 0;
      int pfd = -1;
      CHECK(mesh->recv_fd(p, &sym, &sz, &pfd) == kSuccess && sym == (uint32_t)s && sz == bytes[s], "recv fd");
      uint64_t ph = 0;
      CHECK(be->import_fd(pfd, bytes[s], &ph) == kSuccess, "import");
      close(pfd);
      CHECK(be->reserve(bytes[s], 0, &seg[s].va[p]) == kSuccess, "reserve peer");
      CHECK(be->map(seg[s].va[p], bytes[s], ph, 0) == kSuccess, "map peer");
      Allocation b = a;
      b.va = seg[s].va[p];
      b.handle = ph;
      b.type = kPeerPosix;
      b.tag = kTagP2PPeer;
      b.exporter_rank = p;
      b.importers = 0;
      CHECK(reg.add(b) == kSuccess, "registry add peer");
    }
  }
  CHECK(mesh->barrier() == kSuccess, "barrier");
  EngineOptions opt;
  PauseResumeStats st;
  volatile uint32_t* my_ctrl = (volatile uint32_t*)seg[0].va[rank];
  for (int c = 0; c < cycles; ++c) {
    for (size_t i = 0; i < kCtrlBytes / 4; i += 1024) my_ctrl[i] = (uint32_t)(rank * 1000003 + c * 7 + i);
    // a word in every peer's staging, through the imported mapping
    for (int p = 0; p < n; ++p)
      if (p != rank) ((volatile uint32_t*)seg[1].va[p])[rank * 16] = (uint32_t)(c + 1);
    CHECK(mesh->barrier() == kSuccess, "barrier before pause");
    const size_t live_before = be->live_physical_bytes();
    CHECK(pause_scope(reg, be, owner, 0, mesh, opt, &st) == kSuccess, "pause cycle %d", c);
    CHECK(st.n_release_local == 2 && (int)st.n_release_peer == 2 * (n - 1), "pause released %llu local %llu peer",
          (unsigned long long)st.n_release_local, (unsigned long long)st.n_release_peer);
    CHECK(st.bytes_offloaded == kCtrlBytes, "only the stateful segment is saved (%llu B)", (unsigned long long)st.bytes_offloaded);
    (void)live_before;
    // the registry and memory statistics may be read by anybody while others pause or resume
    MemStats ms;
    reg.stats(&ms);
    CHECK(resume_scope(reg, be, owner, 0, mesh, opt, &st) == kSuccess, "resume cycle %d", c);
    for (size_t i = 0; i < kCtrlBytes / 4; i += 1024)
      CHECK(my_ctrl[i] == (uint32_t)(rank * 1000003 + c * 7 + i), "rank %d cycle %d: control word %zu lost", rank, c, i);
    // peers reach my staging again at the same address
    for (int p = 0; p < n; ++p)
      if (p != rank) ((volatile uint32_t*)seg[1].va[p])[rank * 16 + 1] = (uint32_t)(0xabc00000u + c);
    CHECK(mesh->barrier() == kSuccess, "barrier after resume");
    for (int p = 0; p < n; ++p)
      if (p != rank)
        CHECK(((volatile uint32_t*)seg[1].va[rank])[p * 16 + 1] == (uint32_t)(0xabc00000u + c), "rank %d cycle %d: peer %d's store did not land", rank, c, p);
    CHECK(mesh->barrier() == kSuccess, "barrier end of cycle");
  }
  // tear down
  for (int s = 0; s < 2; ++s)
    for (int p = 0; p < n; ++p) {
      Allocation a;
      CHECK(reg.find(seg[s].va[p], &a), "record missing");
      be->unmap(a.va, a.size);
      be->release(a.handle);
      if (a.shadow) be->host_free(a.shadow, a.size);
      reg.remove(a.va);
      be->free_va(a.va, a.size);
    }
  reg.forget_owner(owner);
  mesh->barrier();
  delete mesh;
}

int main(int argc, char** argv) {
  int n = argc > 1 ? atoi(argv[1]) : 3, cycles = argc > 2 ? atoi(argv[2]) : 20;
  setenv("AMEM_BACKEND", "mock", 1);
  UniqueId uid;
  if (make_unique_id(&uid) != kSuccess) {
    fprintf(stderr, "make_unique_id failed: %s\n", last_error_slot().c_str());
    return 2;
  }
  std::vector<std::thread> th;
  for (int r = 0; r < n; ++r) th.emplace_back(rank_main, uid, r, n, cycles);
  for (auto& t : th) t.join();
  size_t leaked = mock_backend()->live_physical_bytes();
  if (leaked) {
    fprintf(stderr, "leak: %zu bytes of physical memory still held\n", leaked);
    return 3;
  }
  if (g_failures.load()) return 1;
  printf("engine stress ok: %d ranks x %d cycles\n", n, cycles);
  return 0;
}
