// Rank rendez-vous and the per-communicator socket mesh.
//
// The reference elects an "admin" by racing on bind(), publishes a multi-megabyte control
// block in POSIX shared memory and runs an admin thread plus a worker thread per rank
// (amem_nccl_plugin/gmm_singleton.h:40-70, gmm_server_impl.cpp:73-232,
// gmm_worker_impl.cpp:198-431).  Here the ncclUniqueId itself names the meeting point:
// it carries the socket directory, the group id and a nonce, so rank r listens on
// <dir>/amem_<gid>_<nonce>.<r> and connects to every lower rank.  The result is one
// persistent stream socket per pair of ranks, used synchronously by the thread that calls
// the communicator (no background threads, no shared-memory block, no polling sleeps).
#pragma once
#include <cstdint>
#include <mutex>
#include <string>
#include <vector>

#include "../vmm/pause_resume.h"
#include "uds.h"

namespace amem {

// Laid over the 128 bytes of ncclUniqueId.
struct UniqueId {
  uint32_t magic;
  int32_t group_id;
  uint64_t nonce;
  int32_t root_pid;
  char dir[108];
};
static_assert(sizeof(UniqueId) == 128, "UniqueId must fill ncclUniqueId exactly");

Status make_unique_id(UniqueId* out);

class Mesh : public PeerExchange {
 public:
  // Blocks until all `nranks` ranks have met or the init deadline (AMEM_INIT_TIMEOUT_MS,
  // default 120 s) passes.
  static Status connect(const UniqueId& id, int rank, int nranks, Mesh** out);
  ~Mesh() override;

  int rank() const override { return rank_; }
  int nranks() const override { return nranks_; }
  uint64_t comm_id() const { return comm_id_; }

  Status barrier() override;
  Status all_ok(bool mine, bool* all) override;
  Status barrier_begin() override;
  Status barrier_end() override;
  Status vote_begin(bool mine) override;
  Status vote_end(bool* all) override;
  Status send_fd(int to, uint32_t sym_id, uint64_t size, int fd) override;
  Status recv_fd(int from, uint32_t* sym_id, uint64_t* size, int* fd) override;
  Status send_no_fd(int to, uint32_t sym_id) override;
  void begin_attempt() override;

  // Every rank contributes `len` bytes (at most 16 KiB); `all` receives nranks * len.
  Status allgather(const void* mine, size_t len, void* all);
  // One message of `len` bytes (at most 16 KiB) to / from a single peer; nobody else takes part.
  Status send_blob(int to, const void* data, size_t len);
  Status recv_blob(int from, void* data, size_t len);
  // Closes every socket; peers see end-of-file on their next receive (ncclCommAbort).
  void shutdown_all();

 private:
  Mesh() {}
  Status send_frame(int to, uint16_t op, uint32_t arg, uint64_t val, int fd);
  Status recv_frame(int from, uint16_t op, Frame* f, int* fd);
  double op_timeout_ms_ = 30000;
  int rank_ = 0, nranks_ = 1;
  uint64_t comm_id_ = 0;
  uint32_t seq_ = 0;
  std::vector<int> socks_;  // socks_[peer], -1 for self
  // A frame of a LATER step that arrived where an earlier one was expected (the earlier one was
  // lost): kept here, with its descriptor, and handed to the receive that asks for it, so one
  // lost message fails one attempt instead of putting the whole stream out of step.
  std::vector<Frame> held_;
  std::vector<char> has_held_;
  std::vector<int> held_fd_;
  uint32_t epoch_ = 0;      // attempt number stamped on every frame sent
  std::mutex mu_;
};

}  // namespace amem
