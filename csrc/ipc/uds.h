// Unix-domain stream sockets with deadlines and file-descriptor passing.
//
// Replaces the reference's gmm_send/gmm_recv (amem_nccl_plugin/gmm_common_impl.cpp:341-434):
// fixed-size framed messages, an optional descriptor riding as SCM_RIGHTS ancillary data.
// Every blocking step takes a deadline and reports a timeout, a closed peer or a short
// frame as a Status instead of blocking for ever or aborting the process.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

#include "../core/status.h"

namespace amem {

struct Deadline {
  double end_ms;
  static Deadline after_ms(double ms);
  double remaining_ms() const;
  bool expired() const { return remaining_ms() <= 0; }
};

// One control-plane message.  `val`/`arg` meaning depends on `op`.
struct Frame {
  uint32_t magic;
  uint16_t op;
  uint16_t src;     // sender's rank in the communicator
  uint64_t comm;    // communicator id
  uint32_t seq;
  uint32_t arg;
  uint64_t val;
};
static const uint32_t kFrameMagic = 0x414d454d;  // "AMEM"

enum FrameOp : uint16_t {
  kOpHello = 1,      // bootstrap: rank introduces itself to the root / to a mesh peer
  kOpTable = 2,      // bootstrap: root publishes the gathered table
  kOpBlob = 3,       // all-gather of small host blobs
  kOpBarrier = 4,
  kOpVote = 5,       // all_ok agreement
  kOpFd = 6,         // a shareable handle: arg = segment id, val = size, fd attached
  kOpAbort = 7,
};

Status uds_listen(const std::string& path, int* listen_fd);
Status uds_accept(int listen_fd, Deadline dl, int* fd);
// Retries while the listener does not exist yet, until the deadline.
Status uds_connect(const std::string& path, Deadline dl, int* fd);
// Sends exactly `len` bytes; if pass_fd >= 0 it rides with the first byte.
Status uds_send(int fd, const void* buf, size_t len, int pass_fd, Deadline dl);
// Receives exactly `len` bytes; *got_fd is the descriptor that arrived with them or -1.
Status uds_recv(int fd, void* buf, size_t len, int* got_fd, Deadline dl);

// Host-side fault injection for tests: the nth next send (counted over the process) is
// "drop" (nothing is sent, success is reported), "short" (half the bytes are sent, then
// the socket is shut down), "nofd" (the descriptor is withheld) or "delay" (the send
// sleeps `param_ms` first).  nth <= 0 clears.
void uds_inject(const char* kind, int nth, int param_ms);

}  // namespace amem
