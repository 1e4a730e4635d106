// Reference parity: replaces the admin thread + shared-memory directory + lock file of the reference
// (amem_nccl_plugin/gmm_server_impl.cpp:95-101, gmm_common.h:418-473) by socket names derived from
// the ncclUniqueId.
#include "rendezvous.h"

#include <fcntl.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <random>

#include "../core/log.h"
#include "../vmm/registry.h"

namespace amem {

static const uint32_t kIdMagic = 0x42323030;  // "B200"

Status make_unique_id(UniqueId* out) {
  memset(out, 0, sizeof(*out));
  out->magic = kIdMagic;
  out->group_id = Registry::instance().group_id();
  static std::atomic<uint64_t> counter{0};
  uint64_t nonce = 0;
  int fd = open("/dev/urandom", O_RDONLY | O_CLOEXEC);
  if (fd >= 0) {
    ssize_t r = read(fd, &nonce, sizeof(nonce));
    (void)r;
    close(fd);
  }
  nonce ^= ((uint64_t)getpid() << 32) ^ (uint64_t)(now_ms() * 1000.0) ^ (counter.fetch_add(1) << 20);
  out->nonce = nonce;
  out->root_pid = (int32_t)getpid();
  std::string dir = env_str("GMM_IPC_DIR", "/tmp");
  if (dir.size() >= sizeof(out->dir) - 40) return fail(kInvalidArgument, "GMM_IPC_DIR is too long for a socket path: %s", dir.c_str());
  memcpy(out->dir, dir.c_str(), dir.size());
  return kSuccess;
}

static std::string sock_path(const UniqueId& id, int rank) {
  char buf[256];
  // Names carry the group id so co-located groups never touch each other's files.
  snprintf(buf, sizeof(buf), "%s/amem_%x_%llx.%d", id.dir, (unsigned)id.group_id, (unsigned long long)id.nonce, rank);
  return buf;
}

Status Mesh::connect(const UniqueId& id, int rank, int nranks, Mesh** out) {
  if (id.magic != kIdMagic) return fail(kInvalidArgument, "unique id was not produced by ncclGetUniqueId of this library");
  if (nranks < 1 || rank < 0 || rank >= nranks) return fail(kInvalidArgument, "rank %d of %d", rank, nranks);
  if (nranks > 32) return fail(kInvalidArgument, "at most 32 ranks per communicator (one NVLink domain)");
  Mesh* m = new Mesh();
  m->rank_ = rank;
  m->nranks_ = nranks;
  m->comm_id_ = id.nonce | 1;  // never 0: owner 0 means "process level" in the registry
  m->op_timeout_ms_ = (double)env_long("AMEM_OP_TIMEOUT_MS", 30000);
  m->socks_.assign(nranks, -1);
  m->held_.assign(nranks, Frame{});
  m->has_held_.assign(nranks, 0);
  m->held_fd_.assign(nranks, -1);
  if (nranks == 1) {
    *out = m;
    return kSuccess;
  }
  Deadline dl = Deadline::after_ms((double)env_long("AMEM_INIT_TIMEOUT_MS", 120000));
  std::string mine = sock_path(id, rank);
  int lfd = -1;
  Status st = kSuccess;
  bool listening = rank < nranks - 1;  // the last rank only connects
  if (listening) st = uds_listen(mine, &lfd);
  // Connect downwards ...
  for (int p = 0; p < rank && st == kSuccess; ++p) {
    int fd = -1;
    st = uds_connect(sock_path(id, p), dl, &fd);
    if (st != kSuccess) break;
    m->socks_[p] = fd;
    Frame f{kFrameMagic, kOpHello, (uint16_t)rank, m->comm_id_, 0, (uint32_t)nranks, (uint64_t)getpid()};
    st = uds_send(fd, &f, sizeof(f), -1, dl);
  }
  // ... and accept from above; the hello frame says who called.
  for (int k = rank + 1; k < nranks && st == kSuccess; ++k) {
    int fd = -1;
    st = uds_accept(lfd, dl, &fd);
    if (st != kSuccess) break;
    Frame f;
    st = uds_recv(fd, &f, sizeof(f), nullptr, dl);
    if (st == kSuccess && (f.magic != kFrameMagic || f.op != kOpHello || f.comm != m->comm_id_ || f.src <= rank ||
                           f.src >= nranks || (int)f.arg != nranks || m->socks_[f.src] != -1)) {
      st = fail(kInternalError, "rendezvous: unexpected hello (op %u from rank %u, %u ranks)", f.op, f.src, f.arg);
    }
    if (st != kSuccess) {
      close(fd);
      break;
    }
    m->socks_[f.src] = fd;
  }
  if (lfd >= 0) {
    close(lfd);
    unlink(mine.c_str());
  }
  if (st == kSuccess) st = m->barrier();
  if (st != kSuccess) {
    std::string keep = last_error_slot();
    delete m;
    last_error_slot() = keep;
    return st;
  }
  *out = m;
  return kSuccess;
}

Mesh::~Mesh() { shutdown_all(); }

void Mesh::shutdown_all() {
  std::lock_guard<std::mutex> g(mu_);
  for (int& h : held_fd_) {
    if (h >= 0) close(h);
    h = -1;
  }
  for (int& s : socks_) {
    if (s >= 0) close(s);
    s = -1;
  }
}

Status Mesh::send_frame(int to, uint16_t op, uint32_t arg, uint64_t val, int fd) {
  if (to < 0 || to >= nranks_ || socks_[to] < 0) return fail(kRemoteError, "no connection to rank %d", to);
  Frame f{kFrameMagic, op, (uint16_t)rank_, comm_id_, epoch_, arg, val};
  Status st = uds_send(socks_[to], &f, sizeof(f), fd, Deadline::after_ms(op_timeout_ms_));
  if (st != kSuccess) LOGW("rank %d: send op %u to rank %d failed: %s", rank_, op, to, last_error_slot().c_str());
  return st;
}

void Mesh::begin_attempt() {
  std::lock_guard<std::mutex> g(mu_);
  ++epoch_;
}

// Frames carry the sender's attempt number (one per pause or resume pass; every rank makes the
// same sequence of passes).  A frame of an earlier attempt is what a failed attempt left in the
// socket: it is discarded.  A frame of this attempt with another op, or of a later attempt, means
// the message asked for was lost: the frame is kept for the receive that will ask for it, and this
// receive fails at once.  So one lost message fails one attempt; the next attempt starts clean.
Status Mesh::recv_frame(int from, uint16_t op, Frame* f, int* fd) {
  if (from < 0 || from >= nranks_ || socks_[from] < 0) return fail(kRemoteError, "no connection to rank %d", from);
  if (fd) *fd = -1;
  Deadline dl = Deadline::after_ms(op_timeout_ms_);
  for (;;) {
    int got = -1;
    if (has_held_[from]) {
      Frame& h = held_[from];
      if (h.seq < epoch_) {          // left over from an abandoned attempt
        if (held_fd_[from] >= 0) close(held_fd_[from]);
        held_fd_[from] = -1;
        has_held_[from] = 0;
        continue;
      }
      if (h.seq == epoch_ && h.op == op) {
        *f = h;
        got = held_fd_[from];
        held_fd_[from] = -1;
        has_held_[from] = 0;
        if (fd) *fd = got;
        else if (got >= 0) close(got);
        return kSuccess;
      }
      return fail(kRemoteError, "rank %d: the op %u message of rank %d never arrived (its op %u message of attempt %u is already here)",
                  rank_, op, from, h.op, h.seq);
    }
    Status st = uds_recv(socks_[from], f, sizeof(*f), &got, dl);
    if (st != kSuccess) {
      std::string why = last_error_slot();
      return fail(st, "rank %d waiting for op %u from rank %d: %s", rank_, op, from, why.c_str());
    }
    if (f->magic != kFrameMagic || f->comm != comm_id_ || f->src != from) {
      if (got >= 0) close(got);
      return fail(kInternalError, "rank %d: corrupt frame from rank %d", rank_, from);
    }
    if (f->op == kOpAbort) {
      if (got >= 0) close(got);
      return fail(kRemoteError, "rank %d aborted the communicator", from);
    }
    if (f->seq < epoch_) {           // stale: drop it and read on
      if (got >= 0) close(got);
      continue;
    }
    if (f->seq == epoch_ && f->op == op) {
      if (fd) *fd = got;
      else if (got >= 0) close(got);
      return kSuccess;
    }
    held_[from] = *f;
    held_fd_[from] = got;
    has_held_[from] = 1;
    return fail(kRemoteError, "rank %d: expected op %u from rank %d in attempt %u, got op %u of attempt %u (a message was lost)", rank_, op,
                from, epoch_, f->op, f->seq);
  }
}

Status Mesh::barrier_begin() {
  std::lock_guard<std::mutex> g(mu_);
  ++seq_;
  Status first = kSuccess;
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) continue;
    Status s = send_frame(p, kOpBarrier, 0, 0, -1);   // every peer gets its frame even if one send fails
    if (s != kSuccess && first == kSuccess) first = s;
  }
  return first;
}

Status Mesh::barrier_end() {
  std::lock_guard<std::mutex> g(mu_);
  Status first = kSuccess;
  std::string why;
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) continue;
    Frame f;
    Status s = recv_frame(p, kOpBarrier, &f, nullptr);
    if (s != kSuccess && first == kSuccess) {
      first = s;
      why = last_error_slot();
    }
  }
  if (first != kSuccess) last_error_slot() = why;
  return first;
}

Status Mesh::barrier() {
  AMEM_TRY(barrier_begin());
  return barrier_end();
}

Status Mesh::vote_begin(bool mine) {
  std::lock_guard<std::mutex> g(mu_);
  ++seq_;
  pending_vote_ = mine;
  Status first = kSuccess;
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) continue;
    Status s = send_frame(p, kOpVote, mine ? 1 : 0, 0, -1);
    if (s != kSuccess && first == kSuccess) first = s;
  }
  return first;
}

Status Mesh::vote_end(bool* all) {
  std::lock_guard<std::mutex> g(mu_);
  bool acc = pending_vote_;
  Status first = kSuccess;
  std::string why;
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) continue;
    Frame f;
    Status s = recv_frame(p, kOpVote, &f, nullptr);
    if (s != kSuccess) {
      if (first == kSuccess) {
        first = s;
        why = last_error_slot();
      }
      acc = false;
      continue;
    }
    acc = acc && f.arg != 0;
  }
  *all = acc;
  if (first != kSuccess) last_error_slot() = why;
  return first;
}

Status Mesh::all_ok(bool mine, bool* all) {
  Status s = vote_begin(mine);
  Status e = vote_end(all);
  return s != kSuccess ? s : e;
}

Status Mesh::send_fd(int to, uint32_t sym_id, uint64_t size, int fd) {
  std::lock_guard<std::mutex> g(mu_);
  return send_frame(to, kOpFd, sym_id, size, fd);
}

Status Mesh::send_no_fd(int to, uint32_t sym_id) {
  std::lock_guard<std::mutex> g(mu_);
  return send_frame(to, kOpFd, sym_id, ~0ull, -1);
}

Status Mesh::recv_fd(int from, uint32_t* sym_id, uint64_t* size, int* fd) {
  std::lock_guard<std::mutex> g(mu_);
  Frame f;
  int got = -1;
  AMEM_TRY(recv_frame(from, kOpFd, &f, &got));
  if (f.val == ~0ull) {
    if (got >= 0) close(got);
    return fail(kRemoteError, "rank %d could not export its segment %u", from, f.arg);
  }
  if (got < 0) return fail(kSystemError, "rank %d: handle message from rank %d carried no file descriptor", rank_, from);
  *sym_id = f.arg;
  *size = f.val;
  *fd = got;
  return kSuccess;
}

Status Mesh::send_blob(int to, const void* data, size_t len) {
  if (len > 16384) return fail(kInvalidArgument, "control-plane messages are limited to 16 KiB");
  if (to < 0 || to >= nranks_ || to == rank_) return fail(kInvalidArgument, "send_blob: bad peer %d", to);
  std::lock_guard<std::mutex> g(mu_);
  Deadline dl = Deadline::after_ms(op_timeout_ms_);
  AMEM_TRY(send_frame(to, kOpBlob, (uint32_t)len, 0, -1));
  if (len) AMEM_TRY(uds_send(socks_[to], data, len, -1, dl));
  return kSuccess;
}

Status Mesh::recv_blob(int from, void* data, size_t len) {
  if (from < 0 || from >= nranks_ || from == rank_) return fail(kInvalidArgument, "recv_blob: bad peer %d", from);
  std::lock_guard<std::mutex> g(mu_);
  Deadline dl = Deadline::after_ms(op_timeout_ms_);
  Frame f;
  AMEM_TRY(recv_frame(from, kOpBlob, &f, nullptr));
  if (f.arg != len) return fail(kInternalError, "rank %d sent %u bytes, expected %zu", from, f.arg, len);
  if (len) AMEM_TRY(uds_recv(socks_[from], data, len, nullptr, dl));
  return kSuccess;
}

Status Mesh::allgather(const void* mine, size_t len, void* all) {
  if (len > 16384) return fail(kInvalidArgument, "control-plane all-gather is limited to 16 KiB per rank");
  std::lock_guard<std::mutex> g(mu_);
  ++seq_;
  memcpy((char*)all + (size_t)rank_ * len, mine, len);
  Deadline dl = Deadline::after_ms(op_timeout_ms_);
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) continue;
    AMEM_TRY(send_frame(p, kOpBlob, (uint32_t)len, 0, -1));
    if (len) AMEM_TRY(uds_send(socks_[p], mine, len, -1, dl));
  }
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) continue;
    Frame f;
    AMEM_TRY(recv_frame(p, kOpBlob, &f, nullptr));
    if (f.arg != len) return fail(kInternalError, "all-gather: rank %d sent %u bytes, expected %zu", p, f.arg, len);
    if (len) AMEM_TRY(uds_recv(socks_[p], (char*)all + (size_t)p * len, len, nullptr, dl));
  }
  return kSuccess;
}

}  // namespace amem
