// Reference parity: the framing and SCM_RIGHTS passing of amem_nccl_plugin/gmm_common_impl.cpp:341-434
// (one fixed-size request per message, one descriptor as ancillary data), with deadlines added.
#include "uds.h"

#include <fcntl.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <cstring>
#include <mutex>

#include "../core/log.h"

namespace amem {

Deadline Deadline::after_ms(double ms) { return Deadline{now_ms() + ms}; }
double Deadline::remaining_ms() const { return end_ms - now_ms(); }

namespace {

struct Inject {
  std::mutex mu;
  int drop = 0, shrt = 0, nofd = 0, delay = 0, delay_ms = 0;
} g_inj;

// Returns true once when the countdown of `slot` reaches zero.
bool fire(int* slot) {
  if (*slot <= 0) return false;
  if (--*slot == 0) return true;
  return false;
}

Status fill_addr(const std::string& path, sockaddr_un* sa) {
  memset(sa, 0, sizeof(*sa));
  sa->sun_family = AF_UNIX;
  if (path.size() >= sizeof(sa->sun_path)) return fail(kInvalidArgument, "socket path too long (%zu): %s", path.size(), path.c_str());
  memcpy(sa->sun_path, path.c_str(), path.size());
  return kSuccess;
}

Status wait_fd(int fd, short events, Deadline dl, const char* what) {
  for (;;) {
    double rem = dl.remaining_ms();
    if (rem <= 0) return fail(kSystemError, "%s: timed out", what);
    pollfd p{fd, events, 0};
    int r = poll(&p, 1, (int)(rem < 1 ? 1 : (rem > 1000 ? 1000 : rem)));
    if (r < 0) {
      if (errno == EINTR) continue;
      return fail(kSystemError, "%s: poll: %s", what, strerror(errno));
    }
    if (r == 0) continue;
    if (p.revents & (events | POLLHUP | POLLERR)) return kSuccess;
  }
}

}  // namespace

void uds_inject(const char* kind, int nth, int param_ms) {
  std::lock_guard<std::mutex> g(g_inj.mu);
  if (!strcmp(kind, "drop")) g_inj.drop = nth;
  else if (!strcmp(kind, "short")) g_inj.shrt = nth;
  else if (!strcmp(kind, "nofd")) g_inj.nofd = nth;
  else if (!strcmp(kind, "delay")) {
    g_inj.delay = nth;
    g_inj.delay_ms = param_ms;
  } else if (!strcmp(kind, "clear")) {
    g_inj.drop = g_inj.shrt = g_inj.nofd = g_inj.delay = 0;
  }
}

Status uds_listen(const std::string& path, int* listen_fd) {
  sockaddr_un sa;
  AMEM_TRY(fill_addr(path, &sa));
  int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return fail(kSystemError, "socket: %s", strerror(errno));
  unlink(path.c_str());
  if (bind(fd, (sockaddr*)&sa, sizeof(sa)) != 0) {
    int e = errno;
    close(fd);
    return fail(kSystemError, "bind %s: %s", path.c_str(), strerror(e));
  }
  if (listen(fd, 64) != 0) {
    int e = errno;
    close(fd);
    return fail(kSystemError, "listen %s: %s", path.c_str(), strerror(e));
  }
  *listen_fd = fd;
  return kSuccess;
}

Status uds_accept(int listen_fd, Deadline dl, int* fd) {
  for (;;) {
    AMEM_TRY(wait_fd(listen_fd, POLLIN, dl, "accept"));
    int c = accept4(listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
    if (c >= 0) {
      *fd = c;
      return kSuccess;
    }
    if (errno == EINTR || errno == EAGAIN) continue;
    return fail(kSystemError, "accept: %s", strerror(errno));
  }
}

Status uds_connect(const std::string& path, Deadline dl, int* fd) {
  sockaddr_un sa;
  AMEM_TRY(fill_addr(path, &sa));
  int backoff_us = 200;
  for (;;) {
    int c = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (c < 0) return fail(kSystemError, "socket: %s", strerror(errno));
    if (connect(c, (sockaddr*)&sa, sizeof(sa)) == 0) {
      *fd = c;
      return kSuccess;
    }
    int e = errno;
    close(c);
    if (e != ENOENT && e != ECONNREFUSED && e != EAGAIN && e != EINTR)
      return fail(kSystemError, "connect %s: %s", path.c_str(), strerror(e));
    if (dl.expired()) return fail(kSystemError, "connect %s: timed out (%s)", path.c_str(), strerror(e));
    usleep(backoff_us);
    if (backoff_us < 20000) backoff_us *= 2;
  }
}

Status uds_send(int fd, const void* buf, size_t len, int pass_fd, Deadline dl) {
  bool drop, shrt, nofd, delay;
  int delay_ms;
  {
    std::lock_guard<std::mutex> g(g_inj.mu);
    drop = fire(&g_inj.drop);
    shrt = !drop && fire(&g_inj.shrt);
    nofd = pass_fd >= 0 && fire(&g_inj.nofd);
    delay = fire(&g_inj.delay);
    delay_ms = g_inj.delay_ms;
  }
  if (delay) usleep((useconds_t)delay_ms * 1000);
  if (drop) return kSuccess;
  if (nofd) pass_fd = -1;
  size_t want = shrt ? len / 2 : len;
  const char* p = (const char*)buf;
  size_t done = 0;
  while (done < want) {
    AMEM_TRY(wait_fd(fd, POLLOUT, dl, "send"));
    msghdr msg;
    memset(&msg, 0, sizeof(msg));
    iovec iov{(void*)(p + done), want - done};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int))];
    if (pass_fd >= 0 && done == 0) {
      memset(ctrl, 0, sizeof(ctrl));
      msg.msg_control = ctrl;
      msg.msg_controllen = sizeof(ctrl);
      cmsghdr* c = CMSG_FIRSTHDR(&msg);
      c->cmsg_level = SOL_SOCKET;
      c->cmsg_type = SCM_RIGHTS;
      c->cmsg_len = CMSG_LEN(sizeof(int));
      memcpy(CMSG_DATA(c), &pass_fd, sizeof(int));
    }
    ssize_t n = sendmsg(fd, &msg, MSG_NOSIGNAL | MSG_DONTWAIT);
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
      if (errno == EPIPE || errno == ECONNRESET) return fail(kRemoteError, "send: peer closed the connection");
      return fail(kSystemError, "sendmsg: %s", strerror(errno));
    }
    done += (size_t)n;
  }
  if (shrt) shutdown(fd, SHUT_WR);
  return kSuccess;
}

Status uds_recv(int fd, void* buf, size_t len, int* got_fd, Deadline dl) {
  if (got_fd) *got_fd = -1;
  char* p = (char*)buf;
  size_t done = 0;
  while (done < len) {
    AMEM_TRY(wait_fd(fd, POLLIN, dl, "recv"));
    msghdr msg;
    memset(&msg, 0, sizeof(msg));
    iovec iov{p + done, len - done};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t n = recvmsg(fd, &msg, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
    if (n < 0) {
      if (errno == EINTR || errno == EAGAIN || errno == EWOULDBLOCK) continue;
      if (errno == ECONNRESET) return fail(kRemoteError, "recv: peer reset the connection");
      return fail(kSystemError, "recvmsg: %s", strerror(errno));
    }
    if (n == 0) return fail(kRemoteError, "recv: peer closed the connection after %zu of %zu bytes", done, len);
    for (cmsghdr* c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
      if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
        int f;
        memcpy(&f, CMSG_DATA(c), sizeof(int));
        if (got_fd && *got_fd < 0) *got_fd = f;
        else close(f);
      }
    }
    done += (size_t)n;
  }
  return kSuccess;
}

}  // namespace amem
