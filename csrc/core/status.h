// Result codes and error plumbing shared by every layer of the library.
//
// The numeric values match NCCL's ncclResult_t so that the C API can return them
// unchanged.  The reference only ever returned ncclSuccess from its pause/resume
// entry points (nccl_patch/nccl_2.27.5-1.diff:69-88); here every layer returns a
// real code and leaves a human readable message in a thread-local slot.
#pragma once
#include <cstdarg>
#include <cstdio>
#include <string>

namespace amem {

enum Status : int {
  kSuccess = 0,
  kCudaError = 1,       // ncclUnhandledCudaError
  kSystemError = 2,     // ncclSystemError  (sockets, files, timeouts on the host)
  kInternalError = 3,   // ncclInternalError (device-side wait ran out, broken invariant)
  kInvalidArgument = 4, // ncclInvalidArgument
  kInvalidUsage = 5,    // ncclInvalidUsage  (collective while paused, wrong order)
  kRemoteError = 6,     // ncclRemoteError   (a peer closed its socket / died)
  kInProgress = 7,
};

inline std::string& last_error_slot() {
  static thread_local std::string s;
  return s;
}

inline Status fail(Status st, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  last_error_slot() = buf;
  return st;
}

inline const char* status_name(int st) {
  switch (st) {
    case kSuccess: return "success";
    case kCudaError: return "unhandled cuda error";
    case kSystemError: return "system error";
    case kInternalError: return "internal error";
    case kInvalidArgument: return "invalid argument";
    case kInvalidUsage: return "invalid usage";
    case kRemoteError: return "remote error";
    case kInProgress: return "in progress";
    default: return "unknown result code";
  }
}

#define AMEM_TRY(expr)                         \
  do {                                         \
    ::amem::Status _st = (expr);               \
    if (_st != ::amem::kSuccess) return _st;   \
  } while (0)

}  // namespace amem
