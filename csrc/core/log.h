// Levelled logger and environment helpers.
//
// Keeps the reference's knobs (plugin/gmm_util.h:132-195): level 0..5 from GMM_LOG
// (default 3 = INFO), prefix "AMEM [LEVEL]".  Unlike the reference every line goes to
// stderr in one write() so lines of different ranks do not interleave, and with
// AMEM_LOG_JSON=1 each line is a JSON object for machine consumption.
#pragma once
#include <execinfo.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

namespace amem {

enum LogLevel { kFatal = 0, kError = 1, kWarn = 2, kInfo = 3, kDebug = 4, kVerbose = 5 };

inline long env_long(const char* name, long dflt) {
  const char* v = getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  long r = strtol(v, &end, 0);
  return end == v ? dflt : r;
}

inline std::string env_str(const char* name, const char* dflt) {
  const char* v = getenv(name);
  return (v && *v) ? std::string(v) : std::string(dflt);
}

inline std::atomic<int>& log_level_ref() {
  static std::atomic<int> lvl{(int)env_long("GMM_LOG", kInfo)};
  return lvl;
}

inline bool log_json() {
  static int j = (int)env_long("AMEM_LOG_JSON", 0);
  return j != 0;
}

inline double now_ms() {
  using namespace std::chrono;
  return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

inline void log_write(int level, const char* file, const char* func, int line, const char* fmt, ...) {
  if (level > log_level_ref().load(std::memory_order_relaxed)) return;
  static const char* names[] = {"FATAL", "ERROR", "WARN", "INFO", "DEBUG", "VERBOSE"};
  char msg[768];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  const char* base = strrchr(file, '/');
  base = base ? base + 1 : file;
  char out[1024];
  int n;
  if (log_json()) {
    for (char* p = msg; *p; ++p)
      if (*p == '"' || *p == '\\' || *p == '\n') *p = ' ';
    n = snprintf(out, sizeof(out),
                 "{\"amem\":\"%s\",\"pid\":%d,\"t_ms\":%.3f,\"at\":\"%s:%s:%d\",\"msg\":\"%s\"}\n",
                 names[level], (int)getpid(), now_ms(), base, func, line, msg);
  } else {
    n = snprintf(out, sizeof(out), "AMEM [%s] pid:%d %s:%s:%d %s\n", names[level], (int)getpid(),
                 base, func, line, msg);
  }
  if (n >= (int)sizeof(out)) {  // cut: keep the line well-formed (closing quote / brace, newline)
    n = (int)sizeof(out) - 1;
    if (log_json()) memcpy(out + n - 3, "\"}\n", 3);
    else out[n - 1] = '\n';
  }
  ssize_t w = write(2, out, (size_t)n);
  (void)w;
}

// Dump the current call stack at ERROR level (the reference's gtrace(),
// plugin/gmm_util.h:47-59; its output can be symbolised with addr2line).
inline void log_backtrace() {
  void* frames[32];
  int n = backtrace(frames, 32);
  backtrace_symbols_fd(frames, n, 2);
}

#define AMEM_LOG(level, ...) ::amem::log_write(level, __FILE__, __func__, __LINE__, __VA_ARGS__)
#define LOGE(...) AMEM_LOG(::amem::kError, __VA_ARGS__)
#define LOGW(...) AMEM_LOG(::amem::kWarn, __VA_ARGS__)
#define LOGI(...) AMEM_LOG(::amem::kInfo, __VA_ARGS__)
#define LOGD(...) AMEM_LOG(::amem::kDebug, __VA_ARGS__)

}  // namespace amem
