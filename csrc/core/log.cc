#include "core/log.h"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <strings.h>
#include <unistd.h>

namespace mnccl {
namespace {
std::atomic<int> g_level{-1};
std::mutex g_mu;

int parse_level() {
  const char* e = std::getenv("MINI_NCCL_DEBUG");
  if (!e || !*e) return static_cast<int>(LogLevel::Warn);
  if (!strcasecmp(e, "NONE") || !strcmp(e, "0")) return 0;
  if (!strcasecmp(e, "WARN") || !strcmp(e, "1")) return 1;
  if (!strcasecmp(e, "INFO") || !strcmp(e, "2")) return 2;
  if (!strcasecmp(e, "TRACE") || !strcmp(e, "3")) return 3;
  return 1;
}

void vprint(const char* tag, const char* fmt, va_list ap) {
  char buf[1024];
  vsnprintf(buf, sizeof(buf), fmt, ap);
  std::lock_guard<std::mutex> lk(g_mu);
  fprintf(stderr, "[%s] %s\n", tag, buf);
  fflush(stderr);
}
}  // namespace

LogLevel log_level() {
  int l = g_level.load(std::memory_order_relaxed);
  if (l < 0) {
    l = parse_level();
    g_level.store(l, std::memory_order_relaxed);
  }
  return static_cast<LogLevel>(l);
}

void set_log_level(LogLevel lvl) { g_level.store(static_cast<int>(lvl)); }

void log_always(const char* tag, const char* fmt, ...) {
  if (log_level() == LogLevel::None) return;
  va_list ap;
  va_start(ap, fmt);
  vprint(tag, fmt, ap);
  va_end(ap);
}

void log_at(LogLevel lvl, const char* tag, const char* fmt, ...) {
  if (static_cast<int>(log_level()) < static_cast<int>(lvl)) return;
  va_list ap;
  va_start(ap, fmt);
  vprint(tag, fmt, ap);
  va_end(ap);
}

}  // namespace mnccl
