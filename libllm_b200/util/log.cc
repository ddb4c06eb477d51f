#include "util/log.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <ctime>

namespace llm {

static std::atomic<int> &level_ref() {
  static std::atomic<int> level{[] {
    const char *v = getenv("LIBLLM_B200_LOG");
    if (v && *v == '0') return (int)LogLevel::Warning;
    if (v && *v == '2') return (int)LogLevel::Debug;
    return (int)LogLevel::Info;
  }()};
  return level;
}

void set_log_level(LogLevel level) { level_ref().store((int)level); }
LogLevel log_level() { return (LogLevel)level_ref().load(); }

void log_line(LogLevel level, const char *fmt, va_list ap) {
  if ((int)level < level_ref().load()) return;
  static const char *names[] = {"DEBUG", "INFO", "WARNING", "ERROR"};
  char stamp[32];
  const time_t now = time(nullptr);
  struct tm tmv;
  localtime_r(&now, &tmv);
  strftime(stamp, sizeof(stamp), "%Y-%m-%dT%H:%M:%S", &tmv);
  char msg[1024];
  vsnprintf(msg, sizeof(msg), fmt, ap);
  fprintf(stderr, "%s %s [libllm_b200] %s\n", names[(int)level], stamp, msg);
  fflush(stderr);
}

}  // namespace llm
