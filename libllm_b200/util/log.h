// Lines on standard error with a time stamp and a severity, in the manner of the reference's
// LOG(severity) (src/lutil/log.h:26-54).  LIBLLM_B200_LOG=0 silences everything below a warning.
#pragma once
#include <cstdarg>

namespace llm {

enum class LogLevel : int { Debug = 0, Info = 1, Warning = 2, Error = 3 };
void set_log_level(LogLevel level);
LogLevel log_level();
void log_line(LogLevel level, const char *fmt, va_list ap);

inline void log_info(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
inline void log_info(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  log_line(LogLevel::Info, fmt, ap);
  va_end(ap);
}
inline void log_warning(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
inline void log_warning(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  log_line(LogLevel::Warning, fmt, ap);
  va_end(ap);
}

}  // namespace llm
