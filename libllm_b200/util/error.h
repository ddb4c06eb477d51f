// Errors of the host library.  Every failure inside the library is an `llm::Error` that carries
// the reference's status number (src/libllm/llm.h:42-45) and a finer kind; the C API
// (libllm_b200/capi/llm_api.cc) catches it at the boundary and keeps the message for
// `llm_get_last_error_message`, as the reference does (src/libllm/llm.cc:60-71).
#pragma once
#include <cstdarg>
#include <cstdio>
#include <stdexcept>
#include <string>

namespace llm {

enum class ErrorKind : int {
  InvalidArg = 1,   // an argument or option is not acceptable
  Config = 2,       // config.json misses a key or holds a value the architecture does not allow
  Weights = 3,      // the weight files do not fit the model
  Cache = 4,        // no free slot or page, a slot freed twice
  Unsupported = 5,  // a size or option a kernel refuses rather than computing a wrong result
  Extension = 6,    // a kernel library is missing, cannot be loaded or reported a failure
  Aborted = 7,
  Eof = 8,
};

constexpr int STATUS_OK = 0;
constexpr int STATUS_INVALID_ARG = 0x0100;
constexpr int STATUS_INSUFFICIENT_BUFFER = 0x0101;
constexpr int STATUS_ABORTED = 0x0102;
constexpr int STATUS_EOF = 0x0103;

class Error : public std::runtime_error {
 public:
  Error(ErrorKind kind, const std::string &msg) : std::runtime_error(msg), kind_(kind) {}
  ErrorKind kind() const { return kind_; }
  int status() const {
    switch (kind_) {
      case ErrorKind::InvalidArg:
      case ErrorKind::Config:
      case ErrorKind::Unsupported:
        return STATUS_INVALID_ARG;
      case ErrorKind::Eof:
        return STATUS_EOF;
      default:
        return STATUS_ABORTED;
    }
  }

 private:
  ErrorKind kind_;
};

inline std::string format(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
inline std::string format(const char *fmt, ...) {
  va_list ap, ap2;
  va_start(ap, fmt);
  va_copy(ap2, ap);
  const int n = vsnprintf(nullptr, 0, fmt, ap);
  va_end(ap);
  std::string out(n > 0 ? (size_t)n : 0, '\0');
  if (n > 0) vsnprintf(&out[0], (size_t)n + 1, fmt, ap2);
  va_end(ap2);
  return out;
}

#define LLM_THROW(kind, ...) throw ::llm::Error(::llm::ErrorKind::kind, ::llm::format(__VA_ARGS__))
#define LLM_CHECK_ARG(cond, ...) \
  do {                           \
    if (!(cond)) LLM_THROW(InvalidArg, __VA_ARGS__); \
  } while (0)

}  // namespace llm
