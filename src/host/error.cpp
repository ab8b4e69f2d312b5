// Fatal/warning sinks and the exit-or-throw policy switch.
#include "ibcomm/error.h"

#include <atomic>
#include <vector>

namespace ibcomm {

static std::atomic<int> g_policy{static_cast<int>(ErrorPolicy::kExit)};

ErrorPolicy GetErrorPolicy() noexcept { return static_cast<ErrorPolicy>(g_policy.load()); }
void SetErrorPolicy(ErrorPolicy p) noexcept { g_policy.store(static_cast<int>(p)); }

static std::string VFormat(const char* fmt, va_list ap) {
  va_list ap2;
  va_copy(ap2, ap);
  int n = vsnprintf(nullptr, 0, fmt, ap2);
  va_end(ap2);
  if (n < 0) return std::string(fmt);
  std::vector<char> buf(static_cast<size_t>(n) + 1);
  vsnprintf(buf.data(), buf.size(), fmt, ap);
  return std::string(buf.data(), static_cast<size_t>(n));
}

void Fatal(const char* file, int line, int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::string msg = VFormat(fmt, ap);
  va_end(ap);
  if (GetErrorPolicy() == ErrorPolicy::kThrow) {
    char head[512];
    snprintf(head, sizeof(head), "Error occured at %s:L%d. ", file, line);
    throw Error(code, std::string(head) + msg);
  }
  fprintf(stderr, "Error occured at %s:L%d.\n", file, line);
  fputs(msg.c_str(), stderr);
  if (msg.empty() || msg.back() != '\n') fputc('\n', stderr);
  fflush(stderr);
  exit(code);
}

void Warn(const char* file, int line, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  std::string msg = VFormat(fmt, ap);
  va_end(ap);
  fprintf(stderr, "Warning occured at %s:L%d.\n", file, line);
  fputs(msg.c_str(), stderr);
  if (msg.empty() || msg.back() != '\n') fputc('\n', stderr);
}

}  // namespace ibcomm
