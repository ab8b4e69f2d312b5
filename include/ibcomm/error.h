// Error contract of the library.
//
// The process exit code is the error API: a fatal condition prints
// "Error occured at <file>:L<line>." plus a printf-style message to stderr and
// terminates the process with one of four codes (parity with the reference's
// ibcomm/util.h:31-60).  Language bindings that must not kill the interpreter
// switch the policy to "throw", in which case the same call raises
// ibcomm::Error carrying the code and the formatted message.
#pragma once

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <stdexcept>
#include <string>

namespace util {

enum class IBCOMM_ERROR_CODE : int {
  INVALID_ARGUMENT = 1,
  // Failure of the transport (shared-memory rings, peer mapping, a bounded
  // device-side wait that ran out).  Keeps the reference's name and value.
  IBVERBS_ERROR = 2,
  TRANSPORT_ERROR = 2,
  // Failure of a CUDA runtime or driver call.
  CUDA_ERROR = 3,
  NOT_SUPPORTED = 4
};

}  // namespace util

namespace ibcomm {

// Raised instead of exit() when the policy is kThrow.
class Error : public std::runtime_error {
 public:
  Error(int code, const std::string& what) : std::runtime_error(what), code_(code) {}
  int code() const noexcept { return code_; }

 private:
  int code_;
};

enum class ErrorPolicy : int { kExit = 0, kThrow = 1 };

// Process-wide policy.  kExit is the default and matches the reference.
ErrorPolicy GetErrorPolicy() noexcept;
void SetErrorPolicy(ErrorPolicy p) noexcept;

// Formats, prints and then exits or throws according to the policy.
[[noreturn]] void Fatal(const char* file, int line, int code, const char* fmt, ...)
    __attribute__((format(printf, 4, 5)));
void Warn(const char* file, int line, const char* fmt, ...)
    __attribute__((format(printf, 3, 4)));

}  // namespace ibcomm

namespace util {

template <typename... Args>
[[noreturn]] inline void IbcommError(const char* filename, int line, IBCOMM_ERROR_CODE error_code,
                                     const char* format, Args const&... args) {
#pragma GCC diagnostic push
#pragma GCC diagnostic ignored "-Wformat-security"
#pragma GCC diagnostic ignored "-Wformat-nonliteral"
  ibcomm::Fatal(filename, line, static_cast<int>(error_code), format, args...);
#pragma GCC diagnostic pop
}

template <typename... Args>
inline void IbcommWarning(const char* filename, int line, const char* format,
                          Args const&... args) {
#pragma GCC diagnostic push
#pragma GCC diagnostic ignored "-Wformat-security"
#pragma GCC diagnostic ignored "-Wformat-nonliteral"
  ibcomm::Warn(filename, line, format, args...);
#pragma GCC diagnostic pop
}

}  // namespace util

#define IBCOMM_FAIL(code, ...) \
  ::util::IbcommError(__FILE__, __LINE__, ::util::IBCOMM_ERROR_CODE::code, __VA_ARGS__)
#define IBCOMM_WARN(...) ::util::IbcommWarning(__FILE__, __LINE__, __VA_ARGS__)

#ifdef USE_CUDA
#include <cuda_runtime.h>
#define CUDACHECK(cmd)                                                        \
  do {                                                                        \
    cudaError_t e__ = (cmd);                                                  \
    if (e__ != cudaSuccess) {                                                 \
      ::util::IbcommError(__FILE__, __LINE__,                                 \
                          ::util::IBCOMM_ERROR_CODE::CUDA_ERROR, "%s\n",      \
                          cudaGetErrorString(e__));                           \
    }                                                                         \
  } while (0)
#endif
