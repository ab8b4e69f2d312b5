// Small host utilities: size-string parser, integer helpers, trace stamp.
// Behavioural parity with the reference's ibcomm/util.h:62-175.
#pragma once

#include <time.h>

#include <cctype>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "ibcomm/error.h"

namespace util {

// Thrown by parse_number for any string that is not
//   [+-] digits [k|m|g] [b]      (letters case-insensitive).
class MalformedNumber : public std::runtime_error {
 public:
  explicit MalformedNumber(const std::string& s) : std::runtime_error(s) {}
};

// "31kb" -> 31744.  Binary multipliers (k = 1024).  "0.5", "0x", "97MiB",
// "b" and the empty string are malformed.  Overflow of int64 is malformed too.
inline int64_t parse_number(const std::string& text) {
  const char* p = text.c_str();
  const char* const end = p + text.size();
  bool negative = false;
  if (p != end && (*p == '+' || *p == '-')) {
    negative = (*p == '-');
    ++p;
  }
  if (p == end || !isdigit(static_cast<unsigned char>(*p)))
    throw MalformedNumber("Malformed number: '" + text + "' (digits expected)");
  unsigned __int128 mag = 0;
  const unsigned __int128 kLimit = static_cast<unsigned __int128>(INT64_MAX) + 1;
  while (p != end && isdigit(static_cast<unsigned char>(*p))) {
    mag = mag * 10 + static_cast<unsigned>(*p - '0');
    if (mag > kLimit) throw MalformedNumber("Malformed number: '" + text + "' (out of range)");
    ++p;
  }
  if (p != end) {
    int shift = -1;
    switch (tolower(static_cast<unsigned char>(*p))) {
      case 'k': shift = 10; break;
      case 'm': shift = 20; break;
      case 'g': shift = 30; break;
      default: break;
    }
    if (shift >= 0) {
      mag <<= shift;
      ++p;
    }
  }
  if (p != end && tolower(static_cast<unsigned char>(*p)) == 'b') ++p;
  if (p != end)
    throw MalformedNumber("Malformed number: '" + text + "' (unexpected '" + std::string(p) + "')");
  if (mag > kLimit || (!negative && mag == kLimit))
    throw MalformedNumber("Malformed number: '" + text + "' (out of range)");
  int64_t v = static_cast<int64_t>(static_cast<uint64_t>(mag));
  return negative ? -v : v;
}

template <typename A, typename B>
constexpr auto ceilDiv(A a, B b) -> decltype(a / b) {
  return (a + b - 1) / b;
}

// p when n == 2^p, otherwise 0.  n = 1 therefore gives 0 as well; callers use
// the value as a "power of two with at least two members" gate.
inline int GetExpOfTwo(uint64_t n) {
  if (n == 0 || (n & (n - 1)) != 0) return 0;
  int p = 0;
  while ((n >>= 1) != 0) ++p;
  return p;
}

// Largest power of two that is <= n (n >= 1).
inline uint64_t FloorPow2(uint64_t n) {
  uint64_t p = 1;
  while ((p << 1) <= n) p <<= 1;
  return p;
}

// Appends a CLOCK_MONOTONIC_RAW stamp.  A null vector is an argument error.
inline void trace(std::vector<struct timespec>* v) {
  if (v == nullptr) IBCOMM_FAIL(INVALID_ARGUMENT, "v is nullptr.\n");
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC_RAW, &ts);
  v->push_back(ts);
}

}  // namespace util
