// Minimal test harness (googletest is not available offline): CHECK macros
// that count failures, and a runner that prints one line per case.
#pragma once

#include <cstdio>
#include <functional>
#include <string>
#include <vector>

namespace mini {

struct Case {
  std::string name;
  std::function<void()> fn;
};

inline std::vector<Case>& Cases() {
  static std::vector<Case> c;
  return c;
}
inline int& Failures() {
  static int f = 0;
  return f;
}

struct Registrar {
  Registrar(const char* name, std::function<void()> fn) { Cases().push_back({name, std::move(fn)}); }
};

inline int RunAll(const char* filter = nullptr) {
  int failed_cases = 0;
  for (const Case& c : Cases()) {
    if (filter != nullptr && c.name.find(filter) == std::string::npos) continue;
    int before = Failures();
    c.fn();
    bool ok = Failures() == before;
    printf("[%s] %s\n", ok ? "  OK  " : "FAILED", c.name.c_str());
    if (!ok) ++failed_cases;
  }
  printf("%d case(s) failed\n", failed_cases);
  return failed_cases == 0 ? 0 : 1;
}

}  // namespace mini

#define MINI_TEST(name)                                         \
  static void mini_test_##name();                               \
  static ::mini::Registrar mini_reg_##name(#name, mini_test_##name); \
  static void mini_test_##name()

#define CHECK_EQ(a, b)                                                                  \
  do {                                                                                  \
    auto va__ = (a);                                                                    \
    auto vb__ = (b);                                                                    \
    if (!(va__ == vb__)) {                                                              \
      ++::mini::Failures();                                                             \
      fprintf(stderr, "%s:%d: CHECK_EQ(%s, %s) failed\n", __FILE__, __LINE__, #a, #b); \
    }                                                                                   \
  } while (0)

#define CHECK_TRUE(a)                                                             \
  do {                                                                            \
    if (!(a)) {                                                                   \
      ++::mini::Failures();                                                       \
      fprintf(stderr, "%s:%d: CHECK_TRUE(%s) failed\n", __FILE__, __LINE__, #a); \
    }                                                                             \
  } while (0)

#define CHECK_THROWS(expr, Exc)                                                           \
  do {                                                                                    \
    bool thrown__ = false;                                                                \
    try {                                                                                 \
      (void)(expr);                                                                       \
    } catch (const Exc&) {                                                                \
      thrown__ = true;                                                                    \
    }                                                                                     \
    if (!thrown__) {                                                                      \
      ++::mini::Failures();                                                               \
      fprintf(stderr, "%s:%d: %s did not throw %s\n", __FILE__, __LINE__, #expr, #Exc);  \
    }                                                                                     \
  } while (0)
