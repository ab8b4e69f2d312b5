#include "ibcomm/tunables.h"

#include <cstdlib>
#include <map>
#include <mutex>

namespace ibcomm {

namespace {
std::mutex g_mu;
std::map<std::string, int>& Table() {
  static std::map<std::string, int> t;
  return t;
}
}  // namespace

int Tunable(const char* name, int dflt) {
  {
    std::lock_guard<std::mutex> lock(g_mu);
    auto it = Table().find(name);
    if (it != Table().end()) return it->second;
  }
  const char* s = getenv(name);
  if (s == nullptr || s[0] == '\0') return dflt;
  char* end = nullptr;
  const long v = strtol(s, &end, 10);
  return end == s ? dflt : static_cast<int>(v);
}

void SetTunable(const std::string& name, int value) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (value < 0) Table().erase(name);
  else Table()[name] = value;
}

void ClearTunables() {
  std::lock_guard<std::mutex> lock(g_mu);
  Table().clear();
}

}  // namespace ibcomm
