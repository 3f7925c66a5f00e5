// Host-side registry of per-translation-unit device status words.
#include "common.cuh"

#include <cstdlib>
#include <mutex>
#include <vector>

namespace swb {
namespace {
std::vector<StatusUnit>& units() {
  static std::vector<StatusUnit> u;
  return u;
}
std::mutex& units_mu() {
  static std::mutex m;
  return m;
}
}  // namespace

namespace {
int g_pdl = -1;
}
bool pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("SWB_PDL");
    g_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pdl == 1;
}

void register_status_unit(const StatusUnit& u) {
  std::lock_guard<std::mutex> g(units_mu());
  units().push_back(u);
}
}  // namespace swb

extern "C" {

// Reads the first non-zero status word among all kernel units into out8 (8 ints); returns its code.
int swb_status_read(int* out8) {
  std::lock_guard<std::mutex> g(swb::units_mu());
  for (int i = 0; i < 8; ++i) out8[i] = 0;
  for (auto& u : swb::units()) {
    int tmp[8];
    if (u.read(tmp) != 0) return -1;
    if (tmp[0] != 0) {
      for (int i = 0; i < 8; ++i) out8[i] = tmp[i];
      return tmp[0];
    }
  }
  return 0;
}

int swb_status_clear() {
  std::lock_guard<std::mutex> g(swb::units_mu());
  int rc = 0;
  for (auto& u : swb::units()) rc |= u.clear();
  return rc;
}

// Budget of every bounded device-side wait, in nanoseconds (default 2 s).
int swb_set_wait_limit_ns(unsigned long long ns) {
  std::lock_guard<std::mutex> g(swb::units_mu());
  int rc = 0;
  for (auto& u : swb::units()) rc |= u.set_limit(ns);
  return rc;
}

// Launch timeline (profiling aid): `buf` = device buffer of 8 + 4 * capacity u64 words with buf[1] = capacity and
// buf[0] = 0, or null to switch it off. See g_timeline in common.cuh for the record layout.
int swb_set_timeline(void* buf) {
  std::lock_guard<std::mutex> g(swb::units_mu());
  int rc = 0;
  for (auto& u : swb::units()) rc |= u.set_timeline(reinterpret_cast<unsigned long long*>(buf));
  return rc;
}

// Programmatic dependent launch on (1) / off (0) for every kernel of this library.
void swb_set_pdl(int on) { swb::g_pdl = on ? 1 : 0; }

}  // extern "C"
