// Error bookkeeping and version query of the C ABI.
#include <cstdlib>
#include "frwkv_common.cuh"

#include <cstring>

namespace frwkv {
namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

void clear_error() { g_error[0] = '\0'; }

bool chained_launch_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("FRWKV_DISABLE_CHAINED_LAUNCH");
    return !(e != nullptr && e[0] == '1');
  }();
  return on;
}

}  // namespace frwkv

extern "C" int frwkv_abi_version(void) { return 2; }

extern "C" const char* frwkv_last_error(void) { return frwkv::g_error; }
