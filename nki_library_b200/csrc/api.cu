// Error reporting and version query of the C ABI.
#include "common.cuh"

namespace b200moe {
namespace {
thread_local char g_error[512] = "";
}
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
}  // namespace b200moe

extern "C" const char* b200moe_last_error(void) { return b200moe::g_error; }
extern "C" int b200moe_version(void) { return 100; }
