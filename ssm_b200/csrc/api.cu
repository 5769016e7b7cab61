// Library-level entry points: ABI version and the thread-local error message.
#include <cstdarg>

#include "common.cuh"

namespace ssmb {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
}  // namespace ssmb

extern "C" int ssm_b200_abi_version(void) { return SSM_B200_ABI_VERSION; }
extern "C" const char* ssm_b200_last_error(void) { return ssmb::g_err; }
