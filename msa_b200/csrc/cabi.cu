// Error reporting and version of the C ABI.
#include "common.cuh"

namespace msa {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

}  // namespace msa

extern "C" const char* msa_last_error(void) { return msa::g_error; }
extern "C" int msa_abi_version(void) { return MSA_ABI_VERSION; }
