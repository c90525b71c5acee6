// Host-side error bookkeeping of the C ABI.
#include <cstdarg>
#include <cstdio>

#include "moe_common.cuh"

namespace moe {
static thread_local char g_err[512] = "";
static unsigned long long g_wait_limit_ns = 2000000000ull;
unsigned long long wait_limit_ns() { return g_wait_limit_ns; }

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
}
}  // namespace moe

extern "C" int moe_abi_version(void) { return 1; }
extern "C" unsigned long long moe_set_wait_limit_ns(unsigned long long ns) {
  const unsigned long long old = moe::g_wait_limit_ns;
  if (ns != 0) moe::g_wait_limit_ns = ns;
  return old;
}
extern "C" const char* moe_last_error(void) { return moe::g_err; }
