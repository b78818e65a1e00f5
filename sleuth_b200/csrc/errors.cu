// Error reporting shared by every launcher: a message per host thread, read through slb_last_error().
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace slb {

static thread_local char g_message[1024] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_message, sizeof(g_message), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(2, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return 0;
}

}  // namespace slb

extern "C" const char* slb_last_error() { return slb::g_message; }

extern "C" int slb_abi_version() { return 1; }
