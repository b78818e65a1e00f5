// Error reporting shared by every launcher: a message per host thread, read through slb_last_error().
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>

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

static int g_pdl = -1;

int pdl_mode() {
  if (g_pdl < 0) {
    const char* e = getenv("SLEUTH_B200_PDL");
    g_pdl = e ? (e[0] == '0' ? 0 : (e[0] == '1' ? 1 : 2)) : 2;   // default 2: measured fastest on a B200
  }
  return g_pdl;
}

static thread_local cudaError_t g_launch_error = cudaSuccess;

void note_launch_error(cudaError_t e) { g_launch_error = e; }

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = g_launch_error;
  g_launch_error = cudaSuccess;
  if (e != cudaSuccess) return fail(2, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return 0;
}

int sm_count() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  static int cached[64] = {0};
  if (cached[dev] > 0) return cached[dev];
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return 148;
  cached[dev] = sms;
  return sms;
}

}  // namespace slb

// Streaming multiprocessors of the current device: the launch heuristics on both sides of the binding count with it.
extern "C" int slb_sm_count() { return slb::sm_count(); }

extern "C" const char* slb_last_error() { return slb::g_message; }

extern "C" int slb_abi_version() { return 1; }

// 1: kernels may start while their predecessor still runs (programmatic dependent launch); 0: strictly one after another.
extern "C" void slb_set_pdl(int mode) { slb::g_pdl = mode < 0 || mode > 2 ? 0 : mode; }
extern "C" int slb_get_pdl() { return slb::pdl_mode(); }
