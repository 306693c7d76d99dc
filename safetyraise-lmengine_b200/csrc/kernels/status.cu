#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace srlm {
static thread_local char g_error[512] = "";

int refuse(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int launched() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_error, sizeof(g_error), "CUDA: %s", cudaGetErrorString(e));
    return static_cast<int>(e);
  }
  return ST_OK;
}
}  // namespace srlm

namespace srlm {
static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }
}  // namespace srlm

// 1: kernels of the forward pass may start before their predecessor in the stream has finished
// (programmatic dependent launch, the default); 0: plain stream order.
extern "C" void srlm_set_pdl(int on) { srlm::g_pdl = on != 0; }

extern "C" const char* srlm_last_error() { return srlm::g_error; }
extern "C" int srlm_kernels_abi() { return 1; }
