// Shared declarations of the kernel library: element types, status codes and
// small device helpers.  Every exported function is extern "C", takes raw
// device pointers and a stream, allocates nothing, and returns 0, a positive
// cudaError_t, or a negative refusal code whose text srlm_last_error() gives.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace srlm {

enum DType : int { DT_F32 = 0, DT_BF16 = 1 };

enum Status : int {
  ST_OK = 0,
  ST_BAD_SIZE = -1,      // a size the kernel does not take
  ST_BAD_DTYPE = -2,
  ST_BAD_ALIGN = -3,
  ST_DEVICE_FLAG = -4,   // the kernel raised its error flag (bounded wait ran out)
};

int refuse(int code, const char* fmt, ...);   // records the text, returns code
int launched();                                // cudaGetLastError() as a status
bool pdl_enabled();                            // programmatic dependent launch on (default) or off

// Launches a kernel that may begin before the kernel ahead of it in the stream has finished
// (programmatic dependent launch).  Such a kernel must call pdl_wait() before it reads anything
// an earlier kernel wrote or writes anything an earlier kernel reads; what it does before that
// (barrier set-up, TMEM allocation, loads of weights, which no kernel writes) overlaps the
// earlier kernel's tail.  pdl_trigger() lets the kernel behind start its own preamble.
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block in a fixed order (depends on blockDim only).  scratch: 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nwarps = (blockDim.x + 31) >> 5;
  float t = (lane < nwarps) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

}  // namespace srlm

#define SRLM_DISPATCH_ACT(dtype, T, ...)                         \
  do {                                                           \
    if ((dtype) == srlm::DT_F32) { using T = float; __VA_ARGS__; } \
    else if ((dtype) == srlm::DT_BF16) { using T = srlm::bf16; __VA_ARGS__; } \
    else return srlm::refuse(srlm::ST_BAD_DTYPE, "dtype code %d is not known", (int)(dtype)); \
  } while (0)
