// Sampling over float32 logits [n, V]: greedy argmax (ties go to the lowest id,
// src/frontend/sampling.rs:181-189) and a non-finite check (sampling.rs:97-99).
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

// One block per row.  out_token[row] = argmax; bad[0] set if a logit is not finite.
__global__ void argmax_kernel(const float* __restrict__ logits, long long row_stride, int V,
                              int* __restrict__ out_token, int* __restrict__ bad) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  bool nonfinite = false;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (!isfinite(v)) nonfinite = true;
    if (v > bv) { bv = v; bi = i; }          // strided scan: ascending i per thread
  }
  if (nonfinite) atomicExch(bad, 1);
  auto better = [](float v1, int i1, float v2, int i2) { return v1 > v2 || (v1 == v2 && i1 < i2); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    bv = lane < nw ? best_v[lane] : -CUDART_INF_F;
    bi = lane < nw ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out_token[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

}  // namespace srlm

using namespace srlm;

extern "C" int srlm_argmax(const float* logits, long long row_stride, int n, int V, int* out_token,
                           int* bad_flag, cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (V <= 0 || row_stride < V) return refuse(ST_BAD_SIZE, "argmax: V=%d stride=%lld", V, row_stride);
  const int block = V >= 4096 ? 1024 : 256;
  argmax_kernel<<<n, block, 0, stream>>>(logits, row_stride, V, out_token, bad_flag);
  return launched();
}
