// Paged causal attention for a ragged batch, plain SIMT arithmetic in float32.
//
// One warp per (token, query head).  The warp walks the request's keys in
// blocks of 32 aligned to multiples of 32 from the start of the sequence, so
// the order of every sum depends only on the token's position: the result is
// the same however the tokens were cut into steps or batched.  This is the
// attention of the float32 path, and the reference the tensor-core kernels are
// tested against.  Formula: src/model/math.rs:102-155 (scale 1/sqrt(hd) or the
// given one, query head h reads KV head h / (nq/nkv), online softmax).
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

constexpr int kMaxDimsPerLane = 8;   // head_dim <= 256

template <typename TA, typename TC>
__global__ void paged_attention_simt_kernel(
    const TA* __restrict__ q, const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
    TA* __restrict__ out, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ entry_of_token, const int* __restrict__ positions, int T, int nq, int nkv,
    int hd, int page_size, float scale, int window) {
  extern __shared__ float q_sh[];      // [warps per block][hd]
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + warp_in_block;
  if (warp >= (long long)T * nq) return;
  const int t = (int)(warp / nq), h = (int)(warp % nq);
  const int kvh = h / (nq / nkv);
  const int pos = positions[t];
  const int* table = block_table + (size_t)entry_of_token[t] * table_stride;

  float* qv = q_sh + warp_in_block * hd;
  const TA* qsrc = q + ((size_t)t * nq + h) * hd;
  for (int d = lane; d < hd; d += 32) qv[d] = to_float(qsrc[d]);
  __syncwarp();

  float acc[kMaxDimsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] = 0.f;
  float m = -CUDART_INF_F, z = 0.f;

  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  for (int jb = (first_key / 32) * 32; jb <= pos; jb += 32) {
    const int j = jb + lane;
    const bool valid = j >= first_key && j <= pos;
    float s = -CUDART_INF_F;
    size_t row = 0;
    if (valid) {
      const int page = table[j / page_size];
      row = ((size_t)page * nkv + kvh) * page_size + (j % page_size);
      const TC* kp = k_cache + row * hd;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot += qv[d] * to_float(kp[d]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float alpha = expf(m - m_new);          // m = -inf at first: exp(-inf) = 0
    const float p = valid ? expf(s - m_new) : 0.f;
    z = z * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kMaxDimsPerLane; ++i) acc[i] *= alpha;
    const int n_here = min(32, pos - jb + 1);
    for (int jj = 0; jj < n_here; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const size_t rj = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
      if (pj == 0.f) continue;                    // masked by the window (uniform over the warp)
      const TC* vp = v_cache + rj * hd;
#pragma unroll
      for (int i = 0; i < kMaxDimsPerLane; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] += pj * to_float(vp[d]);
      }
    }
    m = m_new;
  }
  TA* o = out + ((size_t)t * nq + h) * hd;
  const float inv = 1.f / z;
#pragma unroll
  for (int i = 0; i < kMaxDimsPerLane; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) o[d] = from_float<TA>(acc[i] * inv);
  }
}

}  // namespace srlm

using namespace srlm;

extern "C" int srlm_paged_attention_simt(const void* q, const void* k_cache, const void* v_cache,
                                         void* out, int act_dtype, int cache_dtype,
                                         const int* block_table, int table_stride,
                                         const int* entry_of_token, const int* positions, int T, int nq,
                                         int nkv, int hd, int page_size, float scale, int window,
                                         cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (nq <= 0 || nkv <= 0 || nq % nkv || hd <= 0 || hd > 32 * kMaxDimsPerLane || page_size <= 0)
    return refuse(ST_BAD_SIZE,
                  "paged_attention_simt: nq=%d nkv=%d hd=%d page_size=%d (needs nq %% nkv == 0, hd <= %d)",
                  nq, nkv, hd, page_size, 32 * kMaxDimsPerLane);
  if (act_dtype != cache_dtype)
    return refuse(ST_BAD_DTYPE, "paged_attention_simt: cache dtype %d differs from activations %d",
                  cache_dtype, act_dtype);
  const int warps_per_block = 4;
  const long long warps = (long long)T * nq;
  const long long grid = (warps + warps_per_block - 1) / warps_per_block;
  const size_t smem = (size_t)warps_per_block * hd * sizeof(float);
  SRLM_DISPATCH_ACT(act_dtype, TA, (paged_attention_simt_kernel<TA, TA>
      <<<(unsigned)grid, warps_per_block * 32, smem, stream>>>(
          (const TA*)q, (const TA*)k_cache, (const TA*)v_cache, (TA*)out, block_table, table_stride,
          entry_of_token, positions, T, nq, nkv, hd, page_size, scale, window)));
  return launched();
}
