// Embedding gather, residual-add + RMSNorm, SwiGLU and casts.
//
// The residual stream is float32 in every mode; norms reduce in float32 in an
// order fixed by the row width alone, so a row's result does not depend on
// what else is in the batch.  Formulas: src/model/native.rs:213-229 (gather),
// src/model/math.rs:28-50 (RMSNorm), src/model/math.rs:11-22 (SiLU).
#include "common.cuh"

namespace srlm {

__global__ void patch_words_kernel(int* __restrict__ words, long long words_len, const int* __restrict__ pairs,
                                   const int* __restrict__ src, int src_len, int n, int* __restrict__ flag) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int to = pairs[2 * i], from = pairs[2 * i + 1];
  if (to < 0 || to >= words_len || from < 0 || from >= src_len) {
    atomicExch(flag, 1);
    return;
  }
  words[to] = src[from];
}

template <typename TW>
__global__ void embed_gather_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                                    float* __restrict__ out, int H, int vocab, int* __restrict__ bad) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= vocab) {          // the host checks too; never read outside the table
    if (threadIdx.x == 0) atomicExch(bad, 1);
    for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)t * H + i] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[(size_t)t * H + i] = to_float(row[i]);
}

// x = residual[src] (+ delta[src]); residual[src] = x when rows == nullptr;
// out[r] = x * rsqrt(mean(x^2) + eps) * (w (+1)).
template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TA* __restrict__ delta,
                                   const float* __restrict__ weight, float eps, TA* __restrict__ out,
                                   const int* __restrict__ rows, int H, int unit_offset) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* res = residual + src * H;
  const TA* del = delta ? delta + src * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float x = res[i];
    if (del) {
      x += to_float(del[i]);
      if (!rows) res[i] = x;
    }
    ss += x * x;
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  TA* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float x = res[i];
    if (del && rows) x += to_float(del[i]);
    const float w = weight[i] + (unit_offset ? 1.f : 0.f);
    o[i] = from_float<TA>(x * inv * w);
  }
}

// The same with rows of H = 4 * k elements read and written as 16-byte (float32) and 8-byte (bfloat16)
// pieces; a thread keeps up to CACHE pieces in registers, so a row of up to 4 * CACHE * blockDim elements
// is read once.  The sum of squares adds a thread's elements in index order, then the threads in the
// order of block_sum: fixed by the width.
template <int CACHE>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ residual, const bf16* __restrict__ delta, const float* __restrict__ weight,
                       float eps, bf16* __restrict__ out, const int* __restrict__ rows, int H, int unit_offset) {
  __shared__ float scratch[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float4* res = reinterpret_cast<float4*>(residual + src * H);
  const uint2* del = delta ? reinterpret_cast<const uint2*>(delta + src * H) : nullptr;
  const int pieces = H / 4;
  float4 x[CACHE];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CACHE; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < pieces) {
      float4 v = res[i];
      if (del) {
        const uint2 d = del[i];
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d.y));
        v.x += lo.x; v.y += lo.y; v.z += hi.x; v.w += hi.y;
        if (!rows) res[i] = v;
      }
      ss += v.x * v.x; ss += v.y * v.y; ss += v.z * v.z; ss += v.w * v.w;
      x[c] = v;
    }
  }
  const float total = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(total / (float)H + eps);
  uint2* o = reinterpret_cast<uint2*>(out + (size_t)r * H);
  const float4* w4 = reinterpret_cast<const float4*>(weight);
  const float off = unit_offset ? 1.f : 0.f;
#pragma unroll
  for (int c = 0; c < CACHE; ++c) {
    const int i = threadIdx.x + c * blockDim.x;
    if (i < pieces) {
      const float4 w = w4[i];
      const __nv_bfloat162 lo = __floats2bfloat162_rn(x[c].x * inv * (w.x + off), x[c].y * inv * (w.y + off));
      const __nv_bfloat162 hi = __floats2bfloat162_rn(x[c].z * inv * (w.z + off), x[c].w * inv * (w.w + off));
      uint2 p;
      p.x = *reinterpret_cast<const uint32_t*>(&lo);
      p.y = *reinterpret_cast<const uint32_t*>(&hi);
      o[i] = p;
    }
  }
}

__device__ __forceinline__ float silu_f(float x) {
  // branch-stable logistic, src/model/math.rs:11-22
  if (x >= 0.f) return x / (1.f + expf(-x));
  const float e = expf(x);
  return x * (e / (1.f + e));
}

// in[T, 2I]: gate in columns [0, I), up in [I, 2I)  ->  out[T, I]
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ in, TA* __restrict__ out, int I, size_t total) {
  pdl_wait();
  pdl_trigger();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I, i = idx % I;
    const float g = to_float(in[t * 2 * I + i]);
    const float u = to_float(in[t * 2 * I + I + i]);
    out[idx] = from_float<TA>(silu_f(g) * u);
  }
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ in, TO* __restrict__ out, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_float<TO>(to_float(in[i]));
}

// out[t] += delta[t]  (float32 residual, any activation type)
template <typename TA>
__global__ void residual_add_kernel(float* __restrict__ residual, const TA* __restrict__ delta, size_t n) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    residual[i] += to_float(delta[i]);
}

// flag[0] = 1 if any a[i] (+ b[i], when b is given) is NaN or infinite.
template <typename TB>
__global__ void check_finite_kernel(const float* __restrict__ a, const TB* __restrict__ b, size_t n,
                                    int* __restrict__ flag) {
  pdl_wait();
  pdl_trigger();
  bool bad = false;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float x = a[i];
    if (b) x += to_float(b[i]);
    bad |= !(fabsf(x) <= 3.402823466e+38f);
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicExch(flag, 1);
}

static inline int norm_block(int H) {
  int b = 32;
  while (b < 1024 && b * 4 < H) b <<= 1;
  return b;
}
static inline int flat_grid(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  return (int)(g > 148 * 16 ? 148 * 16 : (g == 0 ? 1 : g));
}

}  // namespace srlm

using namespace srlm;

extern "C" int srlm_embed_gather(const int* ids, const void* table, int table_dtype, float* out, int T,
                                 int H, int vocab, int* bad_flag, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (H <= 0 || vocab <= 0) return refuse(ST_BAD_SIZE, "embed_gather: H=%d vocab=%d", H, vocab);
  const int block = H >= 1024 ? 256 : 128;
  SRLM_DISPATCH_ACT(table_dtype, TW, launch_pdl(embed_gather_kernel<TW>, dim3(T), dim3(block), 0, stream,
      ids, (const TW*)table, out, H, vocab, bad_flag));
  return launched();
}

extern "C" int srlm_add_rmsnorm(float* residual, const void* delta, const float* weight, float eps,
                                void* out, int act_dtype, const int* rows, int R, int H, int unit_offset,
                                cudaStream_t stream) {
  if (R <= 0) return ST_OK;
  if (H <= 0 || !(eps > 0.f)) return refuse(ST_BAD_SIZE, "add_rmsnorm: H=%d eps=%g", H, (double)eps);
  if (act_dtype == DT_BF16 && H % 4 == 0 && H <= 4 * 4 * 1024 &&
      (((uintptr_t)residual | (uintptr_t)weight) & 15) == 0 && (((uintptr_t)delta | (uintptr_t)out) & 7) == 0) {
    // whole rows in registers: one read of the residual, vector loads and stores
    const int pieces = H / 4;
    // a thread keeps up to 4 pieces: blocks of 256 threads for rows of up to 4096 elements (several blocks
    // share an SM and their loads overlap each other's reductions), wider blocks only for wider rows
    int block = 32;
    while (block < 1024 && block * 4 < pieces) block <<= 1;
    const int per_thread = (pieces + block - 1) / block;
    if (per_thread <= 1)
      launch_pdl(add_rmsnorm_vec_kernel<1>, dim3(R), dim3(block), 0, stream, residual, (const bf16*)delta, weight, eps,
                 (bf16*)out, rows, H, unit_offset);
    else if (per_thread <= 2)
      launch_pdl(add_rmsnorm_vec_kernel<2>, dim3(R), dim3(block), 0, stream, residual, (const bf16*)delta, weight, eps,
                 (bf16*)out, rows, H, unit_offset);
    else
      launch_pdl(add_rmsnorm_vec_kernel<4>, dim3(R), dim3(block), 0, stream, residual, (const bf16*)delta, weight, eps,
                 (bf16*)out, rows, H, unit_offset);
    return launched();
  }
  SRLM_DISPATCH_ACT(act_dtype, TA, launch_pdl(add_rmsnorm_kernel<TA>, dim3(R), dim3(norm_block(H)), 0, stream,
      residual, (const TA*)delta, weight, eps, (TA*)out, rows, H, unit_offset));
  return launched();
}

extern "C" int srlm_swiglu(const void* in, void* out, int act_dtype, int T, int I, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (I <= 0) return refuse(ST_BAD_SIZE, "swiglu: I=%d", I);
  const size_t total = (size_t)T * I;
  SRLM_DISPATCH_ACT(act_dtype, TA, launch_pdl(swiglu_kernel<TA>, dim3(flat_grid(total, 256)), dim3(256), 0, stream,
      (const TA*)in, (TA*)out, I, total));
  return launched();
}

extern "C" int srlm_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n,
                         cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  const int grid = flat_grid((size_t)n, 256);
  if (in_dtype == DT_F32 && out_dtype == DT_BF16)
    cast_kernel<float, bf16><<<grid, 256, 0, stream>>>((const float*)in, (bf16*)out, (size_t)n);
  else if (in_dtype == DT_BF16 && out_dtype == DT_F32)
    cast_kernel<bf16, float><<<grid, 256, 0, stream>>>((const bf16*)in, (float*)out, (size_t)n);
  else
    return refuse(ST_BAD_DTYPE, "cast: %d -> %d is not offered", in_dtype, out_dtype);
  return launched();
}

extern "C" int srlm_residual_add(float* residual, const void* delta, int act_dtype, long long n,
                                 cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  SRLM_DISPATCH_ACT(act_dtype, TA, (residual_add_kernel<TA><<<flat_grid((size_t)n, 256), 256, 0, stream>>>(
      residual, (const TA*)delta, (size_t)n)));
  return launched();
}

// words[pairs[2 i]] = src[pairs[2 i + 1]] for i < n: token ids that a step takes from what the step before
// it sampled, while the host has not read them yet.  A source index outside [0, src_len) or a destination
// outside [0, words_len) is skipped and raises the flag (the host checks too).
extern "C" int srlm_patch_words(int* words, long long words_len, const int* pairs, const int* src, int src_len,
                                int n, int* flag, cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (!words || !pairs || !src || !flag) return refuse(ST_BAD_SIZE, "patch_words: a null argument");
  launch_pdl(patch_words_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, words, words_len, pairs, src, src_len,
             n, flag);
  return launched();
}

// The non-finite test of a step (src/model/native.rs:276-278, 292-294): a [n] float32, b [n] of the
// activation dtype or null; flag[0] becomes 1 if any a[i] + b[i] is NaN or infinite.
extern "C" int srlm_check_finite(const float* a, const void* b, int b_dtype, long long n, int* flag,
                                 cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (!flag) return refuse(ST_BAD_SIZE, "check_finite: no flag");
  const int grid = flat_grid((size_t)n, 256);
  SRLM_DISPATCH_ACT(b_dtype, TB, launch_pdl(check_finite_kernel<TB>, dim3(grid), dim3(256), 0, stream,
      a, (const TB*)b, (size_t)n, flag));
  return launched();
}
