// Rotation table, and the fused per-head RMSNorm of q and k + rotary encoding +
// append of k and v to the paged cache.
//
// Formulas: per-head norm src/model/native.rs:629-634, rotation
// src/model/math.rs:52-99 (half-split pairs (i, i+half), angle =
// pos / theta^(2i/rotary_dim)), append before attending src/model/native.rs:637.
// The scalar kernel also takes interleaved pairs (2i, 2i+1), which other encodings use.
// The angle is formed in double precision and rounded once, so cos and sin are
// exact to float32 at every position.
#include "common.cuh"

namespace srlm {

__global__ void rope_table_kernel(const int* __restrict__ positions, float* __restrict__ cos_out,
                                  float* __restrict__ sin_out, int T, int half, double theta,
                                  int rotary_dim) {
  pdl_wait();
  pdl_trigger();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, i = idx % half;
  const double angle = (double)positions[t] / pow(theta, (2.0 * i) / (double)rotary_dim);
  double s, c;
  sincos(angle, &s, &c);
  cos_out[idx] = (float)c;
  sin_out[idx] = (float)s;
}

// One warp per (token, head) of the fused projection output
// qkv[T, (nq + 2 nkv) * hd]: heads [0,nq) are queries, [nq, nq+nkv) keys, then values.
// kv_slot[t] = page * page_size + offset of token t in this cache group, or -1 to skip the append.
// Cache layout: [page, kv head, token in page, head_dim], so a KV head's share of a page is contiguous.
template <typename TA, typename TC>
__global__ void qk_norm_rope_append_kernel(
    const TA* __restrict__ qkv, TA* __restrict__ q_out, TC* __restrict__ k_cache,
    TC* __restrict__ v_cache, const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
    float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    const int* __restrict__ kv_slot, int T, int nq, int nkv, int hd, int rotary_half,
    int heads_total, int write_kv, int page_size, int interleaved) {
  pdl_wait();
  pdl_trigger();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T * heads_total) return;
  const int t = warp / heads_total, head = warp % heads_total;
  const int width = (nq + 2 * nkv) * hd;
  const TA* src = qkv + (size_t)t * width + (size_t)head * hd;
  const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
  if (!is_q && !write_kv) return;
  const int slot = is_q ? 0 : kv_slot[t];
  if (!is_q && slot < 0) return;

  if (!is_q && !is_k) {   // value: copy
    TC* dst = v_cache + (((size_t)(slot / page_size) * nkv + (head - nq - nkv)) * page_size + slot % page_size) * hd;
    for (int d = lane; d < hd; d += 32) dst[d] = from_float<TC>(to_float(src[d]));
    return;
  }
  const float* w = is_q ? q_norm_w : k_norm_w;
  float inv = 1.f;
  if (w) {
    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) { const float x = to_float(src[d]); ss += x * x; }
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  TA* qdst = is_q ? q_out + ((size_t)t * nq + head) * hd : nullptr;
  TC* kdst = is_k ? k_cache + (((size_t)(slot / page_size) * nkv + (head - nq)) * page_size + slot % page_size) * hd
                  : nullptr;
  auto put = [&](int d, float v) {
    if (is_q) qdst[d] = from_float<TA>(v); else kdst[d] = from_float<TC>(v);
  };
  auto get = [&](int d) {
    const float x = to_float(src[d]);
    return w ? x * inv * w[d] : x;
  };
  const float* cs = cos_t + (size_t)t * rotary_half;
  const float* sn = sin_t + (size_t)t * rotary_half;
  for (int i = lane; i < rotary_half; i += 32) {
    const int li = interleaved ? 2 * i : i, ri = interleaved ? 2 * i + 1 : i + rotary_half;
    const float l = get(li), r = get(ri);
    const float c = cs[i], s = sn[i];
    put(li, l * c - r * s);
    put(ri, r * c + l * s);
  }
  for (int d = 2 * rotary_half + lane; d < hd; d += 32) put(d, get(d));   // unrotated tail
}

// The same for bfloat16 heads of EPL * LPH elements with a rotation over the whole head (rotary_half =
// head_dim / 2): LPH lanes (16 or 32) share a head, a lane holds EPL consecutive elements in one vector
// load, the partner of a pair (i, i + head_dim / 2) sits LPH / 2 lanes away, and every row is read and
// written once in whole sectors.  A warp takes 32 / LPH heads of one token at a time, PASSES times: the
// loads of all of them are in flight before the first is used, and the token's cosines and sines are
// fetched once.  Heads of different kinds may share a warp, so nothing here branches around a shuffle.
template <int N>
__device__ __forceinline__ void load_floats(const float* __restrict__ p, float (&out)[N]) {      // p: N * 4-byte aligned
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
      out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
    }
  } else {
    const float2 v = __ldg(reinterpret_cast<const float2*>(p));
    out[0] = v.x; out[1] = v.y;
  }
}

template <int EPL, int LPH, int PASSES>
__global__ void __launch_bounds__(256)
qk_norm_rope_append_vec_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ q_out, bf16* __restrict__ k_cache,
                               bf16* __restrict__ v_cache, const float* __restrict__ q_norm_w,
                               const float* __restrict__ k_norm_w, float eps, const float* __restrict__ cos_t,
                               const float* __restrict__ sin_t, const int* __restrict__ kv_slot, int T, int nq,
                               int nkv, int heads_total, int write_kv, int page_size) {
  constexpr int HD = EPL * LPH, HALF = HD / 2, HPP = 32 / LPH, HPW = HPP * PASSES;
  struct alignas(2 * EPL) Vec { bf16 v[EPL]; };
  static_assert((EPL == 2 || EPL % 4 == 0) && (LPH == 16 || LPH == 32), "vector loads; whole heads in a warp");
  pdl_wait();
  pdl_trigger();
  const int groups = (heads_total + HPW - 1) / HPW;          // head groups per token
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= T * groups) return;
  const int t = warp / groups, head0 = (warp % groups) * HPW;
  const int sub = lane / LPH, l = lane % LPH;                 // which head of a pass, which lane of that head
  const int slot = write_kv ? kv_slot[t] : -1;
  Vec raw[PASSES];
  bool live[PASSES];
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int head = head0 + p * HPP + sub;
    live[p] = head < heads_total && (head < nq || slot >= 0);
#pragma unroll
    for (int j = 0; j < EPL; ++j) raw[p].v[j] = __float2bfloat16_rn(0.f);
    if (live[p]) raw[p] = *reinterpret_cast<const Vec*>(qkv + ((size_t)t * heads_total + head) * HD + l * EPL);
  }
  const int i0 = (l % (LPH / 2)) * EPL;
  float c[EPL], sn[EPL];
  load_floats<EPL>(cos_t + (size_t)t * HALF + i0, c);
  load_floats<EPL>(sin_t + (size_t)t * HALF + i0, sn);
  const bool left = l < LPH / 2;    // the first half of the lanes holds the elements i of the pairs, the second i + HALF
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int head = head0 + p * HPP + sub;
    const bool is_q = head < nq, is_k = !is_q && head < nq + nkv;
    const float* w = is_q ? q_norm_w : is_k ? k_norm_w : nullptr;
    float x[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) x[j] = __bfloat162float(raw[p].v[j]);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) ss += x[j] * x[j];
#pragma unroll
    for (int off = LPH / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (w) {
      const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
      float wv[EPL];
      load_floats<EPL>(w + l * EPL, wv);
#pragma unroll
      for (int j = 0; j < EPL; ++j) x[j] = x[j] * inv * wv[j];
    }
    Vec out;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, x[j], LPH / 2);
      out.v[j] = __float2bfloat16_rn(left ? x[j] * c[j] - other * sn[j] : x[j] * c[j] + other * sn[j]);
    }
    if (!live[p]) continue;
    bf16* dst;
    if (is_q) {
      dst = q_out + ((size_t)t * nq + head) * HD;
    } else {
      const int kvh = is_k ? head - nq : head - nq - nkv;
      dst = (is_k ? k_cache : v_cache) + (((size_t)(slot / page_size) * nkv + kvh) * page_size + slot % page_size) * HD;
    }
    *reinterpret_cast<Vec*>(dst + l * EPL) = (is_q || is_k) ? out : raw[p];      // values are copied
  }
}

}  // namespace srlm

using namespace srlm;

extern "C" int srlm_rope_table(const int* positions, float* cos_out, float* sin_out, int T, int half,
                               double theta, int rotary_dim, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (half <= 0 || rotary_dim != 2 * half || !(theta > 0.0))
    return refuse(ST_BAD_SIZE, "rope_table: rotary_dim=%d half=%d theta=%g", rotary_dim, half, theta);
  const int n = T * half;
  launch_pdl(rope_table_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, positions, cos_out, sin_out, T, half,
             theta, rotary_dim);
  return launched();
}

extern "C" int srlm_qk_norm_rope_append(const void* qkv, void* q_out, int act_dtype, void* k_cache,
                                        void* v_cache, int cache_dtype, const float* q_norm_w,
                                        const float* k_norm_w, float eps, const float* cos_t,
                                        const float* sin_t, const int* kv_slot, int T, int nq,
                                        int nkv, int hd, int rotary_half, int write_kv, int page_size,
                                        int interleaved, cudaStream_t stream) {
  if (T <= 0) return ST_OK;
  if (nq <= 0 || nkv <= 0 || hd <= 0 || rotary_half < 0 || 2 * rotary_half > hd || page_size <= 0)
    return refuse(ST_BAD_SIZE, "qk_norm_rope_append: nq=%d nkv=%d hd=%d rotary_half=%d", nq, nkv, hd,
                  rotary_half);
  if (act_dtype != cache_dtype)
    return refuse(ST_BAD_DTYPE, "qk_norm_rope_append: cache dtype %d differs from activations %d",
                  cache_dtype, act_dtype);
  const int heads_total = nq + 2 * nkv;
  const long long warps = (long long)T * heads_total;
  if (rotary_half > 0 && (!cos_t || !sin_t))
    return refuse(ST_BAD_SIZE, "qk_norm_rope_append: a rotation of %d pairs needs its tables", rotary_half);
  if (act_dtype == DT_BF16 && !interleaved && 2 * rotary_half == hd && (hd == 64 || hd == 128 || hd == 256) &&
      (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)cos_t |
        (uintptr_t)sin_t | (uintptr_t)q_norm_w | (uintptr_t)k_norm_w) & 15) == 0) {
    // A head per warp and pass (the same order of additions as the attention kernel that does this work
    // itself in decode steps, so both leave the same bits in the cache; 16 lanes of 8 elements measured no
    // faster); a warp takes 4 heads when that still gives every SM several warps, else one.
#define SRLM_ROPE_VEC(EPL, LPH)                                                                                     \
  do {                                                                                                                \
    const int per_pass = 32 / (LPH);                                                                                  \
    const long long w4 = (long long)T * ((heads_total + 4 * per_pass - 1) / (4 * per_pass));                          \
    if (w4 >= 4096)                                                                                                   \
      launch_pdl(qk_norm_rope_append_vec_kernel<EPL, LPH, 4>, dim3((unsigned)((w4 * 32 + 255) / 256)), dim3(256),    \
                 0, stream, (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, q_norm_w, k_norm_w, eps,  \
                 cos_t, sin_t, kv_slot, T, nq, nkv, heads_total, write_kv, page_size);                                \
    else                                                                                                              \
      launch_pdl(qk_norm_rope_append_vec_kernel<EPL, LPH, 1>,                                                         \
                 dim3((unsigned)(((long long)T * ((heads_total + per_pass - 1) / per_pass) * 32 + 255) / 256)),       \
                 dim3(256), 0, stream, (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, q_norm_w,      \
                 k_norm_w, eps, cos_t, sin_t, kv_slot, T, nq, nkv, heads_total, write_kv, page_size);                 \
  } while (0)
    if (hd == 64) SRLM_ROPE_VEC(2, 32); else if (hd == 128) SRLM_ROPE_VEC(4, 32); else SRLM_ROPE_VEC(8, 32);
#undef SRLM_ROPE_VEC
    return launched();
  }
  const int block = 128;
  const long long grid = (warps * 32 + block - 1) / block;
  SRLM_DISPATCH_ACT(act_dtype, TA, launch_pdl(qk_norm_rope_append_kernel<TA, TA>, dim3((unsigned)grid), dim3(block), 0, stream,
      (const TA*)qkv, (TA*)q_out, (TA*)k_cache, (TA*)v_cache, q_norm_w, k_norm_w, eps, cos_t, sin_t,
      kv_slot, T, nq, nkv, hd, rotary_half, heads_total, write_kv, page_size, interleaved ? 1 : 0));
  return launched();
}
