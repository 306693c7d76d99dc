// Sampling over float32 logits [n, V]: greedy argmax (ties go to the lowest id,
// src/frontend/sampling.rs:181-189) and a non-finite check (sampling.rs:97-99).
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

// Calls f(i, row[i]) for this thread's share of a row, every index once, in ascending order per thread.
// Rows of a multiple of 4 floats on a 16-byte boundary are read as float4, two loads in flight.
template <typename F>
__device__ __forceinline__ void for_each_of_row(const float* __restrict__ row, int V, F f) {
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2, step = blockDim.x;
    for (int j = threadIdx.x; j < n4; j += 2 * step) {
      const float4 a = row4[j];
      const bool more = j + step < n4;
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (more) b = row4[j + step];
      f(4 * j, a.x); f(4 * j + 1, a.y); f(4 * j + 2, a.z); f(4 * j + 3, a.w);
      if (more) {
        const int i = 4 * (j + step);
        f(i, b.x); f(i + 1, b.y); f(i + 2, b.z); f(i + 3, b.w);
      }
    }
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) f(i, row[i]);
  }
}

// One block per row.  out_token[row] = argmax; bad[0] set if a logit is not finite.
__global__ void argmax_kernel(const float* __restrict__ logits, long long row_stride, int V,
                              int* __restrict__ out_token, int* __restrict__ bad) {
  __shared__ float best_v[32];
  __shared__ int best_i[32];
  const float* row = logits + (size_t)blockIdx.x * row_stride;
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  bool nonfinite = false;
  for_each_of_row(row, V, [&](int i, float v) {
    if (!isfinite(v)) nonfinite = true;
    if (v > bv) { bv = v; bi = i; }          // ascending i per thread: the first of equal values stays
  });
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

// ---------------------------------------------------------------------------
// Temperature / top-k / top-p sampling with a repetition penalty, one block per
// row, in the reference's order of operations (src/frontend/sampling.rs:92-158):
//   penalty -> (temperature == 0: argmax) -> value / temperature -> order by
//   value descending and id ascending -> keep top_k -> softmax over the kept ->
//   keep the shortest prefix whose mass >= top_p -> draw = u * kept mass ->
//   first element whose running mass reaches the draw.
// Nothing is sorted.  The adjusted values are written once to a scratch row; "the
// element at which a running total in sorted order reaches a target" is then found
// by a radix search over the 32 bits of the order key, 8 bits a pass: a pass adds
// the elements that match the prefix found so far into 256 bins, and a scan of the
// bins from the top gives the next 8 bits.  Counts (top-k) and masses are integers
// (a mass is exp(v - max) in units of 2^-31), so the sums do not depend on the
// order of the additions: the same token on every run.  Elements with equal keys
// are ordered by id; a tie on a boundary is resolved by a search over the ids.
// About a dozen passes over the row instead of a hundred.
// ---------------------------------------------------------------------------
namespace srlm {

typedef unsigned long long u64;

__device__ __forceinline__ uint32_t order_key(float v) {   // larger value -> larger key
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {
  return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
// exp(v - vmax) in units of 2^-31: 2^31 for the maximum, 0 below about 2^-31 of it
__device__ __forceinline__ uint32_t mass_of(float v, float vmax) {
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"((v - vmax) * 1.4426950408889634f));
  return (uint32_t)(e * 2147483648.0f);
}

__device__ __forceinline__ int block_sum_i(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  int t = lane < nw ? scratch[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// The kept set: key > kth, or key == kth and id <= id_cut.
struct Kept {
  uint32_t kth;
  int id_cut;
  __device__ __forceinline__ bool has(uint32_t key, int i) const {
    return key > kth || (key == kth && i <= id_cut);
  }
};

constexpr int REPLICAS = 32;          // one copy of the bins per lane: the lanes of a warp never meet
constexpr int REPLICA_STRIDE = 257;   // in bins: the copies of a bin fall on different banks

struct Shared {
  u64 bins[256];          // the pass in progress (the copies added up)
  u64 first[256];         // masses of the kept set by the top 8 bits of the key (reused by both searches)
  u64 found[3];           // digit, sum above it, its own bin
  int low_id[256];        // smallest id that fell into each bin of the last pass (kept for shift == 0)
  int is[32];
  int id_lo, id_hi;
};

// One radix pass: adds `weight(v)` of every element for which `match(key, i)` holds into the bin of its
// digit at `shift`, then scans the bins from the top: the digit at which `above + bins` first reaches
// `target`, the sum above that digit, and the digit's own bin go to sh.found.  The keys of a row share
// few leading digits, so every lane adds into a copy of the bins of its own (`copies`, in dynamic shared
// memory); the copies are summed before the scan.  Integer additions: any order gives the same sums.
template <typename Match, typename Weight>
__device__ __forceinline__ void radix_pass(const float* v, int V, int shift, u64 above, u64 target, Shared& sh,
                                           u64* copies, Match match, Weight weight, bool fill) {
  if (fill) {
    for (int i = threadIdx.x; i < REPLICAS * REPLICA_STRIDE; i += blockDim.x) copies[i] = 0;
    if (shift == 0)
      for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.low_id[i] = 0x7fffffff;
    __syncthreads();
    u64* mine = copies + (threadIdx.x & (REPLICAS - 1)) * REPLICA_STRIDE;
    for_each_of_row(v, V, [&](int i, float x) {
      const uint32_t key = order_key(x);
      if (match(key, i)) {
        const u64 w = weight(x);
        const uint32_t d = (key >> shift) & 255u;
        if (w) atomicAdd(&mine[d], w);
        if (shift == 0) atomicMin(&sh.low_id[d], i);
      }
    });
    __syncthreads();
    for (int d = threadIdx.x; d < 256; d += blockDim.x) {
      u64 sum = 0;
#pragma unroll 8
      for (int c = 0; c < REPLICAS; ++c) sum += copies[c * REPLICA_STRIDE + d];
      sh.bins[d] = sum;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    u64 acc = above;
    int d = 255;
    for (; d > 0; --d) {
      if (acc + sh.bins[d] >= target) break;
      acc += sh.bins[d];
    }
    sh.found[0] = (u64)d;
    sh.found[1] = acc;
    sh.found[2] = sh.bins[d];
  }
  __syncthreads();
}

// The n-th (1-based) smallest id among the elements of the kept set whose key is `key`.
// `first_id`: the smallest such id if the caller knows it (the last radix pass records it), else -1.
__device__ int nth_holder(const float* v, int V, uint32_t key, const Kept& kept, u64 n, u64 holders, int first_id,
                          Shared& sh) {
  if (n <= 1 && first_id >= 0) return first_id;
  if (threadIdx.x == 0) { sh.id_lo = 0x7fffffff; sh.id_hi = -1; }
  __syncthreads();
  int lo = 0x7fffffff, hi = -1;
  for_each_of_row(v, V, [&](int i, float x) {
    if (order_key(x) == key && kept.has(key, i)) { lo = min(lo, i); hi = max(hi, i); }
  });
  if (hi >= 0) { atomicMin(&sh.id_lo, lo); atomicMax(&sh.id_hi, hi); }
  __syncthreads();
  int a = sh.id_lo, b = sh.id_hi;
  __syncthreads();
  if (n <= 1) return a;
  if (n >= holders) return b;
  while (a < b) {                         // smallest id c with #{holders with id <= c} >= n
    const int mid = a + (b - a) / 2;
    int part = 0;
    for_each_of_row(v, V, [&](int i, float x) { part += (i <= mid && order_key(x) == key && kept.has(key, i)); });
    if ((u64)block_sum_i(part, sh.is) >= n) b = mid; else a = mid + 1;
  }
  return a;
}

// The element of the kept set at which the running mass, in the order of key descending and id
// ascending, first reaches `target` (1 <= target <= total mass).  sh.first must hold the kept set's
// masses by the top 8 bits of the key.
__device__ void select_by_mass(const float* v, int V, const Kept& kept, float vmax, u64 target, Shared& sh,
                               u64* copies, uint32_t* key_sel, int* id_sel, u64* mass_through) {
  uint32_t prefix = 0;
  u64 above = 0;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    if (level == 0) {
      for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.bins[i] = sh.first[i];
      __syncthreads();
    }
    const uint32_t pre = prefix;
    radix_pass(v, V, shift, above, target, sh, copies,
               [&](uint32_t key, int i) { return kept.has(key, i) && (key >> (shift + 8)) == pre; },
               [&](float x) { return (u64)mass_of(x, vmax); }, level != 0);
    prefix = (prefix << 8) | (uint32_t)sh.found[0];
    above = sh.found[1];
  }
  const u64 own = sh.found[2];                         // mass of the elements with this very key
  const int first_id = sh.low_id[prefix & 255u];
  __syncthreads();
  const u64 w = (u64)mass_of(key_value(prefix), vmax);
  const u64 holders = w ? own / w : 1;
  u64 need = w ? (target > above ? (target - above + w - 1) / w : 1) : 1;
  if (need < 1) need = 1;
  if (need > holders) need = holders;
  *key_sel = prefix;
  *id_sel = nth_holder(v, V, prefix, kept, need, holders, first_id == 0x7fffffff ? -1 : first_id, sh);
  *mass_through = above + need * w;
}

// One block per row.  hist_offsets[row]..hist_offsets[row+1] index `history` (ids for the penalty).
// scratch: one row of V floats per row of logits.
__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ penalty,
              const float* __restrict__ uniform, const int* __restrict__ history,
              const int* __restrict__ hist_offsets, float* __restrict__ scratch, int* __restrict__ out_token,
              int* __restrict__ bad) {
  extern __shared__ u64 dyn_smem[];                 // the copies of the bins, then the penalty's bitmap
  u64* copies = dyn_smem;
  uint32_t* seen_bits = reinterpret_cast<uint32_t*>(dyn_smem + REPLICAS * REPLICA_STRIDE);   // ceil(V / 32) words
  __shared__ Shared sh;
  __shared__ float s_best_v[32];
  __shared__ int s_best_i[32];
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  float* v = scratch + (size_t)r * V;
  const float temp = temperature[r];
  const float pen = penalty ? penalty[r] : 1.f;
  const bool use_pen = pen != 1.f && history;
  if (use_pen) {
    const int words = (V + 31) >> 5;
    for (int i = threadIdx.x; i < words; i += blockDim.x) seen_bits[i] = 0u;
    __syncthreads();
    for (int i = hist_offsets[r] + threadIdx.x; i < hist_offsets[r + 1]; i += blockDim.x) {
      const int tok = history[i];
      if (tok >= 0 && tok < V) atomicOr(&seen_bits[tok >> 5], 1u << (tok & 31));
    }
    __syncthreads();
  }
  // the adjusted values, once; their argmax (ties to the lowest id) and the non-finite check
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  bool nonfinite = false;
  for_each_of_row(row, V, [&](int i, float x) {
    if (!isfinite(x)) nonfinite = true;
    if (use_pen && (seen_bits[i >> 5] >> (i & 31) & 1u)) x = x < 0.f ? x * pen : x / pen;
    if (temp > 0.f) x = x / temp;
    v[i] = x;
    if (x > bv) { bv = x; bi = i; }
  });
  if (nonfinite) atomicExch(bad, 1);
  auto better = [](float v1, int i1, float v2, int i2) { return v1 > v2 || (v1 == v2 && i1 < i2); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_best_v[warp] = bv; s_best_i[warp] = bi; }
  __syncthreads();                                   // also: every thread's values are in the scratch row
  {
    const int nw = (blockDim.x + 31) >> 5;
    bv = lane < nw ? s_best_v[lane] : -CUDART_INF_F;
    bi = lane < nw ? s_best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
  }
  // every thread of every warp now holds the row's best (value, id)
  if (bi == 0x7fffffff) bi = 0;
  if (__syncthreads_or(nonfinite) || !(temp > 0.f)) {
    if (threadIdx.x == 0) out_token[r] = bi;
    return;
  }
  // top-k: the k-th largest key, and the id cut among the elements equal to it
  Kept kept{0u, 0x7fffffff};
  const int k = top_k ? top_k[r] : 0;
  if (k > 0 && k < V) {
    uint32_t prefix = 0;
    u64 above = 0;
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      const uint32_t pre = prefix;
      radix_pass(v, V, shift, above, (u64)k, sh, copies,
                 [&](uint32_t key, int) { return level == 0 || (key >> (shift + 8)) == pre; },
                 [](float) { return (u64)1; }, true);
      prefix = (prefix << 8) | (uint32_t)sh.found[0];
      above = sh.found[1];
    }
    const u64 ties = sh.found[2];
    const int first_id = sh.low_id[prefix & 255u];
    __syncthreads();
    kept.kth = prefix;
    if (above + ties > (u64)k)             // a tie on the boundary: keep the lowest ids among the equal
      kept.id_cut = nth_holder(v, V, prefix, Kept{0u, 0x7fffffff}, (u64)k - above, ties,
                               first_id == 0x7fffffff ? -1 : first_id, sh);
  }
  // the kept set's masses by the top 8 bits of the key; their sum is the softmax denominator
  radix_pass(v, V, 24, 0, ~(u64)0, sh, copies, [&](uint32_t key, int i) { return kept.has(key, i); },
             [&](float x) { return (u64)mass_of(x, bv); }, true);
  for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.first[i] = sh.bins[i];
  __syncthreads();
  u64 total = 0;
  for (int i = 0; i < 256; ++i) total += sh.first[i];
  if (total == 0) {
    if (threadIdx.x == 0) { atomicExch(bad, 1); out_token[r] = bi; }
    return;
  }
  // top-p cutoff: the shortest prefix whose mass >= top_p
  const float tp = top_p[r];
  uint32_t key_cut = 0;
  int id_cut = 0x7fffffff;
  u64 kept_mass = total;
  if (tp < 1.f) {
    u64 target = (u64)ceil((double)tp * (double)total);
    target = target < 1 ? 1 : (target > total ? total : target);
    select_by_mass(v, V, kept, bv, target, sh, copies, &key_cut, &id_cut, &kept_mass);
  }
  // the draw
  u64 draw = (u64)ceil((double)uniform[r] * (double)kept_mass);
  draw = draw < 1 ? 1 : (draw > kept_mass ? kept_mass : draw);
  uint32_t key_sel;
  int id_sel;
  u64 through;
  select_by_mass(v, V, kept, bv, draw, sh, copies, &key_sel, &id_sel, &through);
  // never beyond the cutoff element (the reference falls back to the last kept element)
  if (key_sel < key_cut || (key_sel == key_cut && id_sel > id_cut)) id_sel = id_cut;
  if (threadIdx.x == 0) out_token[r] = id_sel;
}

}  // namespace srlm

// scratch: n rows of V floats that the kernel may overwrite.
extern "C" int srlm_sample(const float* logits, long long row_stride, int n, int V, const float* temperature,
                           const int* top_k, const float* top_p, const float* penalty, const float* uniform,
                           const int* history, const int* hist_offsets, float* scratch, int* out_token,
                           int* bad_flag, cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (V <= 0 || row_stride < V) return refuse(ST_BAD_SIZE, "sample: V=%d stride=%lld", V, row_stride);
  if (!scratch) return refuse(ST_BAD_SIZE, "sample: a scratch row of V floats per row of logits is needed");
  const size_t smem = (size_t)REPLICAS * REPLICA_STRIDE * 8 + (history ? (size_t)((V + 31) / 32) * 4 : 0);
  if (smem > 190 * 1024) return refuse(ST_BAD_SIZE, "sample: vocabulary %d is too large for the penalty bitmap", V);
  static bool raised = false;
  if (!raised) {
    cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 190 * 1024);
    raised = true;
  }
  sample_kernel<<<n, 1024, smem, stream>>>(logits, row_stride, V, temperature, top_k, top_p, penalty, uniform,
                                           history, hist_offsets, scratch, out_token, bad_flag);
  return launched();
}
