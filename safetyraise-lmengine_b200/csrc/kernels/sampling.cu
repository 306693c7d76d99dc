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

// ---------------------------------------------------------------------------
// Temperature / top-k / top-p sampling with a repetition penalty, one block per
// row, in the reference's order of operations (src/frontend/sampling.rs:92-158):
//   penalty -> (temperature == 0: argmax) -> value / temperature -> order by
//   value descending and id ascending -> keep top_k -> softmax over the kept ->
//   keep the shortest prefix whose mass >= top_p -> draw = u * kept mass ->
//   first element whose running mass reaches the draw.
// Nothing is sorted.  "The element at which a running total in sorted order
// reaches a target" is found by bisection on the 32 bits of the order key:
// each probe is one pass over the row and a block sum in a fixed order, so the
// result is the same on every run.  Equal keys are ordered by id with a second
// bisection on the id, taken only when a tie sits on a boundary.
// ---------------------------------------------------------------------------
namespace srlm {

__device__ __forceinline__ uint32_t order_key(float v) {   // larger value -> larger key
  const uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct RowView {
  const float* logits;
  const uint32_t* seen;     // bitmap of history ids in shared memory, or nullptr
  float penalty, inv_temperature_unused, temperature;
  int V;
  __device__ __forceinline__ float value(int i) const {
    float x = logits[i];
    if (seen && (seen[i >> 5] >> (i & 31) & 1u)) x = x < 0.f ? x * penalty : x / penalty;
    return temperature > 0.f ? x / temperature : x;
  }
};

__device__ __forceinline__ float block_sum_f(float v, float* scratch) { return block_sum(v, scratch); }

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

// mass(i) of element i, zero outside the kept set.
struct Mass {
  RowView row;
  Kept kept;
  float vmax, total;
  __device__ __forceinline__ float of(int i, uint32_t* key_out) const {
    const float v = row.value(i);
    const uint32_t key = order_key(v);
    *key_out = key;
    return kept.has(key, i) ? expf(v - vmax) / total : 0.f;
  }
};

// Running mass in sorted order reaches `target` at element (key*, id*): returns them and the mass
// up to and including that element.  If the whole mass stays below target, returns the last
// element of the kept set (smallest kept key, largest id).
__device__ void select_by_mass(const Mass& m, float target, float* fs, int* is, uint32_t* key_sel,
                               int* id_sel, float* mass_through) {
  const int V = m.row.V;
  // largest key k with  sum_{key >= k} mass >= target
  uint32_t lo = 0, hi = 0xffffffffu;      // invariant: G(lo) >= target (or lo == 0), G(hi+1) < target
  bool any = false;
  for (int bit = 31; bit >= 0; --bit) {
    const uint32_t probe = lo | (1u << bit);
    float part = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      uint32_t key;
      const float w = m.of(i, &key);
      if (key >= probe) part += w;
    }
    const float g = block_sum_f(part, fs);
    if (g >= target) { lo = probe; any = true; }
  }
  (void)hi;
  __shared__ uint32_t s_min_key;
  if (!any) {
    // even the whole kept mass is below the target (rounding, e.g. top_p = 1): the last kept
    // element, i.e. the smallest kept key and among its holders the largest id
    if (threadIdx.x == 0) s_min_key = 0xffffffffu;
    __syncthreads();
    uint32_t local = 0xffffffffu;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const uint32_t key = order_key(m.row.value(i));
      if (m.kept.has(key, i)) local = min(local, key);
    }
    atomicMin(&s_min_key, local);
    __syncthreads();
    lo = s_min_key;
  }
  // mass strictly above lo, and how many elements share the key lo
  float above_p = 0.f;
  int ties_p = 0, min_id = 0x7fffffff, max_id = -1;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    uint32_t key;
    const float w = m.of(i, &key);
    if (key > lo) above_p += w;
    if (key == lo && m.kept.has(key, i)) { ties_p += 1; min_id = min(min_id, i); max_id = max(max_id, i); }
  }
  const float above = block_sum_f(above_p, fs);
  const int ties = block_sum_i(ties_p, is);
  // min / max id over the block
  __shared__ int s_min, s_max;
  if (threadIdx.x == 0) { s_min = 0x7fffffff; s_max = -1; }
  __syncthreads();
  if (ties_p) { atomicMin(&s_min, min_id); atomicMax(&s_max, max_id); }
  __syncthreads();
  int pick = s_min;
  float through;
  if (ties <= 1 || !any) {
    if (!any) pick = s_max;
    float part = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      uint32_t key;
      const float w = m.of(i, &key);
      if (key == lo && i <= pick) part += w;
    }
    through = above + block_sum_f(part, fs);
  } else {
    // smallest id c with above + sum_{key == lo, id <= c} mass >= target
    int a = s_min, b = s_max;
    while (a < b) {
      const int mid = a + (b - a) / 2;
      float part = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        uint32_t key;
        const float w = m.of(i, &key);
        if (key == lo && i <= mid) part += w;
      }
      if (above + block_sum_f(part, fs) >= target) b = mid; else a = mid + 1;
    }
    // a may fall between ids that hold the key; move it to the holder at or below... the smallest
    // holder >= a that satisfies the bound is a itself or the next holder; find the smallest holder >= a
    __syncthreads();
    if (threadIdx.x == 0) s_min = 0x7fffffff;
    __syncthreads();
    int local = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      if (i >= a && order_key(m.row.value(i)) == lo && m.kept.has(lo, i)) { local = i; break; }
    if (local != 0x7fffffff) atomicMin(&s_min, local);
    __syncthreads();
    pick = s_min == 0x7fffffff ? s_max : s_min;
    float part = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      uint32_t key;
      const float w = m.of(i, &key);
      if (key == lo && i <= pick) part += w;
    }
    through = above + block_sum_f(part, fs);
  }
  __syncthreads();
  *key_sel = lo;
  *id_sel = pick;
  *mass_through = through;
}

// One block per row.  hist_offsets[row]..hist_offsets[row+1] index `history` (ids for the penalty).
__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ penalty,
              const float* __restrict__ uniform, const int* __restrict__ history,
              const int* __restrict__ hist_offsets, int* __restrict__ out_token, int* __restrict__ bad) {
  extern __shared__ uint32_t seen_bits[];           // ceil(V / 32) words when a penalty applies
  __shared__ float fs[32];
  __shared__ int is[32];
  __shared__ float s_best_v[32];
  __shared__ int s_best_i[32];
  const int r = blockIdx.x;
  RowView row;
  row.logits = logits + (size_t)r * row_stride;
  row.V = V;
  row.temperature = temperature[r];
  row.penalty = penalty ? penalty[r] : 1.f;
  row.seen = nullptr;
  if (row.penalty != 1.f && history) {
    const int words = (V + 31) >> 5;
    for (int i = threadIdx.x; i < words; i += blockDim.x) seen_bits[i] = 0u;
    __syncthreads();
    for (int i = hist_offsets[r] + threadIdx.x; i < hist_offsets[r + 1]; i += blockDim.x) {
      const int tok = history[i];
      if (tok >= 0 && tok < V) atomicOr(&seen_bits[tok >> 5], 1u << (tok & 31));
    }
    __syncthreads();
    row.seen = seen_bits;
  }
  // argmax of the adjusted values (ties to the lowest id) and the non-finite check
  float bv = -CUDART_INF_F;
  int bi = 0x7fffffff;
  bool nonfinite = false;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row.value(i);
    if (!isfinite(row.logits[i])) nonfinite = true;
    if (v > bv) { bv = v; bi = i; }
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
  if (lane == 0) { s_best_v[warp] = bv; s_best_i[warp] = bi; }
  __syncthreads();
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
  if (__syncthreads_or(nonfinite) || !(row.temperature > 0.f)) {
    if (threadIdx.x == 0) out_token[r] = bi;
    return;
  }
  // top-k: the k-th largest key, and the id cut among elements equal to it
  Kept kept{0u, 0x7fffffff};
  const int k = top_k ? top_k[r] : 0;
  if (k > 0 && k < V) {
    uint32_t lo = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t probe = lo | (1u << bit);
      int part = 0;
      for (int i = threadIdx.x; i < V; i += blockDim.x) part += order_key(row.value(i)) >= probe;
      if (block_sum_i(part, is) >= k) lo = probe;
    }
    int above_p = 0, ties_p = 0;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const uint32_t key = order_key(row.value(i));
      above_p += key > lo;
      ties_p += key == lo;
    }
    const int above = block_sum_i(above_p, is);
    const int ties = block_sum_i(ties_p, is);
    kept.kth = lo;
    if (above + ties > k) {            // a tie on the boundary: keep the lowest ids among the equal
      int a = 0, b = V - 1;
      const int need = k - above;
      while (a < b) {
        const int mid = a + (b - a) / 2;
        int part = 0;
        for (int i = threadIdx.x; i < V; i += blockDim.x)
          part += (i <= mid && order_key(row.value(i)) == lo);
        if (block_sum_i(part, is) >= need) b = mid; else a = mid + 1;
      }
      kept.id_cut = a;
    }
  }
  // softmax over the kept set
  Mass m{row, kept, bv, 1.f};
  float part = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    uint32_t key;
    part += m.of(i, &key);
  }
  const float total = block_sum_f(part, fs);
  if (!(total > 0.f) || !isfinite(total)) {
    if (threadIdx.x == 0) { atomicExch(bad, 1); out_token[r] = bi; }
    return;
  }
  m.total = total;
  // top-p cutoff: the shortest prefix whose mass >= top_p
  uint32_t key_cut;
  int id_cut;
  float kept_mass;
  select_by_mass(m, top_p[r], fs, is, &key_cut, &id_cut, &kept_mass);
  // the draw
  const float draw = uniform[r] * kept_mass;
  uint32_t key_sel;
  int id_sel;
  float through;
  select_by_mass(m, draw, fs, is, &key_sel, &id_sel, &through);
  // never beyond the cutoff element (the reference falls back to the last kept element)
  if (key_sel < key_cut || (key_sel == key_cut && id_sel > id_cut)) id_sel = id_cut;
  if (threadIdx.x == 0) out_token[r] = id_sel;
}

}  // namespace srlm

extern "C" int srlm_sample(const float* logits, long long row_stride, int n, int V, const float* temperature,
                           const int* top_k, const float* top_p, const float* penalty, const float* uniform,
                           const int* history, const int* hist_offsets, int* out_token, int* bad_flag,
                           cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (V <= 0 || row_stride < V) return refuse(ST_BAD_SIZE, "sample: V=%d stride=%lld", V, row_stride);
  const size_t smem = history ? (size_t)((V + 31) / 32) * 4 : 0;
  if (smem > 200 * 1024) return refuse(ST_BAD_SIZE, "sample: vocabulary %d is too large for the penalty bitmap", V);
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    raised = true;
  }
  sample_kernel<<<n, 1024, smem, stream>>>(logits, row_stride, V, temperature, top_k, top_p, penalty, uniform,
                                           history, hist_offsets, out_token, bad_flag);
  return launched();
}
