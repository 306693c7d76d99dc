// Sampling over float32 logits [n, V]: greedy argmax (ties go to the lowest id,
// src/frontend/sampling.rs:181-189) and a non-finite check (sampling.rs:97-99).
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

// A row may be shared by the blocks of a thread-block cluster: block `rank` of `nranks` takes the
// elements [lo, hi) of the row, lo a multiple of 4.
struct Slice {
  int lo, hi;
};
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {       // every thread of every block of the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the 64-bit word at `mine` (an address in this block's shared memory) in block `rank` of the cluster
__device__ __forceinline__ unsigned long long peer_u64(const void* mine, uint32_t rank) {
  uint32_t local = static_cast<uint32_t>(__cvta_generic_to_shared(mine)), remote;
  unsigned long long v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
  return v;
}
__device__ __forceinline__ Slice slice_of(int V) {
  const int n = (int)cluster_size(), r = (int)cluster_rank();
  const int chunk = ((V + n - 1) / n + 3) & ~3;
  Slice s;
  s.lo = min(V, r * chunk);
  s.hi = min(V, s.lo + chunk);
  return s;
}

// Calls f(i, row[i]) for this thread's share of the elements [sl.lo, sl.hi) of a row, every index once,
// in ascending order per thread.  Rows of a multiple of 4 floats on a 16-byte boundary are read as
// float4, four loads in flight.
template <typename F>
__device__ __forceinline__ void for_each_of_row(const float* __restrict__ row, int V, Slice sl, F f) {
  if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int n4 = sl.hi >> 2, step = blockDim.x;          // sl.lo and V are multiples of 4, so sl.hi is
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = (sl.lo >> 2) + threadIdx.x; j < n4; j += 4 * step) {
      const bool has1 = j + step < n4, has2 = j + 2 * step < n4, has3 = j + 3 * step < n4;
      const float4 a = row4[j];
      const float4 b = has1 ? row4[j + step] : zero;
      const float4 c = has2 ? row4[j + 2 * step] : zero;
      const float4 d = has3 ? row4[j + 3 * step] : zero;
      f(4 * j, a.x); f(4 * j + 1, a.y); f(4 * j + 2, a.z); f(4 * j + 3, a.w);
      if (has1) { const int i = 4 * (j + step); f(i, b.x); f(i + 1, b.y); f(i + 2, b.z); f(i + 3, b.w); }
      if (has2) { const int i = 4 * (j + 2 * step); f(i, c.x); f(i + 1, c.y); f(i + 2, c.z); f(i + 3, c.w); }
      if (has3) { const int i = 4 * (j + 3 * step); f(i, d.x); f(i + 1, d.y); f(i + 2, d.z); f(i + 3, d.w); }
    }
  } else {
    for (int i = sl.lo + threadIdx.x; i < sl.hi; i += blockDim.x) f(i, row[i]);
  }
}

// larger value first, then the lower id: one 64-bit word whose maximum is the argmax with ties to the
// lowest id
__device__ __forceinline__ uint32_t order_key(float v) {   // larger value -> larger key; -0 counts as +0
  uint32_t b = __float_as_uint(v);
  if (b == 0x80000000u) b = 0u;
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long best_word(float v, int i) {
  return ((unsigned long long)order_key(v) << 32) | (uint32_t)(0x7fffffff - i);
}

// The best (value, id) of the elements [sl.lo, sl.hi) over the block, then over the cluster; the same
// word in every thread of every block.  `slot`: one 64-bit word of shared memory, `warp_best`: 32.
template <typename F>
__device__ unsigned long long cluster_best(const float* row, int V, Slice sl, unsigned long long* warp_best,
                                           unsigned long long* slot, F adjust) {
  unsigned long long best = 0;
  for_each_of_row(row, V, sl, [&](int i, float x) {
    const unsigned long long w = best_word(adjust(i, x), i);
    best = w > best ? w : best;
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_best[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long b = 0;
    for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) b = warp_best[w] > b ? warp_best[w] : b;
    *slot = b;
  }
  cluster_sync();
  best = 0;
  for (uint32_t r = 0; r < cluster_size(); ++r) {
    const unsigned long long other = peer_u64(slot, r);
    best = other > best ? other : best;
  }
  cluster_sync();                       // nobody rewrites its slot while another block still reads it
  return best;
}

// One cluster of blocks per row.  out_token[row] = argmax; bad[0] set if a logit is not finite.
__global__ void argmax_kernel(const float* __restrict__ logits, long long row_stride, int V,
                              int* __restrict__ out_token, int* __restrict__ bad) {
  __shared__ unsigned long long warp_best[32];
  __shared__ unsigned long long slot;
  const int r = blockIdx.x / cluster_size();
  const float* row = logits + (size_t)r * row_stride;
  bool nonfinite = false;
  const unsigned long long best = cluster_best(row, V, slice_of(V), warp_best, &slot, [&](int, float x) {
    if (!isfinite(x)) nonfinite = true;
    return x;
  });
  if (nonfinite) atomicExch(bad, 1);
  if (cluster_rank() == 0 && threadIdx.x == 0) out_token[r] = best ? 0x7fffffff - (int)(uint32_t)best : 0;
}

}  // namespace srlm

using namespace srlm;

// One cluster of `cluster` blocks per row (1: plain blocks).
template <typename... KArgs, typename... Args>
static void launch_rows(void (*kernel)(KArgs...), int rows, int cluster, int block, size_t smem, cudaStream_t stream,
                        Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(rows * cluster);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster > 1 ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Blocks per row: a long row is shared by a cluster of up to 8 (the portable size), each block a slice,
// as long as the clusters of all rows find room on the GPU at once.
static int blocks_per_row(int V, int rows) {
  int c = V >= 32768 ? 8 : V >= 8192 ? 2 : 1;
  while (c > 1 && rows * c > 148) c >>= 1;
  return c;
}

extern "C" int srlm_argmax(const float* logits, long long row_stride, int n, int V, int* out_token,
                           int* bad_flag, cudaStream_t stream) {
  if (n <= 0) return ST_OK;
  if (V <= 0 || row_stride < V) return refuse(ST_BAD_SIZE, "argmax: V=%d stride=%lld", V, row_stride);
  const int block = V >= 4096 ? 1024 : 256;
  launch_rows(argmax_kernel, n, blocks_per_row(V, n), block, 0, stream, logits, row_stride, V, out_token, bad_flag);
  return launched();
}

// ---------------------------------------------------------------------------
// Temperature / top-k / top-p sampling with a repetition penalty, one block (for a
// long row a cluster of 8 blocks, each with a slice of the row, their sums combined
// through distributed shared memory) per row, in the reference's order of operations (src/frontend/sampling.rs:92-158):
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
  u64 bins[256];          // the pass in progress: the sums over the whole row
  u64 mine[256];          // ... and over this block's slice (read by the other blocks of the cluster)
  u64 first[256];         // masses of the kept set by the top 8 bits of the key (reused by both searches)
  u64 found[3];           // digit, sum above it, its own bin
  u64 low_id[256];        // smallest id of this block's slice that fell into each bin (kept for shift == 0)
  u64 low_all[256];       // ... and of the whole row
  u64 word;               // one word for the other blocks to read
  unsigned long long warp_best[32];
  int is[32];
};

// The sum over the cluster of one integer per block (the same in every thread of every block).
__device__ u64 cluster_sum(u64 mine, Shared& sh) {
  __syncthreads();
  if (threadIdx.x == 0) sh.word = mine;
  cluster_sync();
  u64 sum = 0;
  for (uint32_t r = 0; r < cluster_size(); ++r) sum += peer_u64(&sh.word, r);
  cluster_sync();
  return sum;
}

// One radix pass: adds `weight(v)` of every element for which `match(key, i)` holds into the bin of its
// digit at `shift`, then scans the bins from the top: the digit at which `above + bins` first reaches
// `target`, the sum above that digit, and the digit's own bin go to sh.found.  The keys of a row share
// few leading digits, so every lane adds into a copy of the bins of its own (`copies`, in dynamic shared
// memory); the copies are summed before the scan.  Integer additions: any order gives the same sums.
template <typename Match, typename Weight>
__device__ __forceinline__ void radix_pass(const float* v, int V, Slice sl, int shift, u64 above, u64 target,
                                           Shared& sh, u64* copies, Match match, Weight weight, bool fill) {
  if (fill) {
    for (int i = threadIdx.x; i < REPLICAS * REPLICA_STRIDE; i += blockDim.x) copies[i] = 0;
    if (shift == 0)
      for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.low_id[i] = 0x7fffffffull;
    __syncthreads();
    u64* lane_copy = copies + (threadIdx.x & (REPLICAS - 1)) * REPLICA_STRIDE;
    for_each_of_row(v, V, sl, [&](int i, float x) {
      const uint32_t key = order_key(x);
      if (match(key, i)) {
        const u64 w = weight(x);
        const uint32_t d = (key >> shift) & 255u;
        if (w) atomicAdd(&lane_copy[d], w);
        if (shift == 0) atomicMin(&sh.low_id[d], (u64)i);
      }
    });
    __syncthreads();
    for (int d = threadIdx.x; d < 256; d += blockDim.x) {
      u64 sum = 0;
#pragma unroll 8
      for (int c = 0; c < REPLICAS; ++c) sum += copies[c * REPLICA_STRIDE + d];
      sh.mine[d] = sum;
    }
    cluster_sync();                       // every block's slice is in its `mine`
    const uint32_t n = cluster_size();
    for (int d = threadIdx.x; d < 256; d += blockDim.x) {
      u64 sum = 0, low = 0x7fffffffull;
      for (uint32_t r = 0; r < n; ++r) {
        sum += peer_u64(&sh.mine[d], r);
        if (shift == 0) { const u64 other = peer_u64(&sh.low_id[d], r); low = other < low ? other : low; }
      }
      sh.bins[d] = sum;
      if (shift == 0) sh.low_all[d] = low;
    }
    cluster_sync();                       // nobody rewrites `mine` or `low_id` while another block reads them
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
__device__ int nth_holder(const float* v, int V, Slice sl, uint32_t key, const Kept& kept, u64 n, u64 holders,
                          int first_id, Shared& sh) {
  if (n <= 1 && first_id >= 0) return first_id;
  // the smallest and the largest holder: one word per block, (0x7fffffff - smallest) above largest + 1
  unsigned long long best = 0;
  {
    int lo = 0x7fffffff, hi = -1;
    for_each_of_row(v, V, sl, [&](int i, float x) {
      if (order_key(x) == key && kept.has(key, i)) { lo = min(lo, i); hi = max(hi, i); }
    });
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh.warp_best[warp] = ((unsigned long long)(uint32_t)(0x7fffffff - lo) << 32) | (uint32_t)(hi + 1);
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t a = 0, b = 0;
      for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) {
        a = max(a, (uint32_t)(sh.warp_best[w] >> 32));
        b = max(b, (uint32_t)sh.warp_best[w]);
      }
      sh.word = ((unsigned long long)a << 32) | b;
    }
    cluster_sync();
    uint32_t a = 0, b = 0;
    for (uint32_t r = 0; r < cluster_size(); ++r) {
      const unsigned long long w = peer_u64(&sh.word, r);
      a = max(a, (uint32_t)(w >> 32));
      b = max(b, (uint32_t)w);
    }
    cluster_sync();
    best = ((unsigned long long)a << 32) | b;
  }
  int a = 0x7fffffff - (int)(uint32_t)(best >> 32), b = (int)(uint32_t)best - 1;
  if (n <= 1) return a;
  if (n >= holders) return b;
  while (a < b) {                         // smallest id c with #{holders with id <= c} >= n
    const int mid = a + (b - a) / 2;
    int part = 0;
    for_each_of_row(v, V, sl, [&](int i, float x) { part += (i <= mid && order_key(x) == key && kept.has(key, i)); });
    const u64 count = cluster_sum((u64)block_sum_i(part, sh.is), sh);
    if (count >= n) b = mid; else a = mid + 1;
  }
  return a;
}

// The element of the kept set at which the running mass, in the order of key descending and id
// ascending, first reaches `target` (1 <= target <= total mass).  sh.first must hold the kept set's
// masses by the top 8 bits of the key.
__device__ void select_by_mass(const float* v, int V, Slice sl, const Kept& kept, float vmax, u64 target, Shared& sh,
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
    radix_pass(v, V, sl, shift, above, target, sh, copies,
               [&](uint32_t key, int i) { return kept.has(key, i) && (key >> (shift + 8)) == pre; },
               [&](float x) { return (u64)mass_of(x, vmax); }, level != 0);
    prefix = (prefix << 8) | (uint32_t)sh.found[0];
    above = sh.found[1];
  }
  const u64 own = sh.found[2];                         // mass of the elements with this very key
  const int first_id = (int)sh.low_all[prefix & 255u];
  __syncthreads();
  const u64 w = (u64)mass_of(key_value(prefix), vmax);
  const u64 holders = w ? own / w : 1;
  u64 need = w ? (target > above ? (target - above + w - 1) / w : 1) : 1;
  if (need < 1) need = 1;
  if (need > holders) need = holders;
  *key_sel = prefix;
  *id_sel = nth_holder(v, V, sl, prefix, kept, need, holders, first_id == 0x7fffffff ? -1 : first_id, sh);
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
  const int r = blockIdx.x / cluster_size();
  const Slice sl = slice_of(V);
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
  // the adjusted values, once (each block its slice); their argmax (ties to the lowest id) and the
  // non-finite check, over the whole row
  bool nonfinite = false;
  const unsigned long long best = cluster_best(row, V, sl, sh.warp_best, &sh.word, [&](int i, float x) {
    if (!isfinite(x)) nonfinite = true;
    if (use_pen && (seen_bits[i >> 5] >> (i & 31) & 1u)) x = x < 0.f ? x * pen : x / pen;
    if (temp > 0.f) x = x / temp;
    v[i] = x;
    return x;
  });
  if (nonfinite) atomicExch(bad, 1);
  const float bv = key_value((uint32_t)(best >> 32));
  const int bi = best ? 0x7fffffff - (int)(uint32_t)best : 0;
  const bool writer = cluster_rank() == 0 && threadIdx.x == 0;
  // the decision must be the same in every block of the cluster: they meet again at every pass
  const bool any_nonfinite = cluster_sum((u64)__syncthreads_or(nonfinite), sh) != 0;
  if (any_nonfinite || !(temp > 0.f)) {
    if (writer) out_token[r] = bi;
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
      radix_pass(v, V, sl, shift, above, (u64)k, sh, copies,
                 [&](uint32_t key, int) { return level == 0 || (key >> (shift + 8)) == pre; },
                 [](float) { return (u64)1; }, true);
      prefix = (prefix << 8) | (uint32_t)sh.found[0];
      above = sh.found[1];
    }
    const u64 ties = sh.found[2];
    const int first_id = (int)sh.low_all[prefix & 255u];
    __syncthreads();
    kept.kth = prefix;
    if (above + ties > (u64)k)             // a tie on the boundary: keep the lowest ids among the equal
      kept.id_cut = nth_holder(v, V, sl, prefix, Kept{0u, 0x7fffffff}, (u64)k - above, ties,
                               first_id == 0x7fffffff ? -1 : first_id, sh);
  }
  // the kept set's masses by the top 8 bits of the key; their sum is the softmax denominator
  radix_pass(v, V, sl, 24, 0, ~(u64)0, sh, copies, [&](uint32_t key, int i) { return kept.has(key, i); },
             [&](float x) { return (u64)mass_of(x, bv); }, true);
  for (int i = threadIdx.x; i < 256; i += blockDim.x) sh.first[i] = sh.bins[i];
  __syncthreads();
  u64 total = 0;
  for (int i = 0; i < 256; ++i) total += sh.first[i];
  if (total == 0) {                       // the same in every block: the bins hold the whole row
    if (writer) { atomicExch(bad, 1); out_token[r] = bi; }
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
    select_by_mass(v, V, sl, kept, bv, target, sh, copies, &key_cut, &id_cut, &kept_mass);
  }
  // the draw
  u64 draw = (u64)ceil((double)uniform[r] * (double)kept_mass);
  draw = draw < 1 ? 1 : (draw > kept_mass ? kept_mass : draw);
  uint32_t key_sel;
  int id_sel;
  u64 through;
  select_by_mass(v, V, sl, kept, bv, draw, sh, copies, &key_sel, &id_sel, &through);
  // never beyond the cutoff element (the reference falls back to the last kept element)
  if (key_sel < key_cut || (key_sel == key_cut && id_sel > id_cut)) id_sel = id_cut;
  if (writer) out_token[r] = id_sel;
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
  launch_rows(sample_kernel, n, blocks_per_row(V, n), 1024, smem, stream, logits, row_stride, V, temperature, top_k, top_p,
              penalty, uniform, history, hist_offsets, scratch, out_token, bad_flag);
  return launched();
}
