// Causal attention over the paged cache for many rows per entry (prefill, large
// portions) on the 5th-generation tensor cores, head size 128.
//
// A block takes up to 256 rows (query tokens x the query heads of one KV group) of
// one entry, as two tiles of 128 rows, and one KV head, and walks the keys in
// tiles of 128.  Both products run as tcgen05.mma with accumulators in tensor
// memory (512 columns: S and O of both row tiles):
//     S = Q . K^T      A = Q tile, B = K tile, both K-major in shared memory
//     O += P . V       A = P in tensor memory (bfloat16, over the columns of S),
//                      B = V tile, MN-major in shared memory
// Warp 0 issues the TMA page loads, one thread of warp 1 issues the MMAs, and two
// groups of four softmax warps own one row per thread (a row of S sits in one
// TMEM lane, so its maximum and sum need no shuffles).  While one group works on
// its S, the tensor core computes the other group's.  O is rescaled in TMEM only
// when a row's maximum has moved by more than 2^8; until then the old maximum
// stays the reference of the exponentials, which the final division by the sum
// (taken with the same reference) makes exact.  Softmax, sums and the output
// accumulation are float32.  Every wait is bounded; when a bound is hit the block
// raises the error flag and leaves.  Formula: src/model/math.rs:102-155.
//
// When the batch has too few rows for every SM (a portion of a prompt behind a long
// context, single tokens beside it), the keys are cut into slices too: blockIdx.y
// is the slice, a block walks only its slice's key tiles and leaves its row tiles'
// unnormalised outputs with their reference maximum and sum in a workspace, and a
// second kernel adds the slices of a row in slice order.
#include <cuda.h>
#include <math_constants.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace srlm {
namespace fmha {

constexpr int HD = 128;
constexpr int BR = 128;            // rows per row tile (the M of one MMA)
constexpr int KT = 128;            // keys per tile
constexpr int KV_STAGES = 2;
constexpr int THREADS = 320;       // warp 0: TMA, warp 1: MMA, warps 2-5 and 6-9: softmax of row tile 0 and 1
constexpr int TILE_BYTES = KT * HD * 2;        // one K, V or Q tile: 32 KB
constexpr float RESCALE_ABOVE = 8.f;           // log2 of the growth of a row's maximum that O is rescaled for
constexpr long long WAIT_CYCLES = 4000000000ll;

struct Args {
  const bf16* q;
  bf16* out;
  const int* block_table;
  int table_stride;
  const int* cu_q;
  const int* kv_lens;
  const int* work;
  int nq, nkv, page_size;
  int tiles_per_block;     // 1 or 2 row tiles; work[][1] counts in blocks
  float scale_log2;
  int window;
  int* err_flag;
  // key slices: 0 / 1 = none.  Slice z of a block is blockIdx.y and covers the keys [z, z + 1) * kv_chunk
  // (a multiple of the key tile); then out is not written, but for the row tile `slab` = ((work item * 2 +
  // row tile) * nkv + KV head) * nsplit + slice: part_o[slab][128 rows][128] (float32, not divided by the
  // sum) and part_ml[slab][128 rows][2] (reference maximum in log2 units, sum; sum 0 = no key in the slice)
  int nsplit;
  int kv_chunk;
  float* part_o;
  float* part_ml;
};

__device__ __forceinline__ uint32_t s32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(s32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err_flag, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > WAIT_CYCLES) {
      atomicExch(err_flag, code);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(s32(dst)), "l"(map), "r"(s32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
// D[tmem] (+)= A[tmem, bfloat16 pairs per column] . B[smem]
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 128-byte swizzled operand tile.  K-major: rows of 128 bytes along K, 8-row groups 1024 bytes apart
// (the leading offset is unused).  MN-major: rows of 128 bytes along MN (64 elements), 8 k-rows per
// 1024-byte group (stride offset), the next 64 elements of MN `lead` bytes further (leading offset).
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t lead_bytes, uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lead_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((stride_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint32_t umma_idesc(int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// 16-byte chunk `c16` (of 16) of row `row` in a tile of two 64-element panels [128 rows][128 bytes].
__device__ __forceinline__ uint32_t tile_addr(uint32_t tile, int row, int c16) {
  return tile + (uint32_t)(c16 >> 3) * (128 * 128) + (uint32_t)row * 128 + (uint32_t)(((c16 & 7) ^ (row & 7)) << 4);
}


// One row of S (128 keys) in registers: the four loads are in flight together.
struct Row {
  uint32_t a[32], b[32], c[32], d[32];
};
__device__ __forceinline__ void load_row(uint32_t s_addr, Row& r) {
  tmem_ld32(s_addr, r.a);
  tmem_ld32(s_addr + 32, r.b);
  tmem_ld32(s_addr + 64, r.c);
  tmem_ld32(s_addr + 96, r.d);
  tmem_wait_ld();
}
// The maximum of the keys [k_lo, k_hi) of the row (all 128 keys when not MASKED).
template <bool MASKED>
__device__ __forceinline__ float row_max(const Row& r, int k_lo, int k_hi) {
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, m2 = -CUDART_INF_F, m3 = -CUDART_INF_F;
  auto part = [&](const uint32_t (&v)[32], int c) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const int k = c + j;
      if (!MASKED || (k >= k_lo && k < k_hi)) m0 = fmaxf(m0, __uint_as_float(v[j]));
      if (!MASKED || (k + 1 >= k_lo && k + 1 < k_hi)) m1 = fmaxf(m1, __uint_as_float(v[j + 1]));
      if (!MASKED || (k + 2 >= k_lo && k + 2 < k_hi)) m2 = fmaxf(m2, __uint_as_float(v[j + 2]));
      if (!MASKED || (k + 3 >= k_lo && k + 3 < k_hi)) m3 = fmaxf(m3, __uint_as_float(v[j + 3]));
    }
  };
  part(r.a, 0);
  part(r.b, 32);
  part(r.c, 64);
  part(r.d, 96);
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}
// P = exp2(S * scale - base) as bfloat16 pairs over the first 64 columns of S; returns the row sum.
template <bool MASKED>
__device__ __forceinline__ float row_exp(uint32_t s_addr, const Row& r, float scale, float base, int k_lo, int k_hi) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  const float nb = -base;
  auto part = [&](const uint32_t (&v)[32], int c) {
    uint32_t pk[16];
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      float p0 = ex2(fmaf(__uint_as_float(v[j]), scale, nb));
      float p1 = ex2(fmaf(__uint_as_float(v[j + 1]), scale, nb));
      float p2 = ex2(fmaf(__uint_as_float(v[j + 2]), scale, nb));
      float p3 = ex2(fmaf(__uint_as_float(v[j + 3]), scale, nb));
      if (MASKED) {
        const int k = c + j;
        p0 = (k >= k_lo && k < k_hi) ? p0 : 0.f;
        p1 = (k + 1 >= k_lo && k + 1 < k_hi) ? p1 : 0.f;
        p2 = (k + 2 >= k_lo && k + 2 < k_hi) ? p2 : 0.f;
        p3 = (k + 3 >= k_lo && k + 3 < k_hi) ? p3 : 0.f;
      }
      s0 += p0; s1 += p1; s2 += p2; s3 += p3;
      pk[j >> 1] = pack2(p0, p1);
      pk[(j >> 1) + 1] = pack2(p2, p3);
    }
    tmem_st16(s_addr + (c >> 1), pk);
  };
  part(r.a, 0);
  part(r.b, 32);
  part(r.c, 64);
  part(r.d, 96);
  return (s0 + s1) + (s2 + s3);
}

__global__ void __launch_bounds__(THREADS, 1)
attention_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                 const Args a) {
  extern __shared__ uint8_t fmha_smem_raw[];
  uint8_t* smem = fmha_smem_raw + ((1024u - (s32(fmha_smem_raw) & 1023u)) & 1023u);
  uint8_t* q_t = smem;                                   // [2] Q tiles
  uint8_t* k_t = q_t + 2 * TILE_BYTES;                   // [KV_STAGES] K tiles
  uint8_t* v_t = k_t + KV_STAGES * TILE_BYTES;           // [KV_STAGES] V tiles
  uint64_t* k_full = reinterpret_cast<uint64_t*>(v_t + KV_STAGES * TILE_BYTES);
  uint64_t* k_empty = k_full + KV_STAGES;
  uint64_t* v_full = k_empty + KV_STAGES;
  uint64_t* v_empty = v_full + KV_STAGES;
  uint64_t* s_full = v_empty + KV_STAGES;                // [2]: per row tile
  uint64_t* p_ready = s_full + 2;                        // [2]
  uint64_t* o_done = p_ready + 2;                        // [2]
  uint64_t* v_clean = o_done + 2;                        // [2]: V rows without a key of the request are zeroed
  uint64_t* q_full = v_clean + 2;                        // the Q tiles are written (every warp but the producer)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < KV_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_ready[i], 4);
      mbar_init(&o_done[i], 1);
    }
    mbar_init(&v_clean[0], 1);
    mbar_init(&v_clean[1], 1);
    mbar_init(q_full, THREADS / 32 - 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();
  pdl_trigger();

  // the grid runs over (block of rows, KV head) with the heads fastest: the work list is sorted by
  // length, and blocks start in the order of their index
  const int item = blockIdx.x / a.nkv, kvh = blockIdx.x % a.nkv;
  const int e = a.work[2 * item], bt = a.work[2 * item + 1];
  const int g = a.nq / a.nkv;
  const int q0 = a.cu_q[e], q_len = a.cu_q[e + 1] - q0, kv_len = a.kv_lens[e], start = kv_len - q_len;
  const int rows_total = q_len * g;
  const int* table = a.block_table + (size_t)e * a.table_stride;
  // Row tile 1 is always there and holds the block's last rows; row tile 0, when the block has two,
  // holds the 128 rows before them (earlier tokens: it may need fewer key tiles).
  const int r_block = bt * a.tiles_per_block * BR;
  const bool two = a.tiles_per_block == 2 && r_block + BR < rows_total;
  const int r_first[2] = {r_block, two ? r_block + BR : r_block};
  const int r_last1 = min(rows_total, r_first[1] + BR) - 1;
  const int pos_first = start + r_block / g;
  const int first_key = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
  const int jb_window = (first_key / KT) * KT;
  const bool sliced = a.nsplit > 1;
  const int slice_lo = sliced ? (int)blockIdx.y * a.kv_chunk : 0;
  const int slice_hi = sliced ? slice_lo + a.kv_chunk : 0x7fffffff - KT;
  const int jb0 = max(jb_window, slice_lo);
  // the keys a row tile sees end behind its last row's position; a slice ends them earlier
  const int end1 = min(start + r_last1 / g + 1, slice_hi);
  const int end0 = two ? min(start + (r_first[1] - 1) / g + 1, slice_hi) : 0;
  const int n_tiles1 = end1 > jb0 ? (end1 - jb0 + KT - 1) / KT : 0;
  const int n_tiles0 = end0 > jb0 ? (end0 - jb0 + KT - 1) / KT : 0;
  // V tiles that hold rows without a key of this request (beyond its length, before the window)
  const bool dirty_first = a.window > 0 && jb0 < first_key;
  const bool dirty_last = jb0 + n_tiles1 * KT > kv_len;

  if (warp != 0) {
    // Q rows -> shared memory in the swizzled K-major layout (zeros beyond the entry's rows), while
    // warp 0 already fetches the first keys
    // (eight loads in flight per thread, then their stores: a store after every load would make each
    // load wait for the one before it, fourteen round trips to memory in a row)
    constexpr int QB = 8;
    const int total = (two ? 2 : 1) * BR * 16;
    for (int base = threadIdx.x - 32; base < total; base += (THREADS - 32) * QB) {
      uint4 v[QB];
#pragma unroll
      for (int j = 0; j < QB; ++j) {
        const int idx = base + j * (THREADS - 32);
        const int row = idx >> 4, c = idx & 15;
        const int r = r_block + row;
        v[j] = make_uint4(0, 0, 0, 0);
        if (idx < total && r < rows_total)
          v[j] = __ldg(reinterpret_cast<const uint4*>(a.q + ((size_t)(q0 + r / g) * a.nq + kvh * g + r % g) * HD + c * 8));
      }
#pragma unroll
      for (int j = 0; j < QB; ++j) {
        const int idx = base + j * (THREADS - 32);
        if (idx < total) {
          const int row = idx >> 4, c = idx & 15;
          // a block of one row tile keeps it in slot 1
          const uint32_t tile = s32(q_t) + ((two ? row >> 7 : 1) * TILE_BYTES);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(tile_addr(tile, row & 127, c)), "r"(v[j].x),
                       "r"(v[j].y), "r"(v[j].z), "r"(v[j].w) : "memory");
        }
      }
    }
    fence_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(q_full);
  }

  if (warp == 0) {
    // ---------------- TMA producer (lane 0 issues; the warp zeroes dirty V rows) ----------------
    const int ps = a.page_size;
    const int box_rows = ps < KT ? ps : KT;
    const int boxes = KT / box_rows;
    // one lane per page box: the table lookups of a tile overlap instead of queueing in one thread
    auto load = [&](const CUtensorMap* map, uint8_t* tile, uint64_t* full, int jb) {
      if (lane == 0) mbar_expect_tx(full, TILE_BYTES);
      __syncwarp();
      if (lane < boxes) {
        const int key = jb + lane * box_rows;
        const int pg = key / ps;
        const int page = (pg < a.table_stride && key < kv_len) ? max(table[pg], 0) : 0;
        const int row = (page * a.nkv + kvh) * ps + key % ps;
        tma_load_2d(tile + lane * box_rows * 128, map, full, 0, row);
        tma_load_2d(tile + KT * 128 + lane * box_rows * 128, map, full, 64, row);
      }
    };
    bool ok = n_tiles1 > 0;             // a slice beyond the block's last key has nothing to fetch
    auto load_v = [&](int tv) {
      const int sv = tv % KV_STAGES;
      ok = mbar_wait(&v_empty[sv], ((tv / KV_STAGES) & 1) ^ 1, a.err_flag, 47);
      if (!ok) return;
      load(&map_v, v_t + sv * TILE_BYTES, &v_full[sv], jb0 + tv * KT);
      const bool df = dirty_first && tv == 0, dl = dirty_last && tv == n_tiles1 - 1;
      if (df || dl) {
        ok = mbar_wait(&v_full[sv], (tv / KV_STAGES) & 1, a.err_flag, 49);
        if (!ok) return;
        const int jb = jb0 + tv * KT;
        const int bad_to = df ? first_key - jb : 0;            // rows [0, bad_to) and [bad_from, KT)
        const int bad_from = dl ? max(kv_len - jb, 0) : KT;
        const uint32_t vt = s32(v_t + sv * TILE_BYTES);
        for (int idx = lane; idx < KT * 16; idx += 32) {
          const int row = idx >> 4, c = idx & 15;
          if (row < bad_to || row >= bad_from)
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(tile_addr(vt, row, c)), "r"(0) : "memory");
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&v_clean[df ? 0 : 1]);   // each is used once: a waiter cannot fall a phase behind
      }
    };
    for (int t = 0; t < n_tiles1 && ok; ++t) {
      const int s = t % KV_STAGES;
      ok = mbar_wait(&k_empty[s], ((t / KV_STAGES) & 1) ^ 1, a.err_flag, 41);
      if (!ok) break;
      load(&map_k, k_t + s * TILE_BYTES, &k_full[s], jb0 + t * KT);
      if (t >= 1) load_v(t - 1);
    }
    if (ok) load_v(n_tiles1 - 1);
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0 && n_tiles1 > 0) {
      const uint32_t idesc_s = umma_idesc(KT, false), idesc_o = umma_idesc(HD, true);
      bool ok = true;
      auto wait_k = [&](int t) {
        ok = ok && mbar_wait(&k_full[t % KV_STAGES], (t / KV_STAGES) & 1, a.err_flag, 42);
        fence_after();
      };
      // descriptors: the start address sits in the low bits, in units of 16 bytes, so a k-step is an addition
      const uint64_t q_desc = umma_desc(s32(q_t), 0, 1024), k_desc = umma_desc(s32(k_t), 0, 1024);
      const uint64_t v_desc = umma_desc(s32(v_t), KT * 128, 1024);
      auto issue_s = [&](int i, int t) {            // S_i = Q_i . K_t^T
        if (!ok) return;
        const uint64_t qd = q_desc + (uint64_t)(i * (TILE_BYTES >> 4));
        const uint64_t kd = k_desc + (uint64_t)((t % KV_STAGES) * (TILE_BYTES >> 4));
        const uint32_t d = tmem + i * 128;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * (128 * 128) + (ks & 3) * 32) >> 4;   // panel, then 32 bytes per k-step
          umma_bf16(d, qd + off, kd + off, idesc_s, ks != 0);
        }
        umma_commit(&s_full[i]);
      };
      auto issue_pv = [&](int i, int t) {           // O_i += P_i . V_t
        ok = ok && mbar_wait(&p_ready[i], t & 1, a.err_flag, 43);
        if (!ok) return;
        fence_after();
        const uint64_t vd = v_desc + (uint64_t)((t % KV_STAGES) * (TILE_BYTES >> 4));
        const uint32_t d = tmem + 256 + i * 128, p = tmem + i * 128;
        // A = P: 16 keys are 8 columns of bfloat16 pairs; B = V: MN-major, 16 keys are 2048 bytes
        umma_bf16_ts(d, p, vd, idesc_o, t != 0);
#pragma unroll
        for (int kk = 1; kk < KT / 16; ++kk) umma_bf16_ts(d, p + kk * 8, vd + kk * (2048 >> 4), idesc_o, 1);
        umma_commit(&o_done[i]);
      };
      ok = mbar_wait(q_full, 0, a.err_flag, 51);
      wait_k(0);
      if (n_tiles0 > 0) issue_s(0, 0);
      issue_s(1, 0);
      if (ok) umma_commit(&k_empty[0]);
      for (int t = 0; t < n_tiles1 && ok; ++t) {
        const int s = t % KV_STAGES;
        ok = mbar_wait(&v_full[s], (t / KV_STAGES) & 1, a.err_flag, 48);
        if (ok && dirty_first && t == 0)
          ok = mbar_wait(&v_clean[0], 0, a.err_flag, 50);
        else if (ok && dirty_last && t == n_tiles1 - 1)
          ok = mbar_wait(&v_clean[1], 0, a.err_flag, 50);
        if (!ok) break;
        const bool more = t + 1 < n_tiles1;
        if (t < n_tiles0) issue_pv(0, t);
        if (more) wait_k(t + 1);
        if (t + 1 < n_tiles0) issue_s(0, t + 1);
        issue_pv(1, t);
        if (ok) umma_commit(&v_empty[s]);
        if (more) {
          issue_s(1, t + 1);
          if (ok) umma_commit(&k_empty[(t + 1) % KV_STAGES]);
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax: one row per thread, warps 2-5 row tile 0, warps 6-9 row tile 1 ----------------
    const int i = (warp - 2) >> 2;
    const int n_tiles = i ? n_tiles1 : n_tiles0;
    const int ew = warp & 3;
    const int row = ew * 32 + lane;                        // TMEM lane = row of the tile
    const uint32_t lane_addr = (uint32_t)(ew * 32) << 16;
    const uint32_t s_addr = tmem + i * 128 + lane_addr, o_addr = tmem + 256 + i * 128 + lane_addr;
    const int r = r_first[i] + row;
    const int r_end = i ? rows_total : r_first[1];         // rows of this tile: [r_first, min(r_first + 128, r_end))
    const int pos = start + min(r, r_end - 1) / g;
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    // every row of the tile sees all keys of tiles within [full_from, full_to)
    const int pos_min = start + r_first[i] / g;
    const int pos_max = start + (min(r_first[i] + BR, r_end) - 1) / g;
    const int lo_max = a.window > 0 ? max(0, pos_max - a.window + 1) : 0;
    float m_run = -CUDART_INF_F, l_run = 0.f;
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int jb = jb0 + t * KT;
      ok = mbar_wait(&s_full[i], t & 1, a.err_flag, 44);
      if (!ok) break;
      fence_after();
      const bool full = jb >= lo_max && jb + KT - 1 <= pos_min;
      const int k_lo = max(0, lo - jb), k_hi = min(KT, pos - jb + 1);
      Row srow;
      load_row(s_addr, srow);
      const float mx = (full ? row_max<false>(srow, 0, KT) : row_max<true>(srow, k_lo, k_hi)) * a.scale_log2;
      // the reference of the exponentials moves only when the maximum has grown by more than 2^8
      const bool grow = mx > m_run + RESCALE_ABOVE || m_run == -CUDART_INF_F;
      const float m_new = grow ? fmaxf(mx, m_run) : m_run;
      if (t > 0 && __any_sync(0xffffffffu, m_new != m_run)) {
        const float alpha = m_new == m_run ? 1.f : ex2(m_run - m_new);     // m_run = -inf gives 0
        ok = mbar_wait(&o_done[i], (t - 1) & 1, a.err_flag, 45);          // P.V of the tile before is in O
        fence_after();
#pragma unroll 1
        for (int c = 0; c < HD; c += 16) {
          uint32_t v[16];
          tmem_ld16(o_addr + c, v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
          tmem_st16(o_addr + c, v);
        }
        l_run *= alpha;
      }
      m_run = m_new;
      const float base = m_run == -CUDART_INF_F ? 0.f : m_run;
      l_run += full ? row_exp<false>(s_addr, srow, a.scale_log2, base, 0, KT)
                    : row_exp<true>(s_addr, srow, a.scale_log2, base, k_lo, k_hi);
      tmem_wait_st();
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[i]);
    }
    if (ok && n_tiles > 0) ok = mbar_wait(&o_done[i], (n_tiles - 1) & 1, a.err_flag, 46);
    fence_after();
    const bool have = n_tiles > 0 && __all_sync(0xffffffffu, ok);   // the loads are warp-wide: rows beyond the tile run them too
    if (sliced) {
      // this slice's share of the row: unnormalised, with the reference of its exponentials and its sum
      if (i == 1 || two) {
        const size_t slab = (((size_t)item * 2 + i) * a.nkv + kvh) * a.nsplit + blockIdx.y;
        *reinterpret_cast<float2*>(a.part_ml + (slab * BR + row) * 2) = make_float2(m_run, have ? l_run : 0.f);
        if (have) {
          float* dst = a.part_o + (slab * BR + row) * HD;
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            uint32_t v[32];
            tmem_ld32(o_addr + c, v);
            tmem_wait_ld();
#pragma unroll
            for (int q = 0; q < 8; ++q)
              *reinterpret_cast<uint4*>(dst + c + 4 * q) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          }
        }
      }
    } else if (have) {
      // the output row: O / l
      const bool mine = r < min(r_first[i] + BR, r_end);
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const int rr = min(r, r_end - 1);
      bf16* dst = a.out + ((size_t)(q0 + rr / g) * a.nq + kvh * g + rr % g) * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t v[32];
        tmem_ld32(o_addr + c, v);
        tmem_wait_ld();
        if (mine) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o4;
            o4.x = pack2(__uint_as_float(v[8 * q]) * inv, __uint_as_float(v[8 * q + 1]) * inv);
            o4.y = pack2(__uint_as_float(v[8 * q + 2]) * inv, __uint_as_float(v[8 * q + 3]) * inv);
            o4.z = pack2(__uint_as_float(v[8 * q + 4]) * inv, __uint_as_float(v[8 * q + 5]) * inv);
            o4.w = pack2(__uint_as_float(v[8 * q + 6]) * inv, __uint_as_float(v[8 * q + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c + 8 * q) = o4;
          }
        }
      }
    }
  }
  fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
  }
}

// Adds the key slices of every row tile: blockIdx.x = (work item, row tile, KV head), blockIdx.y = eight of
// the tile's rows, a warp takes one row, a lane four of its 128 dimensions.  out = sum_z O_z 2^(m_z - M) / sum_z l_z 2^(m_z - M) with M
// the largest reference among the slices that saw a key; slices are added in slice order.
__global__ void __launch_bounds__(256) attention_prefill_merge_kernel(const Args a) {
  pdl_wait();
  pdl_trigger();
  const int kvh = blockIdx.x % a.nkv, i = (blockIdx.x / a.nkv) & 1, item = blockIdx.x / (2 * a.nkv);
  const int e = a.work[2 * item], bt = a.work[2 * item + 1];
  const int g = a.nq / a.nkv;
  const int q0 = a.cu_q[e], q_len = a.cu_q[e + 1] - q0;
  const int rows_total = q_len * g;
  const int r_block = bt * a.tiles_per_block * BR;
  const bool two = a.tiles_per_block == 2 && r_block + BR < rows_total;
  if (i == 0 && !two) return;
  const int r_first = i ? (two ? r_block + BR : r_block) : r_block;
  const int r_end = i ? rows_total : r_block + BR;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t slab0 = (((size_t)item * 2 + i) * a.nkv + kvh) * a.nsplit;
  const int row = blockIdx.y * 8 + warp;
  if (r_first + row < r_end) {
    float m_z = -CUDART_INF_F, l_z = 0.f;
    if (lane < a.nsplit) {
      const float2 ml = *reinterpret_cast<const float2*>(a.part_ml + ((slab0 + lane) * BR + row) * 2);
      m_z = ml.y > 0.f ? ml.x : -CUDART_INF_F;
      l_z = ml.y;
    }
    float M = m_z;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float w_z = l_z > 0.f ? exp2f(m_z - M) : 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float L = 0.f;
    for (int z = 0; z < a.nsplit; ++z) {
      const float w = __shfl_sync(0xffffffffu, w_z, z);
      L += w * __shfl_sync(0xffffffffu, l_z, z);
      if (w > 0.f) {
        const float4 o = *reinterpret_cast<const float4*>(a.part_o + ((slab0 + z) * BR + row) * HD + lane * 4);
        acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
      }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int rr = r_first + row;
    bf16* dst = a.out + ((size_t)(q0 + rr / g) * a.nq + kvh * g + rr % g) * HD + lane * 4;
    uint2 o2;
    o2.x = pack2(acc.x * inv, acc.y * inv);
    o2.y = pack2(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(dst) = o2;
  }
}

// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}
struct Key {
  const void* ptr; long long rows; int box_rows;
  bool operator<(const Key& o) const { return std::tie(ptr, rows, box_rows) < std::tie(o.ptr, o.rows, o.box_rows); }
};
static std::map<Key, CUtensorMap> g_maps;
static std::mutex g_mutex;

// copies the map into *out under the lock: no pointer into the cache leaves this function
static bool cache_map(CUtensorMap* out, const void* ptr, long long rows, int box_rows) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Key key{ptr, rows, box_rows};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps.emplace(key, m);
  *out = m;
  return true;
}

}  // namespace fmha
}  // namespace srlm

using namespace srlm;

// 1 if srlm_paged_attention_prefill_tcgen05 takes these sizes.
extern "C" int srlm_attention_prefill_tcgen05_takes(int hd, int page_size) {
  return hd == 128 && (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64 ||
                       (page_size > 0 && page_size % 128 == 0));
}

// Ragged batch; work: n_work pairs (entry, block of tiles_per_block x 128 rows), rows = query tokens x
// (nq / nkv); tiles_per_block is 1 or 2.  nsplit > 1 cuts the keys into slices of kv_chunk (a multiple of
// 128) with a block each; part_o then holds n_work * 2 * nkv * nsplit * 128 * 128 floats and part_ml
// n_work * 2 * nkv * nsplit * 128 * 2, and a second kernel adds the slices.
extern "C" int srlm_paged_attention_prefill_tcgen05(const void* q, const void* k_cache, const void* v_cache, void* out,
                                                    long long num_pages, const int* block_table, int table_stride,
                                                    const int* cu_q, const int* kv_lens, const int* work, int n_work,
                                                    int nq, int nkv, int hd, int page_size, float scale, int window,
                                                    int tiles_per_block, int nsplit, int kv_chunk, float* part_o,
                                                    float* part_ml, int* err_flag, cudaStream_t stream) {
  if (n_work <= 0) return ST_OK;
  if (nsplit < 1) nsplit = 1;
  if (nsplit > 1 && (nsplit > 32 || kv_chunk <= 0 || kv_chunk % fmha::KT || !part_o || !part_ml))
    return refuse(ST_BAD_SIZE, "attention_prefill_tcgen05: nsplit=%d kv_chunk=%d (slices of whole key tiles, at most 32, "
                  "with their workspace)", nsplit, kv_chunk);
  if (!srlm_attention_prefill_tcgen05_takes(hd, page_size) || nq <= 0 || nkv <= 0 || nq % nkv ||
      tiles_per_block < 1 || tiles_per_block > 2)
    return refuse(ST_BAD_SIZE, "attention_prefill_tcgen05: nq=%d nkv=%d hd=%d page_size=%d tiles_per_block=%d", nq,
                  nkv, hd, page_size, tiles_per_block);
  const int box_rows = page_size < fmha::KT ? page_size : fmha::KT;
  const long long rows = num_pages * nkv * page_size;
  CUtensorMap mk_copy, mv_copy;
  const CUtensorMap *mk = &mk_copy, *mv = &mv_copy;
  if (!fmha::cache_map(&mk_copy, k_cache, rows, box_rows) || !fmha::cache_map(&mv_copy, v_cache, rows, box_rows))
    return refuse(ST_BAD_SIZE, "attention_prefill_tcgen05: cuTensorMapEncodeTiled refused the cache");
  constexpr int SMEM = 2 * fmha::TILE_BYTES + fmha::KV_STAGES * 2 * fmha::TILE_BYTES + 24 * 8 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fmha::attention_prefill_tcgen05_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return refuse((int)e, "attention_prefill_tcgen05: cannot get %d bytes of shared memory", SMEM);
    configured = true;
  }
  fmha::Args a{(const bf16*)q, (bf16*)out, block_table, table_stride, cu_q, kv_lens, work, nq, nkv, page_size,
               tiles_per_block, scale * 1.4426950408889634f, window, err_flag, nsplit, kv_chunk, part_o, part_ml};
  launch_pdl(fmha::attention_prefill_tcgen05_kernel, dim3(n_work * nkv, nsplit), dim3(fmha::THREADS), SMEM, stream,
             *mk, *mv, a);
  if (nsplit > 1)
    launch_pdl(fmha::attention_prefill_merge_kernel, dim3(n_work * 2 * nkv, fmha::BR / 8), dim3(256), 0, stream, a);
  return launched();
}

