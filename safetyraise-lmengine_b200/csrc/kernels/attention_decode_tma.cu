// Decode attention over the paged cache with TMA: at most 16 rows (query tokens
// x query heads of one KV group) per entry and KV head, keys in slices.
//
// A block takes one entry, one KV head and one slice of the keys.  One producer
// thread walks the block table and brings whole pages in with tiled TMA copies
// (a KV head's share of a page is one contiguous [page_size, head_dim] block of
// the cache), 128-byte swizzled, into a ring of stages guarded by mbarriers.
// Four consumer warps each take 16 of a tile's 64 keys through both products
// (mma.sync m16n8k16, float32 accumulation) with a running maximum, sum and
// output of their own; the four are merged once, in warp order, after the last
// tile.  The slices of an (entry, KV head) are merged in slice order: when they
// are at most 8, the blocks form a thread-block cluster and each adds a share of
// the output elements out of the others' shared memory; otherwise through
// partial results in global memory, by whichever block finishes last.  Every
// wait is bounded: when a bound is hit the block raises the error flag and goes
// on to the merge without waiting again, so every block of a cluster reaches
// the cluster's barriers.
//
// For head sizes 64, 128 and 256 with a rotation over the whole head the kernel
// can also take q and the step's new keys and values straight from the q/k/v
// projection (see Args::qkv): the consumer warps normalise and rotate the q rows
// on their way into shared memory, and the warp that owns a new key's row puts
// the normalised, rotated key and the value into the tile (over what the TMA copy
// brought for a row nobody had written) and into the cache.
//
// Taken when head_dim is a multiple of 64 and page_size is 8, 16, 32 or a
// multiple of 64; other sizes use the cp.async kernel in attention_mma.cu.
// Formulas: src/model/math.rs:102-155 (attention), :25-99 (norm, rotation).
#include <cuda.h>
#include <math_constants.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace srlm {
namespace dec {

constexpr int KT = 64;
constexpr int STAGES = 3;
constexpr int CONSUMERS = 4;
constexpr int THREADS = (CONSUMERS + 1) * 32;
constexpr long long WAIT_CYCLES = 4000000000ll;

struct Args {
  const bf16* q;
  bf16* out;
  const int* block_table;
  int table_stride;
  const int* cu_q;
  const int* kv_lens;
  int nq, nkv, hd, page_size;
  float scale_log2;
  int window;
  int kv_chunk, nsplit;
  int clustered;           // 1: the nsplit blocks of an (entry, KV head) form a thread-block cluster and merge
                           //    their slices through distributed shared memory; 0: through part_o / part_ml
  float* part_o;
  float* part_ml;
  int* slice_counters;
  int* err_flag;
  // Fused with the step before it (head_dim 64, 128 or 256, rotation over the whole head): q and the
  // step's new keys and values are taken from the projection's output qkv [tokens, (nq + 2 nkv) * hd],
  // normalised per head (if the weights are given) and rotated here; the new keys and values go to the
  // cache and, in the block whose slice holds their positions, straight into the tile in shared memory.
  const bf16* qkv;          // null: q is given and the cache already holds this step's keys and values
  const float* q_norm_w;
  const float* k_norm_w;
  float norm_eps;
  const float* cos_t;       // [tokens, hd / 2]
  const float* sin_t;
  bf16* k_cache;
  bf16* v_cache;
  int write_kv;
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
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(s32(dst)), "l"(map), "r"(s32(bar)), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void cluster_sync() {       // every thread of every block of the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the float at `mine` (an address in this block's shared memory) in block `rank` of the cluster
__device__ __forceinline__ float peer_f32(const float* mine, uint32_t rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(s32(mine)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// One head of one token, HD = 32 * EPL elements, a lane holding EPL consecutive ones: RMSNorm over the
// head (if w is given), then the rotation of the pairs (i, i + HD/2), whose halves sit in lanes l and
// l ^ 16 (src/model/math.rs:25-99).  All 32 lanes call it together.
template <int EPL>
struct alignas(2 * EPL) HeadVec { bf16 v[EPL]; };
template <int EPL>
__device__ __forceinline__ HeadVec<EPL> norm_rotate_head(const HeadVec<EPL>& raw, const float* w, float eps,
                                                         const float* cos_row, const float* sin_row, int lane) {
  constexpr int HD = 32 * EPL;
  float x[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) x[j] = __bfloat162float(raw.v[j]);
  if (w) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) ss += x[j] * x[j];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
    for (int j = 0; j < EPL; ++j) x[j] = x[j] * inv * w[lane * EPL + j];
  }
  const bool left = lane < 16;
  const int i0 = (lane & 15) * EPL;
  HeadVec<EPL> out;
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const float other = __shfl_xor_sync(0xffffffffu, x[j], 16);
    const float c = cos_row[i0 + j], sn = sin_row[i0 + j];
    out.v[j] = __float2bfloat16_rn(left ? x[j] * c - other * sn : x[j] * c + other * sn);
  }
  return out;
}

// Address of the 16-byte chunk `chunk16` (of head_dim/8) of key `key` in a tile made of panels of
// 64 dims: [panel][64 keys][128 bytes], 128-byte swizzle (chunk ^= key & 7).
__device__ __forceinline__ uint32_t tile_addr(uint32_t tile, int key, int chunk16) {
  return tile + (uint32_t)(chunk16 >> 3) * (KT * 128) + (uint32_t)key * 128 +
         (uint32_t)(((chunk16 & 7) ^ (key & 7)) << 4);
}

template <int HD>     // 64, 128, 192 or 256
__global__ void __launch_bounds__(THREADS)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const Args a) {
  constexpr int PANELS = HD / 64;
  constexpr int TILE_BYTES = KT * HD * 2;            // one K or V tile
  constexpr int KS = HD / 16;                        // k steps of Q.K^T
  constexpr int NT_ALL = HD / 8;                     // output n-tiles (every consumer warp holds all dims)
  constexpr int KW = KT / CONSUMERS;                 // keys of a tile per consumer warp
  constexpr int OS = HD + 8;                         // row stride of the merge buffer, in floats
  static_assert(KW == 16, "a consumer warp takes one k-step of 16 keys per tile");
  static_assert((CONSUMERS * 16 * (OS + 2) + 16 * (HD + 2)) * 4 <= STAGES * 2 * TILE_BYTES,
                "the merge buffers live in the tile memory");
  extern __shared__ uint8_t dec_smem_raw[];
  uint8_t* smem = dec_smem_raw + ((1024u - (s32(dec_smem_raw) & 1023u)) & 1023u);
  uint8_t* tiles = smem;                                              // [STAGES][K tile | V tile]
  bf16* q_s = reinterpret_cast<bf16*>(smem + STAGES * 2 * TILE_BYTES);  // [16][HD + 8]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(q_s + 16 * (HD + 8));
  uint64_t* empty_bar = full_bar + STAGES;
  __shared__ int is_last;

  if (threadIdx.x == 0) {                 // nothing here depends on the kernel ahead
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], CONSUMERS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  __syncthreads();                        // the barriers are set up for every warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // When this kernel appends the step's keys itself, no kernel of this step has written anything that the
  // producer warp reads: the batch's layout came before the step's first kernel, and the keys in the cache
  // are those of earlier steps (a row of this step in a tile is stale either way and is replaced in shared
  // memory below).  So the producer fetches its first tiles under the projection's tail.  It does not wait
  // and does not trigger: the block lets its successor start only when its consumers have waited.  A step
  // that reads keys which another kernel of the same step appended (write_kv == 0) must not run ahead: the
  // products between that kernel and this one let their successors start before they have waited
  // themselves, so it may still be running.
  const bool ahead_of_wait = (HD == 64 || HD == 128 || HD == 256) && a.qkv != nullptr && a.write_kv &&
                             warp == CONSUMERS;
  // (the batch's layout is read ahead of the wait by every warp: it was copied before the step's first kernel)
  const int e = blockIdx.x, kvh = blockIdx.y, z = blockIdx.z;
  const int g = a.nq / a.nkv;
  const int q0 = a.cu_q[e], q_len = a.cu_q[e + 1] - q0, kv_len = a.kv_lens[e], start = kv_len - q_len;
  const int rows_total = q_len * g;
  const int* table = a.block_table + (size_t)e * a.table_stride;
  if (!ahead_of_wait) {
    pdl_wait();
    pdl_trigger();
  }

  const int first_key = a.window > 0 ? max(0, start - a.window + 1) : 0;
  const int slice_lo = z * a.kv_chunk, slice_hi = min(kv_len, slice_lo + a.kv_chunk);
  const int jb0 = max(slice_lo, (first_key / KT) * KT);
  const int n_tiles = slice_hi > jb0 ? (slice_hi - jb0 + KT - 1) / KT : 0;

  // Q rows -> shared memory (plain loads: 16 rows at most), by the consumer warps; the producer warp
  // is already fetching the first tiles
  constexpr bool CAN_FUSE = HD == 64 || HD == 128 || HD == 256;
  constexpr int EPL = CAN_FUSE ? HD / 32 : 2;
  const int heads_total = a.nq + 2 * a.nkv;
  if (CAN_FUSE && a.qkv && warp < CONSUMERS) {
    // q rows out of the projection's output: a warp per row, normalised and rotated on the way
#pragma unroll
    for (int row = warp; row < 16; row += CONSUMERS) {
      HeadVec<EPL> out;
#pragma unroll
      for (int j = 0; j < EPL; ++j) out.v[j] = __float2bfloat16_rn(0.f);
      if (row < rows_total) {
        const int tok = q0 + row / g;
        const HeadVec<EPL> raw = *reinterpret_cast<const HeadVec<EPL>*>(
            a.qkv + ((size_t)tok * heads_total + kvh * g + row % g) * HD + lane * EPL);
        out = norm_rotate_head<EPL>(raw, a.q_norm_w, a.norm_eps, a.cos_t + (size_t)tok * (HD / 2),
                                    a.sin_t + (size_t)tok * (HD / 2), lane);
      }
      *reinterpret_cast<HeadVec<EPL>*>(q_s + row * (HD + 8) + lane * EPL) = out;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
  } else if (warp < CONSUMERS) {
    for (int idx = threadIdx.x; idx < 16 * (HD / 8); idx += CONSUMERS * 32) {
      const int row = idx / (HD / 8), c = idx % (HD / 8);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < rows_total)
        v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(q0 + row / g) * a.nq + kvh * g + row % g) * HD + c * 8);
      *reinterpret_cast<uint4*>(q_s + row * (HD + 8) + c * 8) = v;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
  }

  float o[NT_ALL][4];
#pragma unroll
  for (int i = 0; i < NT_ALL; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;

  if (warp == CONSUMERS) {
    // ---------------- producer: lane b fetches page box b of every tile ----------------
    // The page numbers come from the block table in global memory; with one lane per box the
    // look-ups of a tile run side by side, and the next tile's are in flight during the wait.
    const int ps = a.page_size;
    const int box_rows = ps < KT ? ps : KT;          // keys per TMA copy
    const int boxes = KT / box_rows;
    uint64_t stream_once;                            // the cache is read once per step: first to leave L2
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(stream_once));
    auto box_row = [&](int t) {                      // row of the [pages * nkv * ps, HD] view, or -1
      if (lane >= boxes || t >= n_tiles) return -1;
      const int key = jb0 + t * KT + lane * box_rows;
      const int pg = key / ps;
      // beyond the request's pages (keys that no row sees): any valid page will do, they are masked
      const int page = (pg < a.table_stride && key < kv_len) ? max(table[pg], 0) : 0;
      return (page * a.nkv + kvh) * ps + key % ps;
    };
    int row_next = box_row(0);
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % STAGES, j = t / STAGES;
      const int row = row_next;
      row_next = box_row(t + 1);
      if (!mbar_wait(&empty_bar[s], (j & 1) ^ 1, a.err_flag, 11)) break;
      if (lane == 0) mbar_expect_tx(&full_bar[s], 2 * TILE_BYTES);
      __syncwarp();
      if (row >= 0) {
        uint8_t* kt = tiles + s * 2 * TILE_BYTES + lane * box_rows * 128;
        uint8_t* vt = kt + TILE_BYTES;
#pragma unroll
        for (int p = 0; p < PANELS; ++p) {
          tma_load_2d_hint(kt + p * (KT * 128), &map_k, &full_bar[s], p * 64, row, stream_once);
          tma_load_2d_hint(vt + p * (KT * 128), &map_v, &full_bar[s], p * 64, row, stream_once);
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- consumers: warp w takes keys [16 w, 16 w + 16) of every tile ----------------
    // Each warp keeps its own running maximum, sum and output over all dims for its keys; the four
    // are merged once, after the last tile.  No warp repeats another's products.
    uint32_t qf[KS][4];
    {
      const int mi = lane >> 3;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int row = (mi & 1) * 8 + (lane & 7);
        ldsm4(qf[ks], s32(q_s + row * (HD + 8) + (ks * 2 + (mi >> 1)) * 8));
      }
    }
    const int ra = lane >> 2, rb = ra + 8;
    const int pos0 = start + min(ra, rows_total - 1) / g, pos1 = start + min(rb, rows_total - 1) / g;
    const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int lo1 = a.window > 0 ? max(0, pos1 - a.window + 1) : 0;
    const int mi = lane >> 3;
    const int k_warp = warp * KW;                     // this warp's first key within a tile
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int s = t % STAGES, j = t / STAGES;
      ok = mbar_wait(&full_bar[s], j & 1, a.err_flag, 12);
      if (!ok) break;
      const uint32_t kt = s32(tiles + s * 2 * TILE_BYTES), vt = kt + TILE_BYTES;
      const int jb = jb0 + t * KT;
      if (CAN_FUSE && a.qkv && a.write_kv && jb + k_warp + KW > start) {
        // This step's keys and values among this warp's 16 keys of the tile: no kernel has written them
        // to the cache yet, so what the TMA copy brought for their rows is stale.  The warp puts them into
        // the tile (it alone reads these rows) and into the cache for the steps to come; every position
        // belongs to one slice, one tile and one warp, so each row is written once.
        const int p_hi = min(min(kv_len, slice_hi), jb + k_warp + KW);
        for (int p = max(start, jb + k_warp); p < p_hi; ++p) {
          const int tok = q0 + (p - start);
          const bf16* src = a.qkv + ((size_t)tok * heads_total + a.nq + kvh) * HD + lane * EPL;
          const HeadVec<EPL> raw_k = *reinterpret_cast<const HeadVec<EPL>*>(src);
          const HeadVec<EPL> new_v = *reinterpret_cast<const HeadVec<EPL>*>(src + (size_t)a.nkv * HD);
          const HeadVec<EPL> new_k = norm_rotate_head<EPL>(raw_k, a.k_norm_w, a.norm_eps,
                                                           a.cos_t + (size_t)tok * (HD / 2),
                                                           a.sin_t + (size_t)tok * (HD / 2), lane);
          const size_t at = (((size_t)table[p / a.page_size] * a.nkv + kvh) * a.page_size + p % a.page_size) * HD +
                            lane * EPL;
          *reinterpret_cast<HeadVec<EPL>*>(a.k_cache + at) = new_k;
          *reinterpret_cast<HeadVec<EPL>*>(a.v_cache + at) = new_v;
          const int chunk16 = lane * EPL / 8, off = (lane * EPL % 8) * 2;
          const uint32_t ka = tile_addr(kt, p - jb, chunk16) + off, va = tile_addr(vt, p - jb, chunk16) + off;
          const uint32_t* kw = reinterpret_cast<const uint32_t*>(&new_k);
          const uint32_t* vw = reinterpret_cast<const uint32_t*>(&new_v);
#pragma unroll
          for (int i = 0; i < EPL / 2; ++i) {
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(ka + 4 * i), "r"(kw[i]) : "memory");
            asm volatile("st.shared.u32 [%0], %1;" ::"r"(va + 4 * i), "r"(vw[i]) : "memory");
          }
        }
        __syncwarp();
      }
      // scores of this warp's 16 keys
      float sc[2][4];
      sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t b[4];
        ldsm4(b, tile_addr(kt, k_warp + (mi >> 1) * 8 + (lane & 7), ks * 2 + (mi & 1)));
        mma16816(sc[0], qf[ks], b[0], b[1]);
        mma16816(sc[1], qf[ks], b[2], b[3]);
      }
      const bool need_mask = jb + KT > min(slice_hi, start + 1) || a.window > 0;
      float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float v = sc[nt][x] * a.scale_log2;
          if (need_mask) {
            const int key = jb + k_warp + nt * 8 + (lane & 3) * 2 + (x & 1);
            const int pos = x < 2 ? pos0 : pos1, lo = x < 2 ? lo0 : lo1;
            if (key > pos || key < lo || key >= slice_hi) v = -CUDART_INF_F;
          }
          sc[nt][x] = v;
          if (x < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float base0 = mn0 == -CUDART_INF_F ? 0.f : mn0, base1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
      const float alpha0 = exp2f(m0 - base0), alpha1 = exp2f(m1 - base1);
      const bool moved = mn0 != m0 || mn1 != m1;
      m0 = mn0;
      m1 = mn1;
      uint32_t pf[4];
      {
        const float p0 = exp2f(sc[0][0] - base0), p1 = exp2f(sc[0][1] - base0);
        const float p2 = exp2f(sc[0][2] - base1), p3 = exp2f(sc[0][3] - base1);
        const float p4 = exp2f(sc[1][0] - base0), p5 = exp2f(sc[1][1] - base0);
        const float p6 = exp2f(sc[1][2] - base1), p7 = exp2f(sc[1][3] - base1);
        float sum0 = (p0 + p1) + (p4 + p5), sum1 = (p2 + p3) + (p6 + p7);
        pf[0] = pack2(p0, p1);
        pf[1] = pack2(p2, p3);
        pf[2] = pack2(p4, p5);
        pf[3] = pack2(p6, p7);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        l0 = l0 * alpha0 + sum0;
        l1 = l1 * alpha1 + sum1;
      }
      if (__any_sync(0xffffffffu, moved)) {
#pragma unroll
        for (int dn = 0; dn < NT_ALL; ++dn) {
          o[dn][0] *= alpha0; o[dn][1] *= alpha0; o[dn][2] *= alpha1; o[dn][3] *= alpha1;
        }
      }
      // rows of the V tile that no query sees (past the sequence's end in its last tile, before the
      // window's start in its first) may hold anything: a zero weight times a non-finite value would
      // still poison the sum, so this warp clears those among its keys
      {
        const int bad_from = jb + KT > kv_len ? kv_len - jb : KT;             // rows [bad_from, KT)
        const int bad_to = (a.window > 0 && jb < first_key) ? first_key - jb : 0;   // rows [0, bad_to)
        if (bad_from < k_warp + KW || bad_to > k_warp) {
          for (int idx = lane; idx < KW * (HD / 8); idx += 32) {
            const int key = k_warp + idx / (HD / 8), c16 = idx % (HD / 8);
            if (key >= bad_from || key < bad_to)
              asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(tile_addr(vt, key, c16)), "r"(0) : "memory");
          }
          __syncwarp();
        }
      }
      // O += P . V over this warp's keys, all dims
#pragma unroll
      for (int dn = 0; dn < NT_ALL; dn += 2) {
        uint32_t b[4];
        ldsm4_t(b, tile_addr(vt, k_warp + (mi & 1) * 8 + (lane & 7), dn + (mi >> 1)));
        mma16816(o[dn], pf, b[0], b[1]);
        mma16816(o[dn + 1], pf, b[2], b[3]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }

    // ---------------- the four warps' shares of the block's keys are merged ----------------
    // every tile has been consumed, so the tile memory is free: [CONSUMERS][16][HD + 8] floats of
    // scaled partial outputs, then [CONSUMERS][16][2] floats of (maximum, sum)
    float* o_s = reinterpret_cast<float*>(tiles);
    float* ml_s = o_s + CONSUMERS * 16 * OS;
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");     // no warp still reads a tile
    if ((lane & 3) == 0) {
      *reinterpret_cast<float2*>(ml_s + (warp * 16 + ra) * 2) = make_float2(m0, l0);
      *reinterpret_cast<float2*>(ml_s + (warp * 16 + rb) * 2) = make_float2(m1, l1);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
    float mm0 = -CUDART_INF_F, mm1 = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < CONSUMERS; ++w) {
      mm0 = fmaxf(mm0, ml_s[(w * 16 + ra) * 2]);
      mm1 = fmaxf(mm1, ml_s[(w * 16 + rb) * 2]);
    }
    const float f0 = exp2f(m0 - (mm0 == -CUDART_INF_F ? 0.f : mm0)), f1 = exp2f(m1 - (mm1 == -CUDART_INF_F ? 0.f : mm1));
#pragma unroll
    for (int dn = 0; dn < NT_ALL; ++dn) {
      const int d = dn * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(o_s + (warp * 16 + ra) * OS + d) = make_float2(o[dn][0] * f0, o[dn][1] * f0);
      *reinterpret_cast<float2*>(o_s + (warp * 16 + rb) * OS + d) = make_float2(o[dn][2] * f1, o[dn][3] * f1);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS * 32) : "memory");
    // the block's output: the warps' shares are added in warp order
    const size_t slab = ((size_t)e * a.nkv + kvh) * a.nsplit + z;
    for (int idx = threadIdx.x; idx < rows_total * HD; idx += CONSUMERS * 32) {
      const int row = idx / HD, d = idx - row * HD;
      float mm = -CUDART_INF_F;
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) mm = fmaxf(mm, ml_s[(w * 16 + row) * 2]);
      const float base = mm == -CUDART_INF_F ? 0.f : mm;
      float ll = 0.f, oo = 0.f;
#pragma unroll
      for (int w = 0; w < CONSUMERS; ++w) {
        ll += ml_s[(w * 16 + row) * 2 + 1] * exp2f(ml_s[(w * 16 + row) * 2] - base);
        oo += o_s[(w * 16 + row) * OS + d];
      }
      if (a.nsplit == 1) {
        a.out[((size_t)(q0 + row / g) * a.nq + kvh * g + row % g) * HD + d] = __float2bfloat16_rn(ll > 0.f ? oo / ll : 0.f);
      } else if (a.clustered) {
        float* blk_o = ml_s + CONSUMERS * 16 * 2;         // [16][HD], then [16][2]: this block's slice
        blk_o[row * HD + d] = oo;
        if (d == 0) { blk_o[16 * HD + row * 2] = mm; blk_o[16 * HD + row * 2 + 1] = ll; }
      } else {
        a.part_o[(slab * 16 + row) * HD + d] = oo;
        if (d == 0) *reinterpret_cast<float2*>(a.part_ml + (slab * 16 + row) * 2) = make_float2(mm, ll);
      }
    }
  }
  const size_t slab0 = ((size_t)e * a.nkv + kvh) * a.nsplit;
  if (a.nsplit == 1) return;
  if (a.clustered) {
    // The slices of an (entry, KV head) sit in the shared memory of the cluster's blocks: block z adds
    // the elements z, z + nsplit, ... of the output in slice order, reading the other blocks' memory.
    // Every thread of every block passes both barriers (no path above returns before this point).
    const float* blk_o = reinterpret_cast<const float*>(tiles) + CONSUMERS * 16 * (OS + 2);
    const float* blk_ml = blk_o + 16 * HD;
    cluster_sync();
    const uint32_t n = (uint32_t)a.nsplit;
    for (int idx = z * THREADS + threadIdx.x; idx < rows_total * HD; idx += (int)n * THREADS) {
      const int row = idx / HD, d = idx - row * HD;
      float mm = -CUDART_INF_F;
      for (uint32_t sl = 0; sl < n; ++sl) mm = fmaxf(mm, peer_f32(blk_ml + row * 2, sl));
      const float base = mm == -CUDART_INF_F ? 0.f : mm;
      float ll = 0.f, oo = 0.f;
      for (uint32_t sl = 0; sl < n; ++sl) {
        const float f = exp2f(peer_f32(blk_ml + row * 2, sl) - base);
        ll += peer_f32(blk_ml + row * 2 + 1, sl) * f;
        oo += peer_f32(blk_o + row * HD + d, sl) * f;
      }
      a.out[((size_t)(q0 + row / g) * a.nq + kvh * g + row % g) * HD + d] = __float2bfloat16_rn(ll > 0.f ? oo / ll : 0.f);
    }
    cluster_sync();                       // nobody leaves while another block still reads its memory
    return;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* counter = a.slice_counters + e * a.nkv + kvh;
    const int prev = atomicAdd(counter, 1);
    is_last = prev == a.nsplit - 1;
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // The last block of an (entry, KV head) adds the slices in slice order.  First a warp per row: lane s
  // takes slice s's (maximum, sum) and the row's weights exp2(m_s - max) / total go to shared memory;
  // then every thread adds its elements with the loads of all slices in flight together.
  float* fac = reinterpret_cast<float*>(tiles);            // [16][32]
  for (int row = warp; row < rows_total; row += THREADS / 32) {
    float m = -CUDART_INF_F, l = 0.f;
    if (lane < a.nsplit) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml + ((slab0 + lane) * 16 + row) * 2));
      m = ml.x;
      l = ml.y;
    }
    const float mm = warp_max(m);
    const float f = exp2f(m - (mm == -CUDART_INF_F ? 0.f : mm));
    const float ll = warp_sum(l * f);
    fac[row * 32 + lane] = ll > 0.f ? f / ll : 0.f;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < rows_total * HD; idx += THREADS) {
    const int row = idx / HD, d = idx - row * HD;
    float oo = 0.f;
    int sl = 0;
    for (; sl + 4 <= a.nsplit; sl += 4) {
      const float v0 = __ldcg(&a.part_o[((slab0 + sl) * 16 + row) * HD + d]);
      const float v1 = __ldcg(&a.part_o[((slab0 + sl + 1) * 16 + row) * HD + d]);
      const float v2 = __ldcg(&a.part_o[((slab0 + sl + 2) * 16 + row) * HD + d]);
      const float v3 = __ldcg(&a.part_o[((slab0 + sl + 3) * 16 + row) * HD + d]);
      oo += v0 * fac[row * 32 + sl];
      oo += v1 * fac[row * 32 + sl + 1];
      oo += v2 * fac[row * 32 + sl + 2];
      oo += v3 * fac[row * 32 + sl + 3];
    }
    for (; sl < a.nsplit; ++sl) oo += __ldcg(&a.part_o[((slab0 + sl) * 16 + row) * HD + d]) * fac[row * 32 + sl];
    a.out[((size_t)(q0 + row / g) * a.nq + kvh * g + row % g) * HD + d] = __float2bfloat16_rn(oo);
  }
}

// ---------------------------------------------------------------------------
// Rows-split attention with the same TMA page loads, for many rows per entry (prefill, mixed
// batches): a block takes 128 rows (query tokens x query heads of one KV group) of one entry and
// one KV head; eight consumer warps of 16 rows each share the key/value tiles that the producer
// thread brings in; every warp keeps its rows' whole output in registers.
// ---------------------------------------------------------------------------
constexpr int ROWS_CONSUMERS = 8;
constexpr int ROWS_STAGES = 3;           // one block per SM (its registers fill the SM): a deeper ring instead
constexpr int ROWS_THREADS = (ROWS_CONSUMERS + 1) * 32;
constexpr int ROWS_PER_BLOCK = ROWS_CONSUMERS * 16;

struct RowsArgs {
  const bf16* q;
  bf16* out;
  const int* block_table;
  int table_stride;
  const int* cu_q;
  const int* kv_lens;
  const int* work;            // (entry, tile of 128 rows) pairs
  int nq, nkv, hd, page_size;
  float scale_log2;
  int window;
  int* err_flag;
};

template <int HD>
__global__ void __launch_bounds__(ROWS_THREADS, 1)
attention_rows_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                          const RowsArgs a) {
  constexpr int PANELS = HD / 64;
  constexpr int TILE_BYTES = KT * HD * 2;
  constexpr int KS = HD / 16;
  constexpr int NT_O = HD / 8;
  extern __shared__ uint8_t dec_smem_raw[];
  uint8_t* smem = dec_smem_raw + ((1024u - (s32(dec_smem_raw) & 1023u)) & 1023u);
  uint8_t* tiles = smem;                                                  // [ROWS_STAGES][K tile | V tile]
  bf16* q_s = reinterpret_cast<bf16*>(smem + ROWS_STAGES * 2 * TILE_BYTES);    // [128][HD + 8]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(q_s + ROWS_PER_BLOCK * (HD + 8));
  uint64_t* empty_bar = full_bar + ROWS_STAGES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ROWS_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], ROWS_CONSUMERS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  pdl_wait();
  pdl_trigger();
  const int e = a.work[2 * blockIdx.x], rt = a.work[2 * blockIdx.x + 1], kvh = blockIdx.y;
  const int g = a.nq / a.nkv;
  const int q0 = a.cu_q[e], q_len = a.cu_q[e + 1] - q0, kv_len = a.kv_lens[e], start = kv_len - q_len;
  const int rows_total = q_len * g;
  const int* table = a.block_table + (size_t)e * a.table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int r_first = rt * ROWS_PER_BLOCK;
  const int r_last = min(rows_total, r_first + ROWS_PER_BLOCK) - 1;
  const int n_keys = start + r_last / g + 1;                             // keys the last row sees
  const int pos_first = start + r_first / g;
  const int first_key = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
  const int jb0 = (first_key / KT) * KT;
  const int n_tiles = (n_keys - jb0 + KT - 1) / KT;

  for (int idx = threadIdx.x; idx < ROWS_PER_BLOCK * (HD / 8); idx += ROWS_THREADS) {
    const int row = idx / (HD / 8), c = idx % (HD / 8);
    const int r = r_first + row;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows_total)
      v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(q0 + r / g) * a.nq + kvh * g + r % g) * HD + c * 8);
    *reinterpret_cast<uint4*>(q_s + row * (HD + 8) + c * 8) = v;
  }
  __syncthreads();

  if (warp == ROWS_CONSUMERS) {
    if (lane == 0) {
      const int ps = a.page_size;
      const int box_rows = ps < KT ? ps : KT;
      const int boxes = KT / box_rows;
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % ROWS_STAGES, j = t / ROWS_STAGES;
        if (!mbar_wait(&empty_bar[s], (j & 1) ^ 1, a.err_flag, 31)) break;
        mbar_expect_tx(&full_bar[s], 2 * TILE_BYTES);
        uint8_t* kt = tiles + s * 2 * TILE_BYTES;
        uint8_t* vt = kt + TILE_BYTES;
        const int jb = jb0 + t * KT;
        for (int b = 0; b < boxes; ++b) {
          const int key = jb + b * box_rows;
          const int pg = key / ps;
          const int page = (pg < a.table_stride && key < kv_len) ? max(table[pg], 0) : 0;
          const int row = (page * a.nkv + kvh) * ps + key % ps;
#pragma unroll
          for (int p = 0; p < PANELS; ++p) {
            tma_load_2d(kt + p * (KT * 128) + b * box_rows * 128, &map_k, &full_bar[s], p * 64, row);
            tma_load_2d(vt + p * (KT * 128) + b * box_rows * 128, &map_v, &full_bar[s], p * 64, row);
          }
        }
      }
    }
    __syncwarp();
    return;
  }

  // ---------------- consumers: 16 rows each ----------------
  const int mi = lane >> 3;
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int row = warp * 16 + (mi & 1) * 8 + (lane & 7);
    ldsm4(qf[ks], s32(q_s + row * (HD + 8) + (ks * 2 + (mi >> 1)) * 8));
  }
  float o[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
  const int ra = r_first + warp * 16 + (lane >> 2), rb = ra + 8;
  const int pos0 = start + min(ra, rows_total - 1) / g, pos1 = start + min(rb, rows_total - 1) / g;
  const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int lo1 = a.window > 0 ? max(0, pos1 - a.window + 1) : 0;
  const int warp_pos_max = start + min(r_first + warp * 16 + 15, rows_total - 1) / g;
  const int warp_pos_min = start + min(r_first + warp * 16, rows_total - 1) / g;
  const int warp_lo = a.window > 0 ? max(0, warp_pos_max - a.window + 1) : 0;   // first key any row of the warp sees... of its last row
  const int warp_lo_min = a.window > 0 ? max(0, warp_pos_min - a.window + 1) : 0;
  const bool warp_live = r_first + warp * 16 < rows_total;

  bool ok = true;
  for (int t = 0; t < n_tiles && ok; ++t) {
    const int s = t % ROWS_STAGES, j = t / ROWS_STAGES;
    ok = mbar_wait(&full_bar[s], j & 1, a.err_flag, 32);
    if (!ok) break;
    const uint32_t kt = s32(tiles + s * 2 * TILE_BYTES), vt = kt + TILE_BYTES;
    const int jb = jb0 + t * KT;
    if (jb + KT > kv_len || (a.window > 0 && jb < first_key)) {
      // rows of the V tile that hold no key of this request may contain anything; a zero weight times
      // a non-finite value would poison the sum.  Every warp clears them all (the same zeros) before it reads.
      const int bad_from = jb + KT > kv_len ? kv_len - jb : KT;
      const int bad_to = (a.window > 0 && jb < first_key) ? first_key - jb : 0;
      for (int idx = lane; idx < KT * (HD / 8); idx += 32) {
        const int key = idx / (HD / 8), c16 = idx % (HD / 8);
        if (key >= bad_from || key < bad_to)
          asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(tile_addr(vt, key, c16)), "r"(0) : "memory");
      }
      __syncwarp();
    }
    if (warp_live && jb <= warp_pos_max && jb + KT > warp_lo_min) {
      float sc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int nt = 0; nt < 8; nt += 2) {
          uint32_t b[4];
          ldsm4(b, tile_addr(kt, (nt + (mi >> 1)) * 8 + (lane & 7), ks * 2 + (mi & 1)));
          mma16816(sc[nt], qf[ks], b[0], b[1]);
          mma16816(sc[nt + 1], qf[ks], b[2], b[3]);
        }
      }
      // a tile needs the mask unless every key of it is visible to every row of the warp
      const bool need_mask = jb + KT - 1 > warp_pos_min || jb < warp_lo || jb + KT > n_keys;
      float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float v = sc[nt][x] * a.scale_log2;
          if (need_mask) {
            const int key = jb + nt * 8 + (lane & 3) * 2 + (x & 1);
            const int pos = x < 2 ? pos0 : pos1, lo = x < 2 ? lo0 : lo1;
            if (key > pos || key < lo) v = -CUDART_INF_F;
          }
          sc[nt][x] = v;
          if (x < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float base0 = mn0 == -CUDART_INF_F ? 0.f : mn0, base1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
      const float alpha0 = exp2f(m0 - base0), alpha1 = exp2f(m1 - base1);
      m0 = mn0;
      m1 = mn1;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pf[4][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const float p0 = exp2f(sc[nt][0] - base0), p1 = exp2f(sc[nt][1] - base0);
        const float p2 = exp2f(sc[nt][2] - base1), p3 = exp2f(sc[nt][3] - base1);
        sum0 += p0 + p1;
        sum1 += p2 + p3;
        pf[nt >> 1][(nt & 1) * 2 + 0] = pack2(p0, p1);
        pf[nt >> 1][(nt & 1) * 2 + 1] = pack2(p2, p3);
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      l0 = l0 * alpha0 + sum0;
      l1 = l1 * alpha1 + sum1;
#pragma unroll
      for (int dn = 0; dn < NT_O; ++dn) {
        o[dn][0] *= alpha0; o[dn][1] *= alpha0; o[dn][2] *= alpha1; o[dn][3] *= alpha1;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int dn = 0; dn < NT_O; dn += 2) {
          uint32_t b[4];
          ldsm4_t(b, tile_addr(vt, kk * 16 + (mi & 1) * 8 + (lane & 7), dn + (mi >> 1)));
          mma16816(o[dn], pf[kk], b[0], b[1]);
          mma16816(o[dn + 1], pf[kk], b[2], b[3]);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
  }
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
  for (int dn = 0; dn < NT_O; ++dn) {
    const int d = dn * 8 + (lane & 3) * 2;
    if (ra < rows_total)
      *reinterpret_cast<uint32_t*>(a.out + ((size_t)(q0 + ra / g) * a.nq + kvh * g + ra % g) * HD + d) =
          pack2(o[dn][0] * inv0, o[dn][1] * inv0);
    if (rb < rows_total)
      *reinterpret_cast<uint32_t*>(a.out + ((size_t)(q0 + rb / g) * a.nq + kvh * g + rb % g) * HD + d) =
          pack2(o[dn][2] * inv1, o[dn][3] * inv1);
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
  const void* ptr; long long rows; int hd, box_rows;
  bool operator<(const Key& o) const { return std::tie(ptr, rows, hd, box_rows) < std::tie(o.ptr, o.rows, o.hd, o.box_rows); }
};
static std::map<Key, CUtensorMap> g_maps;
static std::mutex g_mutex;

// the cache as a matrix [rows = pages * kv_heads * page_size, head_dim]; box = [box_rows, 64 dims]
// (copied into *out under the lock: no pointer into the cache of maps leaves this function)
static bool cache_map(CUtensorMap* out, const void* ptr, long long rows, int hd, int box_rows) {
  std::lock_guard<std::mutex> lock(g_mutex);
  Key key{ptr, rows, hd, box_rows};
  auto it = g_maps.find(key);
  if (it != g_maps.end()) { *out = it->second; return true; }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
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

template <int HD>
static int launch(const CUtensorMap* mk, const CUtensorMap* mv, const Args& a, int n_entries, cudaStream_t stream) {
  constexpr int SMEM = STAGES * 2 * KT * HD * 2 + 16 * (HD + 8) * 2 + 2 * STAGES * 8 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_decode_tma_kernel<HD>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (err != cudaSuccess) return refuse((int)err, "attention_decode_tma: cannot get %d bytes of shared memory", SMEM);
    configured = true;
  }
  if (!a.clustered) {
    launch_pdl(attention_decode_tma_kernel<HD>, dim3(n_entries, a.nkv, a.nsplit), dim3(THREADS), SMEM, stream, *mk,
               *mv, a);
    return launched();
  }
  // the slices of an (entry, KV head) as one thread-block cluster along z
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_entries, a.nkv, a.nsplit);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = a.nsplit;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaLaunchKernelEx(&cfg, attention_decode_tma_kernel<HD>, *mk, *mv, a);
  return launched();
}

template <int HD>
static int launch_rows(const CUtensorMap* mk, const CUtensorMap* mv, const RowsArgs& a, int n_work, cudaStream_t stream) {
  constexpr int SMEM = ROWS_STAGES * 2 * KT * HD * 2 + ROWS_PER_BLOCK * (HD + 8) * 2 + 2 * ROWS_STAGES * 8 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_rows_tma_kernel<HD>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (err != cudaSuccess) return refuse((int)err, "attention_rows_tma: cannot get %d bytes of shared memory", SMEM);
    configured = true;
  }
  launch_pdl(attention_rows_tma_kernel<HD>, dim3(n_work, a.nkv), dim3(ROWS_THREADS), SMEM, stream, *mk, *mv, a);
  return launched();
}

}  // namespace dec
}  // namespace srlm

using namespace srlm;

// 1 if srlm_paged_attention_decode_tma takes these sizes.
extern "C" int srlm_attention_decode_tma_takes(int hd, int page_size) {
  const bool hd_ok = hd == 64 || hd == 128 || hd == 192 || hd == 256;
  const bool ps_ok = page_size == 8 || page_size == 16 || page_size == 32 || (page_size > 0 && page_size % 64 == 0);
  return hd_ok && ps_ok;
}

// Same contract as srlm_paged_attention_keys (attention_mma.cu); num_pages is the pool's page count.
namespace srlm {
namespace dec {
struct FusedInputs {          // see Args: all null / zero when q is given
  const void* qkv;
  const float* q_norm_w;
  const float* k_norm_w;
  float eps;
  const float* cos_t;
  const float* sin_t;
  int write_kv;
};
static int decode_entry(const void* q, const FusedInputs& f, const void* k_cache, const void* v_cache, void* out,
                        long long num_pages, const int* block_table, int table_stride, const int* cu_q,
                        const int* kv_lens, int n_entries, int nq, int nkv, int hd, int page_size, float scale,
                        int window, int kv_chunk, int nsplit, float* part_o, float* part_ml, int* slice_counters,
                        int cluster, int* err_flag, cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  if (!srlm_attention_decode_tma_takes(hd, page_size) || nq <= 0 || nkv <= 0 || nq % nkv)
    return refuse(ST_BAD_SIZE, "attention_decode_tma: nq=%d nkv=%d hd=%d page_size=%d", nq, nkv, hd, page_size);
  if (f.qkv && ((hd != 64 && hd != 128 && hd != 256) || !f.cos_t || !f.sin_t || ((uintptr_t)f.qkv & 15)))
    return refuse(ST_BAD_SIZE, "attention_decode_tma: the fused form takes head_dim 64, 128 or 256 with a rotation "
                  "over the whole head (head_dim %d)", hd);
  // up to 8 slices (the portable cluster size) can merge through distributed shared memory; more, or
  // cluster == 0, go through part_o / part_ml and the counters
  const int clustered = cluster && nsplit > 1 && nsplit <= 8;
  if (nsplit < 1 || kv_chunk <= 0 || kv_chunk % KT ||
      (nsplit > 1 && !clustered && (!part_o || !part_ml || !slice_counters)))
    return refuse(ST_BAD_SIZE, "attention_decode_tma: nsplit=%d kv_chunk=%d", nsplit, kv_chunk);
  if (nsplit > 32 || nkv > 65535)
    return refuse(ST_BAD_SIZE, "attention_decode_tma: nsplit=%d nkv=%d (at most 32 slices: the merge gives a lane to each)",
                  nsplit, nkv);
  const int box_rows = page_size < KT ? page_size : KT;
  const long long rows = num_pages * nkv * page_size;
  CUtensorMap mk_copy, mv_copy;
  const CUtensorMap *mk = &mk_copy, *mv = &mv_copy;
  if (!cache_map(&mk_copy, k_cache, rows, hd, box_rows) || !cache_map(&mv_copy, v_cache, rows, hd, box_rows))
    return refuse(ST_BAD_SIZE, "attention_decode_tma: cuTensorMapEncodeTiled refused the cache");
  Args a{(const bf16*)q, (bf16*)out, block_table, table_stride, cu_q, kv_lens, nq, nkv, hd, page_size,
         scale * 1.4426950408889634f, window, kv_chunk, nsplit, clustered, part_o, part_ml, slice_counters,
         err_flag, (const bf16*)f.qkv, f.q_norm_w, f.k_norm_w, f.eps, f.cos_t, f.sin_t,
         (bf16*)const_cast<void*>(k_cache), (bf16*)const_cast<void*>(v_cache), f.write_kv};
  switch (hd) {
    case 64: return launch<64>(mk, mv, a, n_entries, stream);
    case 128: return launch<128>(mk, mv, a, n_entries, stream);
    case 192: return launch<192>(mk, mv, a, n_entries, stream);
    default: return launch<256>(mk, mv, a, n_entries, stream);
  }
}
}  // namespace dec
}  // namespace srlm

extern "C" int srlm_paged_attention_decode_tma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                               long long num_pages, const int* block_table, int table_stride,
                                               const int* cu_q, const int* kv_lens, int n_entries, int nq, int nkv,
                                               int hd, int page_size, float scale, int window, int kv_chunk,
                                               int nsplit, float* part_o, float* part_ml, int* slice_counters,
                                               int cluster, int* err_flag, cudaStream_t stream) {
  const dec::FusedInputs none{nullptr, nullptr, nullptr, 0.f, nullptr, nullptr, 0};
  return dec::decode_entry(q, none, k_cache, v_cache, out, num_pages, block_table, table_stride, cu_q, kv_lens,
                           n_entries, nq, nkv, hd, page_size, scale, window, kv_chunk, nsplit, part_o, part_ml,
                           slice_counters, cluster, err_flag, stream);
}

// The same with the step before it folded in: q and this step's keys and values come from qkv
// [tokens, (nq + 2 nkv) * hd], the output of the q/k/v projection.  Per-head RMSNorm of q and k with
// q_norm_w / k_norm_w [hd] (null: none) and eps, rotation of the pairs (i, i + hd/2) by cos_t / sin_t
// [tokens, hd/2]; with write_kv the new keys and values are written to the cache (without it the cache
// must already hold them).  head_dim 64, 128 or 256.
extern "C" int srlm_paged_attention_decode_fused(const void* qkv, const float* q_norm_w, const float* k_norm_w,
                                                 float eps, const float* cos_t, const float* sin_t, int write_kv,
                                                 void* k_cache, void* v_cache, void* out, long long num_pages,
                                                 const int* block_table, int table_stride, const int* cu_q,
                                                 const int* kv_lens, int n_entries, int nq, int nkv, int hd,
                                                 int page_size, float scale, int window, int kv_chunk, int nsplit,
                                                 float* part_o, float* part_ml, int* slice_counters, int cluster,
                                                 int* err_flag, cudaStream_t stream) {
  if (!qkv) return refuse(ST_BAD_SIZE, "attention_decode_fused: no qkv");
  const dec::FusedInputs f{qkv, q_norm_w, k_norm_w, eps, cos_t, sin_t, write_kv ? 1 : 0};
  return dec::decode_entry(nullptr, f, k_cache, v_cache, out, num_pages, block_table, table_stride, cu_q, kv_lens,
                           n_entries, nq, nkv, hd, page_size, scale, window, kv_chunk, nsplit, part_o, part_ml,
                           slice_counters, cluster, err_flag, stream);
}

// Ragged batch with TMA page loads.  work: n_work pairs (entry, tile of 128 rows); an entry with q tokens has
// ceil(q * (nq/nkv) / 128) tiles.  Same size rules as srlm_paged_attention_decode_tma (head_dim 64 or 128 here).
extern "C" int srlm_paged_attention_rows_tma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                             long long num_pages, const int* block_table, int table_stride,
                                             const int* cu_q, const int* kv_lens, const int* work, int n_work, int nq,
                                             int nkv, int hd, int page_size, float scale, int window, int* err_flag,
                                             cudaStream_t stream) {
  if (n_work <= 0) return ST_OK;
  if (!srlm_attention_decode_tma_takes(hd, page_size) || hd > 128 || nq <= 0 || nkv <= 0 || nq % nkv)
    return refuse(ST_BAD_SIZE, "attention_rows_tma: nq=%d nkv=%d hd=%d page_size=%d", nq, nkv, hd, page_size);
  const int box_rows = page_size < dec::KT ? page_size : dec::KT;
  const long long rows = num_pages * nkv * page_size;
  CUtensorMap mk_copy, mv_copy;
  const CUtensorMap *mk = &mk_copy, *mv = &mv_copy;
  if (!dec::cache_map(&mk_copy, k_cache, rows, hd, box_rows) || !dec::cache_map(&mv_copy, v_cache, rows, hd, box_rows))
    return refuse(ST_BAD_SIZE, "attention_rows_tma: cuTensorMapEncodeTiled refused the cache");
  dec::RowsArgs a{(const bf16*)q, (bf16*)out, block_table, table_stride, cu_q, kv_lens, work, nq, nkv, hd, page_size,
                  scale * 1.4426950408889634f, window, err_flag};
  return hd == 64 ? dec::launch_rows<64>(mk, mv, a, n_work, stream) : dec::launch_rows<128>(mk, mv, a, n_work, stream);
}
