// Paged causal attention for bfloat16 on the tensor cores (warp-level
// mma.sync m16n8k16, float32 accumulation, flash-style online softmax).
//
// The query heads of one KV group are stacked as rows: row r of an entry is
// (token r / g, head kh*g + r % g), so each key/value byte of a KV head is read
// once for all g query heads that share it.
//
//  * rows-split kernel (prefill, mixed batches): a block takes 64 rows of one
//    entry and one KV head, 16 rows per warp, and walks the keys in tiles of 64
//    loaded with cp.async through the block table.
//  * keys-split kernel (decode: at most 16 rows per entry and KV head): a block
//    takes one entry, one KV head and one slice of the keys; its four warps
//    share the 16 rows and each takes 16 keys of every tile; the warps' partial
//    results are merged in shared memory, and the slices' by whichever block of an
//    (entry, KV head) finishes last.
//
// Softmax, its running maximum and sum, and the output accumulation are
// float32.  Formula: src/model/math.rs:102-155.
#include <math_constants.h>

#include "common.cuh"

namespace srlm {

constexpr int KT = 64;                 // keys per tile
constexpr int ATT_THREADS = 128;
constexpr int ROWS_PER_BLOCK = 64;

struct AttnArgs {
  const bf16* q;
  const bf16* k_cache;
  const bf16* v_cache;
  bf16* out;
  const int* block_table;
  int table_stride;
  const int* cu_q;
  const int* kv_lens;
  const int* work;          // rows-split: (entry, row tile) pairs
  int nq, nkv, hd, page_size;
  float scale_log2;         // softmax scale * log2(e)
  int window;
  int kv_chunk;             // keys-split: keys per slice (multiple of KT)
  int nsplit;
  float* part_o;            // keys-split with nsplit > 1: [entry, kv head, slice, 16, hd]
  float* part_ml;           //                             [entry, kv head, slice, 16, 2]
  int* slice_counters;      //                             [entry, kv head], zero on entry, left zero
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;      // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Loads keys [jb, jb+KT) of one KV head into a K tile and a V tile, each [KT][stride] (bf16); keys
// outside [first_key, n_keys) become zeros.  One block-table lookup serves both tiles.
__device__ __forceinline__ void load_kv_tiles(bf16* k_tile, bf16* v_tile, const int* table, int jb,
                                              int first_key, int n_keys, int kvh, const AttnArgs& a,
                                              int stride) {
  const int chunks = a.hd >> 3;                       // 16-byte chunks per row
  const bool pow2 = (a.page_size & (a.page_size - 1)) == 0;
  const int shift = 31 - __clz(a.page_size);
  auto one = [&](int key, int c) {
    const int j = jb + key;
    const bool valid = j >= first_key && j < n_keys;
    size_t off = 0;
    if (valid) {
      const int pg = pow2 ? (j >> shift) : (j / a.page_size);
      const int in_page = j - pg * a.page_size;
      off = (((size_t)table[pg] * a.nkv + kvh) * a.page_size + in_page) * a.hd + c * 8;
    }
    cp_async_16(k_tile + key * stride + c * 8, a.k_cache + off, valid);
    cp_async_16(v_tile + key * stride + c * 8, a.v_cache + off, valid);
  };
  if ((chunks & (chunks - 1)) == 0) {                 // head sizes 16, 32, 64, 128, 256: shifts only
    const int cs = 31 - __clz(chunks);
    const int c = threadIdx.x & (chunks - 1), k0 = threadIdx.x >> cs, kstep = ATT_THREADS >> cs;
    for (int key = k0; key < KT; key += kstep) one(key, c);
  } else {
    for (int idx = threadIdx.x; idx < KT * chunks; idx += ATT_THREADS) one(idx / chunks, idx % chunks);
  }
}

// One 16-row slab against `nkeys16` groups of 16 keys starting at key offset `key0` of the tile.
// S (scaled, masked) -> online softmax -> O += P V.
template <int HD_MAX, int NT_S>   // NT_S: n-tiles of 8 keys this warp handles per tile (8 or 2)
struct WarpTile {
  static constexpr int KS = HD_MAX / 16;      // k steps over the head dimension
  static constexpr int NT_O = HD_MAX / 8;     // output n-tiles
  uint32_t qf[KS][4];
  float o[NT_O][4];
  float m[2], l[2];

  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < NT_O; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    m[0] = m[1] = -CUDART_INF_F;
    l[0] = l[1] = 0.f;
  }

  __device__ __forceinline__ void load_q(const bf16* qs, int stride, int hd, int row0) {
    const int lane = threadIdx.x & 31, mi = lane >> 3;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      if (ks * 16 < hd) {
        const int row = row0 + (mi & 1) * 8 + (lane & 7);
        ldmatrix_x4(qf[ks], qs + row * stride + (ks * 2 + (mi >> 1)) * 8);
      }
    }
  }

  // ks_tile/vs_tile: the K and V tiles; key0: first key of this warp's keys within the tile;
  // jb: global index of the tile's first key; pos0/pos1: positions of the thread's two rows;
  // lo0/lo1: first visible key of each row.
  __device__ __forceinline__ void step(const bf16* ks_tile, const bf16* vs_tile, int stride, int hd, int key0,
                                       int jb, int pos0, int pos1, int lo0, int lo1, float scale_log2,
                                       bool need_mask) {
    const int lane = threadIdx.x & 31, mi = lane >> 3;
    float s[NT_S][4];
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      if (ks * 16 < hd) {
#pragma unroll
        for (int nt = 0; nt < NT_S; nt += 2) {
          uint32_t b[4];
          const int key = key0 + (nt + (mi >> 1)) * 8 + (lane & 7);
          ldmatrix_x4(b, ks_tile + key * stride + (ks * 2 + (mi & 1)) * 8);
          mma_bf16(s[nt], qf[ks], b[0], b[1]);
          mma_bf16(s[nt + 1], qf[ks], b[2], b[3]);
        }
      }
    }
    // scale, mask, row maxima
    float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F;
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nt][e] * scale_log2;
        if (need_mask) {
          const int j = jb + key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int pos = (e < 2) ? pos0 : pos1, lo = (e < 2) ? lo0 : lo1;
          if (j > pos || j < lo) v = -CUDART_INF_F;
        }
        s[nt][e] = v;
        if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float base0 = mn0 == -CUDART_INF_F ? 0.f : mn0, base1 = mn1 == -CUDART_INF_F ? 0.f : mn1;
    const float alpha0 = exp2f(m[0] - base0), alpha1 = exp2f(m[1] - base1);
    m[0] = mn0;
    m[1] = mn1;
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pf[NT_S / 2][4];
#pragma unroll
    for (int nt = 0; nt < NT_S; ++nt) {
      const float p0 = exp2f(s[nt][0] - base0), p1 = exp2f(s[nt][1] - base0);
      const float p2 = exp2f(s[nt][2] - base1), p3 = exp2f(s[nt][3] - base1);
      sum0 += p0 + p1;
      sum1 += p2 + p3;
      pf[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
    sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
    sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
    l[0] = l[0] * alpha0 + sum0;
    l[1] = l[1] * alpha1 + sum1;
#pragma unroll
    for (int dn = 0; dn < NT_O; ++dn) {
      o[dn][0] *= alpha0; o[dn][1] *= alpha0; o[dn][2] *= alpha1; o[dn][3] *= alpha1;
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < NT_S / 2; ++kk) {
#pragma unroll
      for (int dn = 0; dn < NT_O; dn += 2) {
        if (dn * 8 < hd) {
          uint32_t b[4];
          const int key = key0 + kk * 16 + (mi & 1) * 8 + (lane & 7);
          ldmatrix_x4_trans(b, vs_tile + key * stride + (dn + (mi >> 1)) * 8);
          mma_bf16(o[dn], pf[kk], b[0], b[1]);
          mma_bf16(o[dn + 1], pf[kk], b[2], b[3]);
        }
      }
    }
  }
};

// ---------------------------------------------------------------------------
// rows-split kernel
// ---------------------------------------------------------------------------
template <int HD_MAX>
__global__ void __launch_bounds__(ATT_THREADS)
attention_rows_kernel(const AttnArgs a) {
  extern __shared__ __align__(16) uint8_t att_smem[];
  const int stride = a.hd + 8;                           // padded rows: no ldmatrix bank conflicts
  bf16* q_s = reinterpret_cast<bf16*>(att_smem);
  bf16* kv_s = q_s + ROWS_PER_BLOCK * stride;            // [2 stages][K tile | V tile]
  const int tile_elems = KT * stride;

  pdl_wait();
  pdl_trigger();
  const int e = a.work[2 * blockIdx.x], rt = a.work[2 * blockIdx.x + 1], kvh = blockIdx.y;
  const int g = a.nq / a.nkv;
  const int q0 = a.cu_q[e], q_len = a.cu_q[e + 1] - q0, kv_len = a.kv_lens[e], start = kv_len - q_len;
  const int rows_total = q_len * g;
  const int* table = a.block_table + (size_t)e * a.table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Q rows of this block -> shared memory (zeros beyond the entry's rows)
  const int chunks = a.hd >> 3;
  for (int idx = threadIdx.x; idx < ROWS_PER_BLOCK * chunks; idx += ATT_THREADS) {
    const int row = idx / chunks, c = idx - row * chunks;
    const int r = rt * ROWS_PER_BLOCK + row;
    const bool valid = r < rows_total;
    const bf16* src = a.q;
    if (valid) src = a.q + ((size_t)(q0 + r / g) * a.nq + kvh * g + r % g) * a.hd + c * 8;
    cp_async_16(q_s + row * stride + c * 8, src, valid);
  }
  const int r_first = rt * ROWS_PER_BLOCK;
  const int r_last = min(rows_total, r_first + ROWS_PER_BLOCK) - 1;
  const int n_keys = start + r_last / g + 1;                              // keys the last row sees
  const int pos_first = start + r_first / g;
  const int first_key = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
  const int jb0 = (first_key / KT) * KT;
  const int n_tiles = (n_keys - jb0 + KT - 1) / KT;

  load_kv_tiles(kv_s, kv_s + tile_elems, table, jb0, first_key, n_keys, kvh, a, stride);
  cp_async_commit();

  WarpTile<HD_MAX, 8> wt;
  wt.init();
  // this thread's two rows
  const int ra = r_first + warp * 16 + (lane >> 2), rb = ra + 8;
  const int pos0 = start + min(ra, rows_total - 1) / g, pos1 = start + min(rb, rows_total - 1) / g;
  const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int lo1 = a.window > 0 ? max(0, pos1 - a.window + 1) : 0;
  const int warp_pos_max = start + min(r_first + warp * 16 + 15, rows_total - 1) / g;
  const int warp_pos_min = start + min(r_first + warp * 16, rows_total - 1) / g;
  const bool warp_live = r_first + warp * 16 < rows_total;

  for (int t = 0; t < n_tiles; ++t) {
    const int jb = jb0 + t * KT;
    bf16* cur = kv_s + (t & 1) * 2 * tile_elems;
    if (t + 1 < n_tiles) {
      bf16* nxt = kv_s + ((t + 1) & 1) * 2 * tile_elems;
      load_kv_tiles(nxt, nxt + tile_elems, table, jb + KT, first_key, n_keys, kvh, a, stride);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (t == 0) wt.load_q(q_s, stride, a.hd, warp * 16);
    if (warp_live && jb <= warp_pos_max) {
      // a tile needs the mask unless every key of it is visible to every row of the warp
      const int warp_lo = a.window > 0 ? max(0, warp_pos_max - a.window + 1) : 0;
      const bool need_mask = jb + KT - 1 > warp_pos_min || jb < warp_lo || jb + KT > n_keys;
      wt.step(cur, cur + tile_elems, stride, a.hd, 0, jb, pos0, pos1, lo0, lo1, a.scale_log2, need_mask);
    }
    __syncthreads();
  }
  // write the rows out
  const float inv0 = wt.l[0] > 0.f ? 1.f / wt.l[0] : 0.f, inv1 = wt.l[1] > 0.f ? 1.f / wt.l[1] : 0.f;
#pragma unroll
  for (int dn = 0; dn < WarpTile<HD_MAX, 8>::NT_O; ++dn) {
    const int d = dn * 8 + (lane & 3) * 2;
    if (d < a.hd) {
      if (ra < rows_total) {
        bf16* dst = a.out + ((size_t)(q0 + ra / g) * a.nq + kvh * g + ra % g) * a.hd + d;
        *reinterpret_cast<uint32_t*>(dst) = pack_bf16(wt.o[dn][0] * inv0, wt.o[dn][1] * inv0);
      }
      if (rb < rows_total) {
        bf16* dst = a.out + ((size_t)(q0 + rb / g) * a.nq + kvh * g + rb % g) * a.hd + d;
        *reinterpret_cast<uint32_t*>(dst) = pack_bf16(wt.o[dn][2] * inv1, wt.o[dn][3] * inv1);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// keys-split kernel (at most 16 rows per entry and KV head)
// ---------------------------------------------------------------------------
constexpr int KEYS_STAGES = 3;

template <int HD_MAX>
__global__ void __launch_bounds__(ATT_THREADS)
attention_keys_kernel(const AttnArgs a) {
  extern __shared__ __align__(16) uint8_t att_smem[];
  __shared__ int is_last;
  const int stride = a.hd + 8;
  bf16* q_s = reinterpret_cast<bf16*>(att_smem);            // [16][stride]
  bf16* kv_s = q_s + 16 * stride;                           // [stages][K tile | V tile]
  const int tile_elems = KT * stride;

  pdl_wait();
  pdl_trigger();
  const int e = blockIdx.x, kvh = blockIdx.y, z = blockIdx.z;
  const int g = a.nq / a.nkv;
  const int q0 = a.cu_q[e], q_len = a.cu_q[e + 1] - q0, kv_len = a.kv_lens[e], start = kv_len - q_len;
  const int rows_total = q_len * g;                         // <= 16
  const int* table = a.block_table + (size_t)e * a.table_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int chunks = a.hd >> 3;
  for (int idx = threadIdx.x; idx < 16 * chunks; idx += ATT_THREADS) {
    const int row = idx / chunks, c = idx - row * chunks;
    const bool valid = row < rows_total;
    const bf16* src = a.q;
    if (valid) src = a.q + ((size_t)(q0 + row / g) * a.nq + kvh * g + row % g) * a.hd + c * 8;
    cp_async_16(q_s + row * stride + c * 8, src, valid);
  }
  const int first_key = a.window > 0 ? max(0, start - a.window + 1) : 0;
  const int slice_lo = z * a.kv_chunk, slice_hi = min(kv_len, slice_lo + a.kv_chunk);
  const int jb0 = max(slice_lo, (first_key / KT) * KT);
  const int n_tiles = slice_hi > jb0 ? (slice_hi - jb0 + KT - 1) / KT : 0;

  WarpTile<HD_MAX, 2> wt;
  wt.init();
  const int ra = lane >> 2, rb = ra + 8;
  const int pos0 = start + min(ra, rows_total - 1) / g, pos1 = start + min(rb, rows_total - 1) / g;
  const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int lo1 = a.window > 0 ? max(0, pos1 - a.window + 1) : 0;

  // prologue: the first STAGES-1 tiles are in flight before the loop (one commit group per tile)
#pragma unroll
  for (int p = 0; p < KEYS_STAGES - 1; ++p) {
    if (p < n_tiles) {
      bf16* dst = kv_s + p * 2 * tile_elems;
      load_kv_tiles(dst, dst + tile_elems, table, jb0 + p * KT, first_key, slice_hi, kvh, a, stride);
    }
    cp_async_commit();
  }
  for (int t = 0; t < n_tiles; ++t) {
    const int jb = jb0 + t * KT;
    bf16* cur = kv_s + (t % KEYS_STAGES) * 2 * tile_elems;
    cp_async_wait<KEYS_STAGES - 2>();                       // tile t has landed
    __syncthreads();                                        // ... and everyone is done with tile t-1
    if (t + KEYS_STAGES - 1 < n_tiles) {
      bf16* dst = kv_s + ((t + KEYS_STAGES - 1) % KEYS_STAGES) * 2 * tile_elems;
      load_kv_tiles(dst, dst + tile_elems, table, jb + (KEYS_STAGES - 1) * KT, first_key, slice_hi, kvh, a,
                    stride);
    }
    cp_async_commit();
    if (t == 0) wt.load_q(q_s, stride, a.hd, 0);
    if (jb + warp * 16 < slice_hi) {
      const bool need_mask = jb + KT > min(slice_hi, start + 1) || a.window > 0;
      wt.step(cur, cur + tile_elems, stride, a.hd, warp * 16, jb, pos0, pos1, lo0, lo1, a.scale_log2,
              need_mask);
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  // merge the four warps: (m, l, O) of each warp -> shared memory (the tiles are no longer needed)
  float* ml_s = reinterpret_cast<float*>(kv_s);             // [4 warps][16 rows][2]
  float* o_s = ml_s + 4 * 16 * 2;                           // [4 warps][16 rows][hd]
  if ((lane & 3) == 0) {
    ml_s[(warp * 16 + ra) * 2 + 0] = wt.m[0];
    ml_s[(warp * 16 + ra) * 2 + 1] = wt.l[0];
    ml_s[(warp * 16 + rb) * 2 + 0] = wt.m[1];
    ml_s[(warp * 16 + rb) * 2 + 1] = wt.l[1];
  }
#pragma unroll
  for (int dn = 0; dn < WarpTile<HD_MAX, 2>::NT_O; ++dn) {
    const int d = dn * 8 + (lane & 3) * 2;
    if (d < a.hd) {
      o_s[(warp * 16 + ra) * a.hd + d] = wt.o[dn][0];
      o_s[(warp * 16 + ra) * a.hd + d + 1] = wt.o[dn][1];
      o_s[(warp * 16 + rb) * a.hd + d] = wt.o[dn][2];
      o_s[(warp * 16 + rb) * a.hd + d + 1] = wt.o[dn][3];
    }
  }
  __syncthreads();
  const size_t slab0 = ((size_t)e * a.nkv + kvh) * a.nsplit;
  for (int idx = threadIdx.x; idx < rows_total * a.hd; idx += ATT_THREADS) {
    const int row = idx / a.hd, d = idx - row * a.hd;
    float mm = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, ml_s[(w * 16 + row) * 2]);
    const float base = mm == -CUDART_INF_F ? 0.f : mm;
    float ll = 0.f, oo = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(ml_s[(w * 16 + row) * 2] - base);
      ll += ml_s[(w * 16 + row) * 2 + 1] * f;
      oo += o_s[(w * 16 + row) * a.hd + d] * f;
    }
    if (a.nsplit == 1) {
      a.out[((size_t)(q0 + row / g) * a.nq + kvh * g + row % g) * a.hd + d] =
          __float2bfloat16_rn(ll > 0.f ? oo / ll : 0.f);
    } else {
      a.part_o[((slab0 + z) * 16 + row) * a.hd + d] = oo;
      if (d == 0) {
        a.part_ml[((slab0 + z) * 16 + row) * 2 + 0] = mm;
        a.part_ml[((slab0 + z) * 16 + row) * 2 + 1] = ll;
      }
    }
  }
  if (a.nsplit == 1) return;
  // the last slice of this (entry, KV head) to finish merges all of them, in slice order
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
  for (int idx = threadIdx.x; idx < rows_total * a.hd; idx += ATT_THREADS) {
    const int row = idx / a.hd, d = idx - row * a.hd;
    float mm = -CUDART_INF_F;
    for (int s = 0; s < a.nsplit; ++s) mm = fmaxf(mm, __ldcg(&a.part_ml[((slab0 + s) * 16 + row) * 2]));
    const float base = mm == -CUDART_INF_F ? 0.f : mm;
    float ll = 0.f, oo = 0.f;
    for (int s = 0; s < a.nsplit; ++s) {
      const float f = exp2f(__ldcg(&a.part_ml[((slab0 + s) * 16 + row) * 2]) - base);
      ll += __ldcg(&a.part_ml[((slab0 + s) * 16 + row) * 2 + 1]) * f;
      oo += __ldcg(&a.part_o[((slab0 + s) * 16 + row) * a.hd + d]) * f;
    }
    a.out[((size_t)(q0 + row / g) * a.nq + kvh * g + row % g) * a.hd + d] =
        __float2bfloat16_rn(ll > 0.f ? oo / ll : 0.f);
  }
}

template <int HD_MAX>
static int launch_rows(const AttnArgs& a, int n_work, cudaStream_t stream) {
  const int stride = a.hd + 8;
  const size_t smem = (size_t)(ROWS_PER_BLOCK + 4 * KT) * stride * 2;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attention_rows_kernel<HD_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (ROWS_PER_BLOCK + 4 * KT) * (HD_MAX + 8) * 2);
    configured = true;
  }
  launch_pdl(attention_rows_kernel<HD_MAX>, dim3(n_work, a.nkv), dim3(ATT_THREADS), smem, stream, a);
  return launched();
}

template <int HD_MAX>
static int launch_keys(const AttnArgs& a, int n_entries, cudaStream_t stream) {
  const int stride = a.hd + 8;
  const size_t smem = (size_t)(16 + 2 * KEYS_STAGES * KT) * stride * 2;   // the merge area fits in the tiles
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attention_keys_kernel<HD_MAX>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (16 + 2 * KEYS_STAGES * KT) * (HD_MAX + 8) * 2);
    configured = true;
  }
  launch_pdl(attention_keys_kernel<HD_MAX>, dim3(n_entries, a.nkv, a.nsplit), dim3(ATT_THREADS), smem, stream, a);
  return launched();
}

}  // namespace srlm

using namespace srlm;

static int check_common(const char* who, int nq, int nkv, int hd, int page_size) {
  if (nq <= 0 || nkv <= 0 || nq % nkv || hd <= 0 || hd % 16 || hd > 256 || page_size <= 0)
    return refuse(ST_BAD_SIZE, "%s: nq=%d nkv=%d hd=%d page_size=%d (needs nq %% nkv == 0, hd a multiple of "
                  "16 up to 256)", who, nq, nkv, hd, page_size);
  return ST_OK;
}

// Ragged batch.  work: n_work pairs (entry, row tile of 64 rows); an entry with q tokens has
// ceil(q * (nq/nkv) / 64) row tiles.
extern "C" int srlm_paged_attention_rows(const void* q, const void* k_cache, const void* v_cache, void* out,
                                         const int* block_table, int table_stride, const int* cu_q,
                                         const int* kv_lens, const int* work, int n_work, int nq, int nkv, int hd,
                                         int page_size, float scale, int window, cudaStream_t stream) {
  if (n_work <= 0) return ST_OK;
  int st = check_common("paged_attention_rows", nq, nkv, hd, page_size);
  if (st != ST_OK) return st;
  AttnArgs a{(const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, block_table, table_stride,
             cu_q, kv_lens, work, nq, nkv, hd, page_size, scale * 1.4426950408889634f, window, 0, 1, nullptr,
             nullptr, nullptr};
  if (hd <= 64) return launch_rows<64>(a, n_work, stream);
  if (hd <= 128) return launch_rows<128>(a, n_work, stream);
  return launch_rows<256>(a, n_work, stream);
}

// Every entry has at most 16 rows (q tokens * nq/nkv).  nsplit slices of kv_chunk keys (a multiple of 64)
// must cover the longest entry.  With nsplit > 1: part_o holds n_entries*nkv*nsplit*16*hd floats, part_ml
// n_entries*nkv*nsplit*32 floats, slice_counters n_entries*nkv ints that are zero on entry (and on exit).
extern "C" int srlm_paged_attention_keys(const void* q, const void* k_cache, const void* v_cache, void* out,
                                         const int* block_table, int table_stride, const int* cu_q,
                                         const int* kv_lens, int n_entries, int nq, int nkv, int hd, int page_size,
                                         float scale, int window, int kv_chunk, int nsplit, float* part_o,
                                         float* part_ml, int* slice_counters, cudaStream_t stream) {
  if (n_entries <= 0) return ST_OK;
  int st = check_common("paged_attention_keys", nq, nkv, hd, page_size);
  if (st != ST_OK) return st;
  if (nsplit < 1 || kv_chunk <= 0 || kv_chunk % KT || (nsplit > 1 && (!part_o || !part_ml || !slice_counters)))
    return refuse(ST_BAD_SIZE, "paged_attention_keys: nsplit=%d kv_chunk=%d", nsplit, kv_chunk);
  if (nsplit > 65535 || nkv > 65535) return refuse(ST_BAD_SIZE, "paged_attention_keys: grid too large");
  AttnArgs a{(const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, block_table, table_stride,
             cu_q, kv_lens, nullptr, nq, nkv, hd, page_size, scale * 1.4426950408889634f, window, kv_chunk, nsplit,
             part_o, part_ml, slice_counters};
  if (hd <= 64) return launch_keys<64>(a, n_entries, stream);
  if (hd <= 128) return launch_keys<128>(a, n_entries, stream);
  return launch_keys<256>(a, n_entries, stream);
}
