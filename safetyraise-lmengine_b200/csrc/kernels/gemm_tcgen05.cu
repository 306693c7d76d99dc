// C[M,N] = X[M,K] . W[N,K]^T in bfloat16 with float32 accumulation on the
// 5th-generation tensor cores: tcgen05.mma reading both operands from shared
// memory (filled by TMA, 128-byte swizzle) and accumulating in tensor memory.
//
// The weight is the MMA's 128-row operand and the tokens are its N side
// (16..256 wide), so the same kernel serves a decode step of a few tokens and a
// prefill of thousands: a weight row is read once whatever the batch.  The
// accumulator tile D[n, m] sits in TMEM with one weight row per lane; the
// epilogue reads it with tcgen05.ld and writes C[m, n], 32 consecutive n per
// warp store.
//
// Three forms.  (1) One tile per block, for up to 64 tokens and for a few hundred
// where there are few tiles: K may be split over grid.z; up to 8 splits are a
// thread-block cluster and add their sums through distributed shared memory,
// more write float32 partial tiles to a workspace and the last to finish a tile
// adds them; always in split order, so the sum is the same on every run.
// (2) Persistent, one block per SM walking over tiles of 128 weight rows x 128
// tokens with a double-buffered accumulator; the k-blocks of tiles that do not
// fill a round may be dealt out evenly.  (3) Persistent pairs: two SMs (a cluster
// of two blocks) on tiles of 256 weight rows x 256 tokens with cta_group::2 MMAs,
// for many tokens; when there are tiles for only part of the pairs and K is long,
// all k-blocks are dealt out evenly to all pairs.
//
// Warp roles: warp 0 issues TMA loads, warp 1 allocates TMEM and issues the
// MMAs, warps 2-5 run the epilogue.  Every wait on an mbarrier is bounded: when
// the bound is hit the kernel raises its error flag and runs to its normal end
// (TMEM is freed), it never spins for ever.
//
// What this replaces in the reference: the naive one-thread-per-output CUDA
// kernel native/cuda/safetyraise_cuda.cu:43-63 and the CPU loop
// src/artifact/mod.rs:377-405.
#include <cuda.h>

#include <cstdlib>
#include <map>
#include <atomic>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace srlm {

constexpr int BM = 128;            // weight rows per tile (MMA M)
constexpr int BK = 64;             // bf16 elements per k block: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int BN256_MIN_TILES = 96;   // tiles of 128 weight rows x 256 tokens from which token tiles are 256 wide
constexpr long long WAIT_CYCLES = 4000000000ll;   // ~2 s: far beyond any real wait

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the flag) if the barrier did not flip within `limit` cycles.
__device__ __forceinline__ bool mbar_wait_for(uint64_t* bar, uint32_t parity, int* err_flag, int code,
                                              long long limit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > limit) {
      atomicExch(err_flag, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err_flag, int code) {
  return mbar_wait_for(bar, parity, err_flag, code, WAIT_CYCLES);
}

// One thread waits, with the wait of the pipelines below and a limit of its own, on a barrier that nobody
// arrives at: the wait runs out, the flag is raised, the kernel ends normally.  For the test of the way from a
// wait that ran out to the host; nothing else launches it.
__global__ void wait_probe_kernel(int* err_flag, long long limit, int code) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_wait_for(&bar, 0, err_flag, code, limit);
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// The same load with an L2 eviction hint: weights are read once per step, so their lines should be
// the first to go and leave the L2 to what is read again (activations) or was fetched ahead.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_load_2d_hint(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart (version 1 = Blackwell).
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);          // start address, bits [0,14)
  d |= (uint64_t)0 << 16;                               // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                               // descriptor version
  d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ uint32_t umma_idesc_bf16_f32(int n) {
  return (1u << 4)                       // D is float32
         | (1u << 7) | (1u << 10)        // A and B are bfloat16
         | ((uint32_t)(n >> 3) << 17)    // N
         | ((uint32_t)(BM >> 4) << 24);  // M = 128; both operands K-major (bits 15, 16 zero)
}

template <int COLS>
__device__ __forceinline__ void tmem_load(uint32_t taddr, uint32_t (&v)[COLS]);
template <>
__device__ __forceinline__ void tmem_load<16>(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_load<32>(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
// Optional fusions of the one-tile kernel with the norms around a product (steps of 1 to 128 tokens;
// the same scheme as the weight-streaming kernel's, gemm_skinny.cu):
//  * scale_parts [n_parts][ld_parts]: the tokens X are (residual * norm weight) in bfloat16, not yet divided
//    by their RMS; the product is scaled per token by rsqrt(sum_p scale_parts[p][token] / norm_width + eps).
//  * residual [M][ldr] float32: the product is added to it in place instead of being stored; with next_w [N]
//    also xw_out [M][ldxw] = bf16(residual * next_w) and ss_out [N tiles][ld_ss] (each tile's share of the
//    rows' sums of squares) are written for the norm that follows.
struct GemmFuse {
  const float* scale_parts;
  int n_parts;
  long long ld_parts;
  float inv_width, eps;
  float* residual;
  long long ldr;
  const float* next_w;
  bf16* xw_out;
  long long ldxw;
  float* ss_out;
  long long ld_ss;
};

struct GemmArgs {
  void* C;
  int c_is_f32;
  int M, N, K;
  long long ldc;
  int* err_flag;
  int kb_per_split;        // k blocks each split handles
  float* partial;          // [splits, tiles, BN tokens, 128] float32 (split-K only)
  int* tile_counters;      // one per output tile, zero on entry (split-K only)
  int swiglu8;             // 1: weight rows come in blocks of 16 (8 gate rows, then the 8 up rows of the same
                           //    features); the output is silu(gate) * up, [M, N/2]
  int clustered;           // 1: the splits of a tile are one thread-block cluster (along z) and add their sums
                           //    through distributed shared memory; partial and tile_counters are not used
  int sk_tiles, sk_blocks; // persistent kernel: the k-blocks of the first sk_tiles tiles are dealt out evenly to
                           //    the first sk_blocks blocks, or pairs of blocks (0: every block takes whole tiles only)
  int m_major;             // persistent kernel: tile t covers token tile t / (tiles along N); else t % (tiles along M)
  GemmFuse fuse;           // one-tile kernel only; all zero: none
};

__device__ __forceinline__ void cluster_sync_all() {   // every thread of every block of the cluster
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes at `mine` (an address in this block's shared memory) in block `rank` of the cluster
__device__ __forceinline__ float4 peer_f32x4(const float* mine, uint32_t rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(mine)), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// x * logistic(x) (src/model/math.rs:11-22) in float32 with the fast exponential and reciprocal:
// one branch-free form serves both signs here, since exp2 of a large argument is +inf and its
// reciprocal 0 (x -> -inf gives -0, as the stable form does); relative error ~1e-6.
__device__ __forceinline__ float silu_stable(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.f + e));
  return x * r;
}

// Writes one finished accumulator value x = D[n, m].  Called by all 32 lanes of a warp together
// (`valid` says whether this lane's element exists).
__device__ __forceinline__ void store_result(const GemmArgs& args, int m, int n, float x, bool valid) {
  if (args.swiglu8) {
    const float other = __shfl_xor_sync(0xffffffffu, x, 8);     // the up row of this gate row, and back
    if (valid && (n & 8) == 0) {
      const float h = silu_stable(x) * other;
      const size_t at = (size_t)m * args.ldc + (n >> 4) * 8 + (n & 7);
      if (args.c_is_f32) reinterpret_cast<float*>(args.C)[at] = h;
      else reinterpret_cast<bf16*>(args.C)[at] = __float2bfloat16_rn(h);
    }
    return;
  }
  if (valid) {
    const size_t at = (size_t)m * args.ldc + n;
    if (args.c_is_f32) reinterpret_cast<float*>(args.C)[at] = x;
    else reinterpret_cast<bf16*>(args.C)[at] = __float2bfloat16_rn(x);
  }
}

template <int BN>
constexpr int stage_bytes() { return BM * BK * 2 + BN * BK * 2; }

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  // swizzled tiles must start on 1024-byte boundaries
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* accum_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);
  float* ss_half = reinterpret_cast<float*>(tmem_slot + 4);     // [2][64] halves of the tokens' sums of squares
                                                                //   (token tiles of 128: [128] whole sums)

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN;
  const int total_kb = (args.K + BK - 1) / BK;
  const int kb_begin = blockIdx.z * args.kb_per_split;
  const int num_kb = min(total_kb, kb_begin + args.kb_per_split) - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // the epilogue warps' state (warps 2..5); thread (ew, lane) writes the tokens m_first, m_first + m_step, ...
  constexpr int SROW = BM + 4;                        // floats per token row of the slab (padded)
  static_assert(BN * SROW * 4 <= STAGES * STAGE, "the epilogue's slab lives in the ring");
  float* slab = reinterpret_cast<float*>(smem);      // [BN tokens][SROW]
  const int ew = warp & 3;
  const int rows = min(BN, args.M - m0);
  bool finish = false;
  const bool split = gridDim.z > 1 && !args.clustered;
  // which tokens this thread finishes: every 4th of the tile, or, of a cluster's tile, every 4th of block z's
  const int m_first = args.clustered ? (int)blockIdx.z + (int)gridDim.z * ew : ew;
  const int m_step = args.clustered ? 4 * (int)gridDim.z : 4;

  // What the fused final stage reads from global memory besides the accumulator: the partial sums of squares
  // of the tile's tokens, this thread's rows of the residual stream and the next norm's weights.  The epilogue
  // warps request the first of it before they wait for the accumulator, so that it arrives under the main loop.
  const GemmFuse& f = args.fuse;
  constexpr int GROUP = 4;                 // tokens of a thread whose residual rows are in flight together
  float4 held[GROUP], next_w4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const int col_f = n0 + 4 * lane;
  const bool res_vec = col_f + 4 <= args.N && f.ldr % 4 == 0 && (reinterpret_cast<uintptr_t>(f.residual) & 15) == 0;
  auto residual_rows = [&](float4 (&into)[GROUP], const int m_from) {
#pragma unroll
    for (int j = 0; j < GROUP; ++j) {
      const int m = m_from + j * m_step;
      float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
      if (m < rows) {
        const float* res = f.residual + (size_t)(m0 + m) * f.ldr + col_f;
        if (res_vec) {
          r = *reinterpret_cast<const float4*>(res);
        } else {
          if (col_f < args.N) r.x = res[0];
          if (col_f + 1 < args.N) r.y = res[1];
          if (col_f + 2 < args.N) r.z = res[2];
          if (col_f + 3 < args.N) r.w = res[3];
        }
      }
      into[j] = r;
    }
  };
  const bool fused = BN <= 128 && (f.scale_parts != nullptr || f.residual != nullptr);

  if (warp == 0) {
    if (lane == 0) {
      // Weights are written by no kernel, so the first stages' weight tiles are requested before the
      // wait on the kernel ahead; the token tiles (its output) follow after it.
      const int early = min(num_kb, STAGES);
      const uint64_t stream_once = l2_policy_evict_first();
      for (int i = 0; i < early; ++i) {
        mbar_expect_tx(&full_bar[i], STAGE);
        tma_load_2d_hint(smem + i * STAGE, &map_w, &full_bar[i], (kb_begin + i) * BK, n0, stream_once);
      }
      pdl_wait();
      for (int i = 0; i < early; ++i)
        tma_load_2d(smem + i * STAGE + A_BYTES, &map_x, &full_bar[i], (kb_begin + i) * BK, m0);
      for (int i = early; i < num_kb; ++i) {
        const int s = i % STAGES, j = i / STAGES;
        if (!mbar_wait(&empty_bar[s], (j & 1) ^ 1, args.err_flag, 1)) break;
        mbar_expect_tx(&full_bar[s], STAGE);
        uint8_t* a = smem + s * STAGE;
        const int k = (kb_begin + i) * BK;
        tma_load_2d_hint(a, &map_w, &full_bar[s], k, n0, stream_once);
        tma_load_2d(a + A_BYTES, &map_x, &full_bar[s], k, m0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_f32(BN);
      bool ok = true;
      for (int i = 0; i < num_kb && ok; ++i) {
        const int s = i % STAGES, j = i / STAGES;
        ok = mbar_wait(&full_bar[s], j & 1, args.err_flag, 2);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * STAGE);
        const uint64_t adesc = umma_desc_k_sw128(a_addr), bdesc = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          // 16 elements further along K inside the swizzle row: 32 bytes, 2 units of 16 bytes
          tcgen05_mma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
        }
        tcgen05_commit(&empty_bar[s]);      // frees the stage when these MMAs have read it
      }
      tcgen05_commit(accum_bar);            // arrives when every MMA issued so far is done
    }
    __syncwarp();
  } else {
    // ---------------- epilogue: four warps ----------------
    // The accumulator D[weight row n, token m] leaves TMEM one weight row per thread; it is turned
    // through shared memory (the ring is free once the accumulator is complete) so that everything
    // behind it -- the rows of C, the partial sums of a K split -- moves as whole 16-byte pieces with
    // the lanes of a warp side by side: thread (warp ew, lane) then owns the tokens ew, ew + 4, ...
    // and the four weight rows 4 * lane .. 4 * lane + 3 of each.
    pdl_wait();
    if (fused) {
      if (f.scale_parts) {
        // thread t adds every second part of token t % 64 (neighbouring threads, neighbouring tokens); the two
        // halves meet in shared memory behind the barrier below.  With 128 tokens a thread adds all parts of one.
        const int t = threadIdx.x - 64, m = BN > 64 ? t : (t & 63);
        const int q0 = BN > 64 ? 0 : (t >> 6), dq = BN > 64 ? 1 : 2;
        float p = 0.f;
        if (m < rows)
          for (int q = q0; q < f.n_parts; q += dq) p += __ldg(f.scale_parts + (size_t)q * f.ld_parts + m0 + m);
        ss_half[t] = p;
      }
      if (f.residual && !split) residual_rows(held, m_first);   // (splits in global memory: the owner is not known yet)
      if (f.next_w) {
        if (col_f < args.N) next_w4.x = __ldg(f.next_w + col_f);
        if (col_f + 1 < args.N) next_w4.y = __ldg(f.next_w + col_f + 1);
        if (col_f + 2 < args.N) next_w4.z = __ldg(f.next_w + col_f + 2);
        if (col_f + 3 < args.N) next_w4.w = __ldg(f.next_w + col_f + 3);
      }
    }
    const bool ok = mbar_wait(accum_bar, 0, args.err_flag, 3);
    tcgen05_fence_after();
    const int lane_base = 32 * ew;                      // the TMEM lanes this warp may read
    constexpr int CH = BN < 32 ? 16 : 32;
    if (ok) {
#pragma unroll 1
      for (int c = 0; c < BN; c += CH) {
        uint32_t v[CH];
        tmem_load<CH>(tmem_base + ((uint32_t)lane_base << 16) + c, v);
        tmem_load_wait();
#pragma unroll
        for (int j = 0; j < CH; ++j) slab[(c + j) * SROW + lane_base + lane] = __uint_as_float(v[j]);
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    finish = ok;
    if (split) {
      // this split's sums go out as [split][tile][token][128 weight rows]; the split that arrives last
      // adds all of them in split order (the same order on every run) and writes the result
      const int tile = blockIdx.y * gridDim.x + blockIdx.x;
      const size_t tile_floats = (size_t)BN * BM;
      const size_t split_floats = (size_t)gridDim.x * gridDim.y * tile_floats;
      float* mine = args.partial + blockIdx.z * split_floats + (size_t)tile * tile_floats;
      for (int m = ew; m < rows; m += 4)
        *reinterpret_cast<float4*>(mine + (size_t)m * BM + 4 * lane) =
            *reinterpret_cast<const float4*>(slab + m * SROW + 4 * lane);
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) {
        const int prev = atomicAdd(&args.tile_counters[tile], 1);
        *last_flag = (prev == (int)gridDim.z - 1);
        if (*last_flag) args.tile_counters[tile] = 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      finish = *last_flag != 0;
      if (finish) {
        __threadfence();
        const int nz = (int)gridDim.z;
        const float* first = args.partial + (size_t)tile * tile_floats + 4 * lane;
        // four tokens at a time, so that 4 x nz loads are in flight per thread
        for (int m = ew; m < rows; m += 16) {
          float4 x[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int z = 0; z < nz; ++z) {
            float4 t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int mm = min(m + 4 * u, rows - 1);
              t[u] = __ldcg(reinterpret_cast<const float4*>(first + z * split_floats + (size_t)mm * BM));
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) { x[u].x += t[u].x; x[u].y += t[u].y; x[u].z += t[u].z; x[u].w += t[u].w; }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (m + 4 * u < rows) *reinterpret_cast<float4*>(slab + (m + 4 * u) * SROW + 4 * lane) = x[u];
        }
      }
      // each thread reads back below what it wrote itself: no barrier needed, except for SwiGLU (the
      // up rows sit in another lane's columns)
      if (finish && args.swiglu8) __syncwarp();
    }
  }
  if (args.clustered) {
    // The splits of this tile are the blocks of one cluster, each with its sums in its slab.  Block z
    // adds the token rows z, z + nz, ... of all slabs in split order (the same on every run) into its
    // own slab -- rows that no other block reads -- and writes them out below.  Every thread of every
    // block passes both cluster barriers: no path above leaves the kernel.
    cluster_sync_all();
    if (warp >= 2) {
      const int nz = (int)gridDim.z;
      for (int m = m_first; m < rows; m += 2 * m_step) {
        const int m2 = m + m_step < rows ? m + m_step : m;       // two rows at a time: 2 nz loads in flight
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x;
        for (int p = 0; p < nz; ++p) {
          const float4 t = peer_f32x4(slab + m * SROW + 4 * lane, (uint32_t)p);
          const float4 u = peer_f32x4(slab + m2 * SROW + 4 * lane, (uint32_t)p);
          x.x += t.x; x.y += t.y; x.z += t.z; x.w += t.w;
          y.x += u.x; y.y += u.y; y.z += u.z; y.w += u.w;
        }
        *reinterpret_cast<float4*>(slab + m * SROW + 4 * lane) = x;
        if (m2 != m) *reinterpret_cast<float4*>(slab + m2 * SROW + 4 * lane) = y;
      }
      __syncwarp();                          // SwiGLU reads the up rows from another lane's columns
    }
  }
  if (warp >= 2 && finish && fused) {
    // ---- rows of the slab -> C or the residual stream, with the norms around the product folded in ----
    // 1 / RMS of token m: the halves are added in one order
    auto scale_of = [&](const int m) {
      return f.scale_parts ? rsqrtf((BN > 64 ? ss_half[m] : ss_half[m] + ss_half[64 + m]) * f.inv_width + f.eps) : 1.f;
    };
    const int esize = args.c_is_f32 ? 4 : 2;
    const bool vec_ok = (args.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.C) & 15) == 0);
    auto store4 = [&](uint8_t* dst, const float (&h)[4], const bool whole, const int left) {
      if (vec_ok && whole) {
        if (args.c_is_f32) {
          *reinterpret_cast<float4*>(dst) = make_float4(h[0], h[1], h[2], h[3]);
        } else {
          const __nv_bfloat162 lo = __floats2bfloat162_rn(h[0], h[1]), hi = __floats2bfloat162_rn(h[2], h[3]);
          uint2 pk;
          pk.x = *reinterpret_cast<const uint32_t*>(&lo);
          pk.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(dst) = pk;
        }
      } else {
        for (int e = 0; e < 4 && e < left; ++e) {
          if (args.c_is_f32) reinterpret_cast<float*>(dst)[e] = h[e];
          else reinterpret_cast<bf16*>(dst)[e] = __float2bfloat16_rn(h[e]);
        }
      }
    };
    auto one_token = [&](const int m, const float sc, const float4 r) {
      if (args.swiglu8) {
        if ((lane & 3) < 2) {
          const int col = (n0 >> 1) + (lane >> 2) * 8 + (lane & 1) * 4;
          const int width = args.N >> 1;
          const float4 g = *reinterpret_cast<const float4*>(slab + m * SROW + 4 * lane);
          const float4 u = *reinterpret_cast<const float4*>(slab + m * SROW + 4 * lane + 8);
          const float h[4] = {silu_stable(g.x * sc) * (u.x * sc), silu_stable(g.y * sc) * (u.y * sc),
                              silu_stable(g.z * sc) * (u.z * sc), silu_stable(g.w * sc) * (u.w * sc)};
          store4(reinterpret_cast<uint8_t*>(args.C) + ((size_t)(m0 + m) * args.ldc + col) * esize, h,
                 col + 4 <= width, width - col);
        }
        return;
      }
      const int col = col_f;
      const float4 x4 = *reinterpret_cast<const float4*>(slab + m * SROW + 4 * lane);
      float h[4] = {x4.x * sc, x4.y * sc, x4.z * sc, x4.w * sc};
      if (!f.residual) {
        store4(reinterpret_cast<uint8_t*>(args.C) + ((size_t)(m0 + m) * args.ldc + col) * esize, h,
               col + 4 <= args.N, args.N - col);
        return;
      }
      // residual += product; the next norm's input and this tile's share of the row's sum of squares
      float* res = f.residual + (size_t)(m0 + m) * f.ldr + col;
      h[0] += r.x; h[1] += r.y; h[2] += r.z; h[3] += r.w;
      if (res_vec) {
        *reinterpret_cast<float4*>(res) = make_float4(h[0], h[1], h[2], h[3]);
      } else {
        for (int e = 0; e < 4; ++e) {
          if (col + e < args.N) res[e] = h[e]; else h[e] = 0.f;
        }
      }
      if (f.next_w) {
        const float y[4] = {h[0] * next_w4.x, h[1] * next_w4.y, h[2] * next_w4.z, h[3] * next_w4.w};
        bf16* xw = f.xw_out + (size_t)(m0 + m) * f.ldxw + col;
        if (col + 4 <= args.N && f.ldxw % 4 == 0 && (reinterpret_cast<uintptr_t>(f.xw_out) & 7) == 0) {
          const __nv_bfloat162 lo = __floats2bfloat162_rn(y[0], y[1]), hi = __floats2bfloat162_rn(y[2], y[3]);
          uint2 pk;
          pk.x = *reinterpret_cast<const uint32_t*>(&lo);
          pk.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(xw) = pk;
        } else {
          for (int e = 0; e < 4 && col + e < args.N; ++e) xw[e] = __float2bfloat16_rn(y[e]);
        }
        float sq = h[0] * h[0] + h[1] * h[1] + h[2] * h[2] + h[3] * h[3];      // (columns past N hold 0)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
        if (lane == 0) f.ss_out[(size_t)blockIdx.x * f.ld_ss + m0 + m] = sq;
      }
    };
    if (!f.residual) {
#pragma unroll 1
      for (int m = m_first; m < rows; m += m_step) one_token(m, scale_of(m), next_w4);
    } else {
      // four tokens at a time; the rows of the next four are requested before these are worked on
      if (split) residual_rows(held, m_first);
#pragma unroll 1
      for (int m = m_first; m < rows; m += GROUP * m_step) {
        float4 ahead[GROUP];
        if (m + GROUP * m_step < rows) residual_rows(ahead, m + GROUP * m_step);
#pragma unroll
        for (int j = 0; j < GROUP; ++j)
          if (m + j * m_step < rows) one_token(m + j * m_step, scale_of(m + j * m_step), held[j]);
#pragma unroll
        for (int j = 0; j < GROUP; ++j) held[j] = ahead[j];
      }
    }
  } else if (warp >= 2) {
    if (finish) {
      // rows of the slab -> C
      const int esize = args.c_is_f32 ? 4 : 2;
      const bool vec_ok = (args.ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.C) & 15) == 0);
      if (args.swiglu8) {
        // the 16 rows 16 b .. 16 b + 15 are 8 gate rows and the 8 up rows of the same features:
        // lanes with lane % 4 < 2 hold gate rows, the up rows are two lanes further
        if ((lane & 3) < 2) {
          const int col = (n0 >> 1) + (lane >> 2) * 8 + (lane & 1) * 4;       // first of 4 columns of C
          const int width = args.N >> 1;
          for (int m = m_first; m < rows; m += m_step) {
            const float4 g = *reinterpret_cast<const float4*>(slab + m * SROW + 4 * lane);
            const float4 u = *reinterpret_cast<const float4*>(slab + m * SROW + 4 * lane + 8);
            const float h[4] = {silu_stable(g.x) * u.x, silu_stable(g.y) * u.y, silu_stable(g.z) * u.z,
                                silu_stable(g.w) * u.w};
            uint8_t* dst = reinterpret_cast<uint8_t*>(args.C) + ((size_t)(m0 + m) * args.ldc + col) * esize;
            if (vec_ok && col + 4 <= width) {
              if (args.c_is_f32) {
                *reinterpret_cast<float4*>(dst) = make_float4(h[0], h[1], h[2], h[3]);
              } else {
                const __nv_bfloat162 lo = __floats2bfloat162_rn(h[0], h[1]), hi = __floats2bfloat162_rn(h[2], h[3]);
                uint2 pk;
                pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dst) = pk;
              }
            } else {
              for (int e = 0; e < 4 && col + e < width; ++e) {
                if (args.c_is_f32) reinterpret_cast<float*>(dst)[e] = h[e];
                else reinterpret_cast<bf16*>(dst)[e] = __float2bfloat16_rn(h[e]);
              }
            }
          }
        }
      } else {
        const int col = n0 + 4 * lane;
        for (int m = m_first; m < rows; m += m_step) {
          const float4 x = *reinterpret_cast<const float4*>(slab + m * SROW + 4 * lane);
          const float h[4] = {x.x, x.y, x.z, x.w};
          uint8_t* dst = reinterpret_cast<uint8_t*>(args.C) + ((size_t)(m0 + m) * args.ldc + col) * esize;
          if (vec_ok && col + 4 <= args.N) {
            if (args.c_is_f32) {
              *reinterpret_cast<float4*>(dst) = x;
            } else {
              const __nv_bfloat162 lo = __floats2bfloat162_rn(h[0], h[1]), hi = __floats2bfloat162_rn(h[2], h[3]);
              uint2 pk;
              pk.x = *reinterpret_cast<const uint32_t*>(&lo);
              pk.y = *reinterpret_cast<const uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(dst) = pk;
            }
          } else {
            for (int e = 0; e < 4 && col + e < args.N; ++e) {
              if (args.c_is_f32) reinterpret_cast<float*>(dst)[e] = h[e];
              else reinterpret_cast<bf16*>(dst)[e] = __float2bfloat16_rn(h[e]);
            }
          }
        }
      }
    }
  }
  if (args.clustered) cluster_sync_all();       // nobody leaves while another block still reads its slab
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// The persistent variant for many tokens (prefill): one block per SM walks over output tiles.  The
// accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of a tile runs while
// the MMAs of the next one are issued, and the shared-memory ring never drains between tiles.
// The epilogue transposes each 32-token slab through shared memory and writes whole rows of C
// (256 contiguous bytes per token and tile) instead of one element per lane.
//
// Tiles seldom come in multiples of the SM count: 384 tiles leave 60 of 148 SMs idle in the third
// round.  So the k-blocks of the tiles that do not fill a round (args.sk_tiles of them, the first;
// see dealt_tiles) are dealt out evenly: block b takes the units [u_lo, u_hi) of the sequence (tile 0, k-block 0),
// (tile 0, k-block 1), ...; then every block takes whole tiles.  A block that holds only part of a
// tile's k-blocks writes its sums to its slot of the workspace (float32) and counts itself in;
// whoever counts in last adds the parts in the order of the blocks -- the same order on every run --
// and writes the tile.  Nobody waits for anybody.
// ---------------------------------------------------------------------------
struct PieceWalk {         // the pieces (tile, k-blocks [kb_lo, kb_hi)) of one block, in the order it runs them
  int num_kb, total_tiles, sk_tiles, stride;
  int u, u_hi, dp_t;
  __device__ PieceWalk(const GemmArgs& a, int num_kb_, int total_tiles_, int block, int blocks)
      : num_kb(num_kb_), total_tiles(total_tiles_), sk_tiles(a.sk_tiles), stride(blocks) {
    u = u_hi = 0;
    if (block < a.sk_blocks) {
      const int units = a.sk_tiles * num_kb, base = units / a.sk_blocks, rem = units % a.sk_blocks;
      u = block * base + min(block, rem);
      u_hi = u + base + (block < rem ? 1 : 0);
    }
    dp_t = a.sk_tiles + block;
  }
  __device__ bool next(int& t, int& kb_lo, int& kb_hi) {
    if (u < u_hi) {
      t = u / num_kb;
      kb_lo = u - t * num_kb;
      const int end = min(u_hi, (t + 1) * num_kb);
      kb_hi = end - t * num_kb;
      u = end;
      return true;
    }
    if (dp_t < total_tiles) {
      t = dp_t;
      kb_lo = 0;
      kb_hi = num_kb;
      dp_t += stride;
      return true;
    }
    return false;
  }
};
// first unit of block b's share of the dealt-out units, and the block that holds unit u
__device__ __forceinline__ int sk_first_unit(int b, int base, int rem) { return b * base + min(b, rem); }
__device__ __forceinline__ int sk_block_of(int u, int base, int rem) {
  return u < rem * (base + 1) ? u / (base + 1) : rem + (u - rem * (base + 1)) / base;
}

// ---- two blocks on one tile (cta_group::2): the even block of the pair issues the MMAs ----------------
// The address of the same shared-memory object in the even block of the pair.
__device__ __forceinline__ uint32_t in_even_block(const void* p) { return smem_u32(p) & 0xFEFFFFFFu; }
// A tiled copy into this block's shared memory that counts its bytes on the even block's barrier.
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(in_even_block(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                      uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this address in both blocks of the pair when the MMAs issued so far are done.
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
// An epilogue warp has read its share of an accumulator: tells the block that issues the MMAs.
template <bool PAIR>
__device__ __forceinline__ void acc_drained(uint64_t* bar) {
  if (PAIR) asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(in_even_block(bar)) : "memory");
  else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

template <int BN, int STAGES, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                               const GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  // PAIR: two blocks (a cluster of 2, on two SMs) share a tile of 256 weight rows x BN tokens: each
  // holds its 128 weight rows and half of the tokens in shared memory, the MMAs (cta_group::2, issued by
  // the even block) read both halves and leave each block's 128 rows of the result in its own TMEM.
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;                 // token rows this block fetches per k-block
  constexpr int TILE_N = PAIR ? 2 * BM : BM;                 // weight rows of a tile
  constexpr int A_BYTES = BM * BK * 2, B_BYTES = B_ROWS * BK * 2, STAGE = A_BYTES + B_BYTES;
  constexpr int TMEM_COLS = 2 * BN;
  constexpr int SLAB = 32;                                   // tokens per epilogue slab
  constexpr int SLAB_ROW = BM * 4 + 16;                      // bytes per token row of the slab (padded)
  uint8_t* slab = smem + STAGES * STAGE;                     // [2][SLAB][SLAB_ROW]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(slab + 2 * SLAB * SLAB_ROW);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;                   // [2]
  uint64_t* acc_empty = acc_full + 2;                        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  int* last_flag = reinterpret_cast<int*>(tmem_slot + 1);

  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank = 0;                                         // of this block in its pair
  if (PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int walker = PAIR ? blockIdx.x / 2 : blockIdx.x, walkers = PAIR ? gridDim.x / 2 : gridDim.x;
  const int tiles_m = (args.M + BN - 1) / BN, tiles_n = (args.N + TILE_N - 1) / TILE_N;
  const int total_tiles = tiles_m * tiles_n;
  const int num_kb = (args.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], PAIR ? 8 : 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 1) {
    if (PAIR) {      // the same warp of both blocks, the same address in both
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                   "r"(TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();        // both blocks' barriers exist before either signals the other's
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();
      int it = 0;
      bool ok = true;
      PieceWalk walk(args, num_kb, total_tiles, walker, walkers);
      int t, kb_lo, kb_hi;
      while (ok && walk.next(t, kb_lo, kb_hi)) {
        const int m0 = (args.m_major ? t / tiles_n : t % tiles_m) * BN + (int)rank * (PAIR ? B_ROWS : 0);
        const int n0 = (args.m_major ? t % tiles_n : t / tiles_m) * TILE_N + (int)rank * BM;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % STAGES, j = it / STAGES;
          ok = mbar_wait(&empty_bar[s], (j & 1) ^ 1, args.err_flag, 21);
          if (!ok) break;
          uint8_t* a = smem + s * STAGE;
          if (PAIR) {
            // both blocks' copies count on the even block's barrier, which expects the bytes of both
            if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE);
            tma_load_2d_pair(a, &map_w, &full_bar[s], kb * BK, n0);
            tma_load_2d_pair(a + A_BYTES, &map_x, &full_bar[s], kb * BK, m0);
          } else {
            mbar_expect_tx(&full_bar[s], STAGE);
            tma_load_2d(a, &map_w, &full_bar[s], kb * BK, n0);
            tma_load_2d(a + A_BYTES, &map_x, &full_bar[s], kb * BK, m0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // PAIR: M = 256 (field at bit 24, in units of 16 rows)
      const uint32_t idesc = PAIR ? ((umma_idesc_bf16_f32(BN) & ~(0x1Fu << 24)) | (16u << 24)) : umma_idesc_bf16_f32(BN);
      int it = 0, local = 0;
      bool ok = true;
      PieceWalk walk(args, num_kb, total_tiles, walker, walkers);
      int t, kb_lo, kb_hi;
      for (; ok && walk.next(t, kb_lo, kb_hi); ++local) {
        const int b = local & 1;
        ok = mbar_wait(&acc_empty[b], ((local >> 1) & 1) ^ 1, args.err_flag, 22);   // epilogue has drained it
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + b * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++it) {
          const int s = it % STAGES, j = it / STAGES;
          ok = mbar_wait(&full_bar[s], j & 1, args.err_flag, 23);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE);
          const uint64_t adesc = umma_desc_k_sw128(a_addr), bdesc = umma_desc_k_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            if (PAIR) tcgen05_mma_bf16_pair(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb != kb_lo || k != 0) ? 1u : 0u);
            else tcgen05_mma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb != kb_lo || k != 0) ? 1u : 0u);
          if (PAIR) tcgen05_commit_pair(&empty_bar[s]); else tcgen05_commit(&empty_bar[s]);
        }
        if (PAIR) tcgen05_commit_pair(&acc_full[b]); else tcgen05_commit(&acc_full[b]);
      }
    }
    __syncwarp();
  } else {
    pdl_wait();
    const int ew = warp & 3;                               // TMEM lanes 32*ew .. 32*ew+31 belong to this warp
    const int lane_base = 32 * ew;
    const int tid_e = ew * 32 + lane;                      // 0..127 among the epilogue threads
    const int out_cols = args.swiglu8 ? BM / 2 : BM;       // columns of C a tile produces
    const int esize = args.c_is_f32 ? 4 : 2;
    const bool vec_ok = (args.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(args.C) & 15) == 0);
    int local = 0, slab_turn = 0;
    bool ok = true;
    PieceWalk walk(args, num_kb, total_tiles, walker, walkers);
    int t, kb_lo, kb_hi;
    const int sk_units = args.sk_tiles * num_kb;
    const int sk_base = args.sk_blocks ? sk_units / args.sk_blocks : 0;
    const int sk_rem = args.sk_blocks ? sk_units % args.sk_blocks : 0;
    const int my_first_unit = sk_first_unit(walker, sk_base, sk_rem);
    // a pair shares its units; each of its blocks keeps its own 128 weight rows of every piece, in slots
    // and under a counter of its own
    const int slot_block = (int)blockIdx.x;
    constexpr size_t SLOT = (size_t)BN * BM;                // floats of a slot: [BN tokens][128 weight rows]
    for (; ok && walk.next(t, kb_lo, kb_hi); ++local) {
      const int b = local & 1;
      const int m0 = (args.m_major ? t / tiles_n : t % tiles_m) * BN;
      const int n0 = (args.m_major ? t % tiles_n : t / tiles_m) * TILE_N + (int)rank * BM;
      ok = mbar_wait(&acc_full[b], (local >> 1) & 1, args.err_flag, 24);
      if (!ok) break;
      tcgen05_fence_after();
      const int c0 = args.swiglu8 ? n0 / 2 : n0;           // first column of C of this tile
      const bool whole = kb_lo == 0 && kb_hi == num_kb;
      int part_first = 0, part_last = -1;                  // the blocks that share this tile
      if (!whole) {
        // this block's sums of a part of the tile's k-blocks -> its slot (0: the piece its share begins
        // with, 1: the piece it ends with)
        float* mine = args.partial + (2 * (size_t)slot_block + (t * num_kb + kb_lo == my_first_unit ? 0 : 1)) * SLOT;
#pragma unroll 1
        for (int c = 0; c < BN; c += SLAB) {
          uint32_t v[SLAB];
          tmem_load<SLAB>(tmem_base + ((uint32_t)lane_base << 16) + b * BN + c, v);
          tmem_load_wait();
          if (c + SLAB >= BN) {
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) acc_drained<PAIR>(&acc_empty[b]);
          }
          if (m0 + c >= args.M) continue;
#pragma unroll
          for (int j = 0; j < SLAB; ++j) mine[(size_t)(c + j) * BM + lane_base + lane] = __uint_as_float(v[j]);
        }
        part_first = sk_block_of(t * num_kb, sk_base, sk_rem);
        part_last = sk_block_of((t + 1) * num_kb - 1, sk_base, sk_rem);
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid_e == 0) {
          int* counter = args.tile_counters + (PAIR ? 2 * t + (int)rank : t);
          const int prev = atomicAdd(counter, 1);
          const int last = prev == part_last - part_first;
          if (last) *counter = 0;                           // clean for the next product
          *last_flag = last;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!*last_flag) continue;                          // somebody else finishes this tile
        __threadfence();
        // The parts of the blocks part_first .. part_last, added in that order, straight from the workspace
        // to C.  A thread takes an item of 8 sums of one token: 8 consecutive weight rows, or through SwiGLU 4
        // gate rows and the 4 up rows of the same features; four items at a time, with the loads of up to
        // three parts of each in flight together.
        const int np = part_last - part_first + 1;
        constexpr int IPT = BM / 8;                         // items per token
        const int items = min(BN, args.M - m0) * IPT;
        const int n_limit = (args.swiglu8 ? args.N / 2 : args.N) - c0;
        auto slot_of = [&](int pb) {
          const int which = sk_first_unit(pb, sk_base, sk_rem) >= t * num_kb ? 0 : 1;
          const size_t blk = PAIR ? 2 * (size_t)pb + rank : (size_t)pb;
          return args.partial + (2 * blk + which) * SLOT;
        };
        constexpr int U = 4, P = 3;
#pragma unroll 1
        for (int base = tid_e; base < items; base += 128 * U) {
          float acc[U][8];
          size_t off[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int idx = min(base + u * 128, items - 1), v = idx % IPT;
            off[u] = (size_t)(idx / IPT) * BM + (args.swiglu8 ? (v >> 1) * 16 + (v & 1) * 4 : v * 8);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
          }
          const int second = args.swiglu8 ? 8 : 4;          // floats from an item's first four sums to its other four
#pragma unroll 1
          for (int p0 = 0; p0 < np; p0 += P) {
            float4 got[P][U][2];
#pragma unroll
            for (int q = 0; q < P; ++q) {
              if (p0 + q < np) {
                const float* src = slot_of(part_first + p0 + q);
#pragma unroll
                for (int u = 0; u < U; ++u) {
                  got[q][u][0] = __ldcg(reinterpret_cast<const float4*>(src + off[u]));
                  got[q][u][1] = __ldcg(reinterpret_cast<const float4*>(src + off[u] + second));
                }
              }
            }
#pragma unroll
            for (int q = 0; q < P; ++q) {
              if (p0 + q < np) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                  acc[u][0] += got[q][u][0].x; acc[u][1] += got[q][u][0].y;
                  acc[u][2] += got[q][u][0].z; acc[u][3] += got[q][u][0].w;
                  acc[u][4] += got[q][u][1].x; acc[u][5] += got[q][u][1].y;
                  acc[u][6] += got[q][u][1].z; acc[u][7] += got[q][u][1].w;
                }
              }
            }
          }
          auto two = [](float lo, float hi) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
            return *reinterpret_cast<const uint32_t*>(&v);
          };
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int idx = base + u * 128;
            if (idx < items) {
              const int j = idx / IPT, v = idx % IPT;
              if (args.swiglu8) {
                const int col = (v >> 1) * 8 + (v & 1) * 4;          // first of 4 columns of C within the tile
                const float h[4] = {silu_stable(acc[u][0]) * acc[u][4], silu_stable(acc[u][1]) * acc[u][5],
                                    silu_stable(acc[u][2]) * acc[u][6], silu_stable(acc[u][3]) * acc[u][7]};
                uint8_t* dst = reinterpret_cast<uint8_t*>(args.C) + ((size_t)(m0 + j) * args.ldc + c0 + col) * esize;
                if (vec_ok && col + 4 <= n_limit) {
                  if (args.c_is_f32) *reinterpret_cast<float4*>(dst) = make_float4(h[0], h[1], h[2], h[3]);
                  else *reinterpret_cast<uint2*>(dst) = make_uint2(two(h[0], h[1]), two(h[2], h[3]));
                } else {
                  for (int e = 0; e < 4 && col + e < n_limit; ++e) {
                    if (args.c_is_f32) reinterpret_cast<float*>(dst)[e] = h[e];
                    else reinterpret_cast<bf16*>(dst)[e] = __float2bfloat16_rn(h[e]);
                  }
                }
              } else {
                const int col = v * 8;                               // first of 8 columns of C within the tile
                uint8_t* dst = reinterpret_cast<uint8_t*>(args.C) + ((size_t)(m0 + j) * args.ldc + c0 + col) * esize;
                if (vec_ok && col + 8 <= n_limit) {
                  if (args.c_is_f32) {
                    reinterpret_cast<float4*>(dst)[0] = make_float4(acc[u][0], acc[u][1], acc[u][2], acc[u][3]);
                    reinterpret_cast<float4*>(dst)[1] = make_float4(acc[u][4], acc[u][5], acc[u][6], acc[u][7]);
                  } else {
                    *reinterpret_cast<uint4*>(dst) = make_uint4(two(acc[u][0], acc[u][1]), two(acc[u][2], acc[u][3]),
                                                                two(acc[u][4], acc[u][5]), two(acc[u][6], acc[u][7]));
                  }
                } else {
                  for (int e = 0; e < 8 && col + e < n_limit; ++e) {
                    if (args.c_is_f32) reinterpret_cast<float*>(dst)[e] = acc[u][e];
                    else reinterpret_cast<bf16*>(dst)[e] = __float2bfloat16_rn(acc[u][e]);
                  }
                }
              }
            }
          }
        }
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < BN; c += SLAB, slab_turn ^= 1) {
        uint32_t v[SLAB];
        tmem_load<SLAB>(tmem_base + ((uint32_t)lane_base << 16) + b * BN + c, v);
        tmem_load_wait();
        if (c + SLAB >= BN) {                               // everything of this tile has left TMEM
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) acc_drained<PAIR>(&acc_empty[b]);
        }
        if (m0 + c >= args.M) continue;                     // slab beyond the last token (same for all warps)
        uint8_t* sl = slab + slab_turn * SLAB * SLAB_ROW;
        // D[n, m] -> slab[m][column of C]
        if (args.swiglu8) {
          // lanes l and l^8 hold the gate and the up row of one feature; they share the work: the
          // gate lane finishes the even token of a pair, the up lane the odd one
          const bool gate_lane = (lane & 8) == 0;
          const int col = (lane_base >> 1) + (lane >> 4) * 8 + (lane & 7);
#pragma unroll
          for (int j = 0; j < SLAB; j += 2) {
            const float mine0 = __uint_as_float(v[j]), mine1 = __uint_as_float(v[j + 1]);
            const float got = __shfl_xor_sync(0xffffffffu, gate_lane ? mine1 : mine0, 8);
            const float hval = gate_lane ? silu_stable(mine0) * got : silu_stable(got) * mine1;
            const int row = gate_lane ? j : j + 1;
            if (args.c_is_f32) *reinterpret_cast<float*>(sl + row * SLAB_ROW + col * 4) = hval;
            else *reinterpret_cast<bf16*>(sl + row * SLAB_ROW + col * 2) = __float2bfloat16_rn(hval);
          }
        } else {
#pragma unroll
          for (int j = 0; j < SLAB; ++j) {
            const float x = __uint_as_float(v[j]);
            const int col = lane_base + lane;
            if (args.c_is_f32) *reinterpret_cast<float*>(sl + j * SLAB_ROW + col * 4) = x;
            else *reinterpret_cast<bf16*>(sl + j * SLAB_ROW + col * 2) = __float2bfloat16_rn(x);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // rows of the slab -> C, 16 bytes per thread
        const int row_bytes = out_cols * esize;
        const int vec_per_row = row_bytes / 16;
        const int n_limit = (args.swiglu8 ? args.N / 2 : args.N) - c0;     // valid columns in this tile
        for (int idx = tid_e; idx < SLAB * vec_per_row; idx += 128) {
          const int j = idx / vec_per_row, vcol = idx % vec_per_row;
          const int m = m0 + c + j;
          if (m >= args.M) continue;
          const int col = vcol * (16 / esize);              // first column of this 16-byte piece
          uint8_t* dst = reinterpret_cast<uint8_t*>(args.C) + ((size_t)m * args.ldc + c0 + col) * esize;
          const uint8_t* src = sl + j * SLAB_ROW + vcol * 16;
          if (vec_ok && col + 16 / esize <= n_limit) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
          } else {
            for (int e = 0; e < 16 / esize && col + e < n_limit; ++e) {
              if (args.c_is_f32) reinterpret_cast<float*>(dst)[e] = reinterpret_cast<const float*>(src)[e];
              else reinterpret_cast<bf16*>(dst)[e] = reinterpret_cast<const bf16*>(src)[e];
            }
          }
        }
        // the other slab buffer is used next; this one is rewritten two slabs later, after another barrier
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();        // neither block leaves while the other may still signal its barriers
  if (warp == 1) {
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                   : "memory");
  }
}

// ---------------------------------------------------------------------------
// host side: tensor maps and launch
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// [rows, K] bfloat16 row-major with leading dimension ld; box = [box_rows, 64]
static bool make_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows,
                     bool weight) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  weight ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

struct MapKey {
  const void* ptr; long long rows, K, ld; int box_rows;
  bool operator<(const MapKey& o) const {
    return std::tie(ptr, rows, K, ld, box_rows) < std::tie(o.ptr, o.rows, o.K, o.ld, o.box_rows);
  }
};
static std::map<MapKey, CUtensorMap> g_maps;
static std::mutex g_maps_mutex;
static const size_t MAP_CACHE_LIMIT = 4096;

// Copies the map into *out under the lock: the cache may be emptied by the next lookup (of this thread
// or another), so no pointer into it ever leaves this function.
static bool cached_map(CUtensorMap* out, const void* ptr, long long rows, long long K, long long ld, int box_rows,
                       bool weight) {
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  MapKey key{ptr, rows, K, ld, box_rows};
  auto it = g_maps.find(key);
  if (it == g_maps.end()) {
    CUtensorMap m;
    if (!make_map(&m, ptr, rows, K, ld, box_rows, weight)) return false;
    if (g_maps.size() >= MAP_CACHE_LIMIT) g_maps.clear();
    it = g_maps.emplace(key, m).first;
  }
  *out = it->second;
  return true;
}

// For tests: the number of cached maps and the cache's limit.
extern "C" int srlm_gemm_tcgen05_map_cache(int* limit) {
  std::lock_guard<std::mutex> lock(g_maps_mutex);
  if (limit) *limit = (int)MAP_CACHE_LIMIT;
  return (int)g_maps.size();
}

template <int BN, int STAGES>
static int launch(const CUtensorMap* mw, const CUtensorMap* mx, const GemmArgs& a, int splits, cudaStream_t stream) {
  constexpr int SMEM = STAGES * stage_bytes<BN>() + (2 * STAGES + 1) * 8 + 16 + 512 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return refuse((int)e, "gemm_tcgen05: cannot get %d bytes of shared memory", SMEM);
    configured = true;
  }
  dim3 grid((a.N + BM - 1) / BM, (a.M + BN - 1) / BN, splits);
  if (!a.clustered) {
    launch_pdl(gemm_tcgen05_kernel<BN, STAGES>, grid, dim3(GEMM_THREADS), SMEM, stream, *mw, *mx, a);
    return launched();
  }
  // the splits of a tile as one thread-block cluster along z
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 1;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = splits;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BN, STAGES>, *mw, *mx, a);
  return launched();
}

// How many tiles (the first ones) the persistent kernel deals out by k-blocks: the ones left over after
// the whole rounds, when they would leave 40 % of the SMs or more without a tile.  Measured on B200:
// dealing out more (a whole round's worth with them, or all tiles when there are fewer than SMs) is
// slower than whole tiles -- blocks that walk the same weight tile no longer do so in step, and what
// one of them fetched has left the L2 when the next one asks; and a share under 8 k-blocks is not
// worth its trip through the workspace.
static int dealt_tiles(int tiles, int num_kb, int walkers) {      // walkers: blocks, or pairs of blocks
  const int left = tiles % walkers;
  if (tiles <= walkers || left == 0 || left * 10 > walkers * 6) return 0;
  const long long units = (long long)left * num_kb;
  if (units / 8 < walkers || left * 8 > 65536) return 0;
  return left;
}

template <int BN, int STAGES>
static int launch_persistent(const CUtensorMap* mw, const CUtensorMap* mx, const GemmArgs& a, long long ws_bytes,
                             cudaStream_t stream) {
  constexpr int SMEM = STAGES * stage_bytes<BN>() + 2 * 32 * (BM * 4 + 16) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static bool configured = false;
  static int sm_count = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<BN, STAGES, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return refuse((int)e, "gemm_tcgen05: cannot get %d bytes of shared memory", SMEM);
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int tiles = ((a.N + BM - 1) / BM) * ((a.M + BN - 1) / BN);
  const int num_kb = (a.K + BK - 1) / BK;
  GemmArgs b = a;
  b.sk_tiles = b.sk_blocks = 0;
  int grid = tiles < sm_count ? tiles : sm_count;
  const long long slots_bytes = 2ll * sm_count * BN * BM * 4;
  if (b.partial && b.tile_counters && ws_bytes >= 65536 + slots_bytes) {
    const int sk = dealt_tiles(tiles, num_kb, sm_count);
    if (sk > 0) {
      b.sk_tiles = sk;
      b.sk_blocks = sm_count;
    }
  }
  launch_pdl(gemm_tcgen05_persistent_kernel<BN, STAGES, false>, dim3(grid), dim3(GEMM_THREADS), SMEM, stream, *mw, *mx, b);
  return launched();
}

// How many tiles the pair form deals out by k-blocks: all of them, when they would occupy at most 70 % of the
// pairs in their one round and every pair still gets 96 k-blocks or more.  The tiles are then numbered with
// the weight tile running fastest (m_major), so that the pairs that work on the same weight rows for different
// token tiles are half the GPU apart and walk their k-blocks in step: what one fetched is in the L2 for the other.
// Measured at 512 tokens (40 tiles on 74 pairs): down projection of 5120 x 17408 92.7 -> 82.8 us, of 5120 x
// 25600 132.4 -> 114.2 us; with shorter shares the trip of the parts through the workspace, all at the end,
// costs more than the idle pairs (5120 x 5120: 33.7 -> 42.3 us; 6144 x 4096: 28.5 -> 41.4 us).
static int dealt_pair_tiles(int tiles, int num_kb, int pairs) {
  if (pairs <= 1 || tiles >= pairs || tiles * 10 > pairs * 7) return 0;
  if ((long long)tiles * num_kb / pairs < 96 || 2 * tiles > 16384) return 0;
  return tiles;
}

// The pair form of the persistent kernel (see PAIR there): tiles of 256 weight rows x BN tokens, a cluster of
// two blocks per tile; whole tiles, or all k-blocks dealt out (dealt_pair_tiles).  mx: the token map with boxes
// of BN / 2 rows.
template <int BN, int STAGES>
static int launch_pair(const CUtensorMap* mw, const CUtensorMap* mx, const GemmArgs& a, long long ws_bytes,
                       cudaStream_t stream) {
  constexpr int SMEM = STAGES * (BM * BK * 2 + (BN / 2) * BK * 2) + 2 * 32 * (BM * 4 + 16) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static_assert(SMEM <= 232448, "shared memory of a block");
  static bool configured = false;
  static int sm_count = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<BN, STAGES, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return refuse((int)e, "gemm_tcgen05: cannot get %d bytes of shared memory", SMEM);
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  const int tiles = ((a.N + 2 * BM - 1) / (2 * BM)) * ((a.M + BN - 1) / BN);
  int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  GemmArgs b = a;
  b.sk_tiles = b.sk_blocks = b.m_major = 0;
  // More tiles than pairs: whole tiles only (dealing the left-over tiles' k-blocks out to the pairs measured
  // slower more often than faster: 1,024 tokens: QKV 68.5 against 56.1 us; 4,096 tokens: down 265 against
  // 277 us).  Fewer: see dealt_pair_tiles.
  static const bool whole_only = getenv("SRLM_GEMM_STREAMK") && !atoi(getenv("SRLM_GEMM_STREAMK"));
  const long long slots_bytes = 2ll * sm_count * BN * BM * 4;
  if (!whole_only && b.partial && b.tile_counters && ws_bytes >= 65536 + slots_bytes) {
    const int sk = dealt_pair_tiles(tiles, (a.K + BK - 1) / BK, sm_count / 2);
    if (sk > 0) {
      pairs = sm_count / 2;
      b.sk_tiles = sk;
      b.sk_blocks = pairs;
      b.m_major = 1;
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaLaunchKernelEx(&cfg, gemm_tcgen05_persistent_kernel<BN, STAGES, true>, *mw, *mx, b);
  return launched();
}

}  // namespace srlm

using namespace srlm;

// workspace (only when splits > 1): one int per output tile, zero on entry and left zero on exit,
// at the start; float32 partials [splits, tiles, token tile, 128] from byte 65536 on, any contents.  err_flag: one int the kernel sets to a nonzero code if a wait ran out.
// The SM count of the current device (0 if it cannot be had).
static int device_sms() {
  static std::atomic<int> known[64];            // per device; 0: not asked yet
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64 && (sms = known[dev].load(std::memory_order_relaxed)) > 0) return sms;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64) known[dev].store(sms, std::memory_order_relaxed);
  return sms;
}

// The width of a product's token tiles.  Up to 128 tokens: the smallest tile that holds them.  Beyond:
// tiles of 256 tokens (pairs of SMs on 256 weight rows x 256 tokens) from BN256_MIN_TILES tiles of 128 rows
// x 256 tokens on -- a pair moves half the operand bytes per SM and product of two SMs on 128 x 128 each,
// but a narrow output has too few such tiles for every pair.  With fewer tiles, whichever form needs fewer
// rounds of the GPU, a round of pairs (four 128 x 128 tiles' work each) counted as 4/3 rounds of single
// SMs.  Measured at 512 tokens: 5120 x 5120 (160 tiles of 128 x 128: two rounds; 40 pairs' tiles: one)
// 49.4 -> 33.0 us, 5120 x 8192 57.2 -> 48.1 us; 4096 x 4096 (128 tiles: one round) 22.9 us against 26.4.
static int token_tile(int M, int N, int sms) {
  if (M <= 128) return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  const long long rows128 = (N + BM - 1) / BM;
  if (rows128 * ((M + 255) / 256) >= BN256_MIN_TILES) return 256;
  if (sms <= 1) return 128;
  const long long tiles128 = rows128 * ((M + 127) / 128), tiles256 = (long long)((N + 255) / 256) * ((M + 255) / 256);
  const long long rounds128 = (tiles128 + sms - 1) / sms, rounds256 = (tiles256 + sms / 2 - 1) / (sms / 2);
  return 4 * rounds256 < 3 * rounds128 ? 256 : 128;
}

static int gemm_entry(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K, long long ldx,
                      long long ldw, long long ldc, int splits, void* workspace, long long workspace_bytes,
                      int* err_flag, int swiglu8, const GemmFuse* fuse, cudaStream_t stream) {
  if (M <= 0) return ST_OK;
  if (N <= 0 || K <= 0 || ldx < K || ldw < K || ldc < (swiglu8 ? N / 2 : N) || (swiglu8 && N % 16))
    return refuse(ST_BAD_SIZE, "gemm_tcgen05: M=%d N=%d K=%d ldx=%lld ldw=%lld ldc=%lld swiglu8=%d", M, N, K, ldx,
                  ldw, ldc, swiglu8);
  if (K % 8 || ldx % 8 || ldw % 8)
    return refuse(ST_BAD_SIZE, "gemm_tcgen05: K=%d and the leading dimensions must be multiples of 8 "
                  "(TMA rows start on 16-byte boundaries)", K);
  if (((uintptr_t)X | (uintptr_t)W) & 15)
    return refuse(ST_BAD_ALIGN, "gemm_tcgen05: operands must be 16-byte aligned");
  if (c_dtype != DT_F32 && c_dtype != DT_BF16) return refuse(ST_BAD_DTYPE, "gemm_tcgen05: output dtype %d", c_dtype);
  const int total_kb = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > total_kb) splits = total_kb;
  int kb_per_split = (total_kb + splits - 1) / splits;
  splits = (total_kb + kb_per_split - 1) / kb_per_split;       // no empty split
  const int bn = token_tile(M, N, device_sms());
  GemmArgs a{C, c_dtype == DT_F32, M, N, K, ldc, err_flag, kb_per_split, nullptr, nullptr, swiglu8 ? 1 : 0, 0};
  if (fuse) {
    if (bn > 128)
      return refuse(ST_BAD_SIZE, "gemm_tcgen05: the norm fusions take at most 128 tokens, got %d", M);
    a.fuse = *fuse;
  }
  // up to 8 splits (the portable cluster size) add their sums inside a thread-block cluster and need no
  // workspace (SRLM_GEMM_CLUSTER=0: through the workspace, as more than 8 splits do)
  static const bool cluster_off = getenv("SRLM_GEMM_CLUSTER") && !atoi(getenv("SRLM_GEMM_CLUSTER"));
  a.clustered = splits > 1 && splits <= 8 && !cluster_off;
  if (splits > 1 && !a.clustered) {
    const long long tiles = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
    const long long need = 65536 + (long long)splits * tiles * BM * bn * 4;
    if (!workspace || workspace_bytes < need || tiles * 4 > 65536)
      return refuse(ST_BAD_SIZE, "gemm_tcgen05: split-K with %d splits needs %lld bytes of workspace, got %lld",
                    splits, need, workspace_bytes);
    a.tile_counters = reinterpret_cast<int*>(workspace);
    a.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 65536);
  }
  CUtensorMap mw_copy, mx_copy, mx128_copy;
  const CUtensorMap *mw = &mw_copy, *mx = &mx_copy;
  if (!cached_map(&mw_copy, W, N, K, ldw, BM, true) || !cached_map(&mx_copy, X, M, K, ldx, bn, false))
    return refuse(ST_BAD_SIZE, "gemm_tcgen05: cuTensorMapEncodeTiled refused the operands");
  if (splits == 1 && bn >= 128 && !fuse) {   // many tokens: the persistent kernel (SRLM_GEMM_PERSISTENT=0: one tile per
                                             // block); the norm fusions live in the one-tile kernel
    static const bool off = getenv("SRLM_GEMM_PERSISTENT") && !atoi(getenv("SRLM_GEMM_PERSISTENT"));
    // SRLM_GEMM_STREAMK=0: whole tiles only
    static const bool whole_only = getenv("SRLM_GEMM_STREAMK") && !atoi(getenv("SRLM_GEMM_STREAMK"));
    if (workspace && !whole_only) {
      a.tile_counters = reinterpret_cast<int*>(workspace);
      a.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + 65536);
    }
    // token tiles of 256: two SMs per tile of 256 x 256 (SRLM_GEMM_PAIR=0: one SM per tile of 128 x 256)
    static const bool pair_off = getenv("SRLM_GEMM_PAIR") && !atoi(getenv("SRLM_GEMM_PAIR"));
    if (!off && bn == 256 && !pair_off) {
      const CUtensorMap* mx128 = &mx128_copy;
      if (!cached_map(&mx128_copy, X, M, K, ldx, 128, false)) return refuse(ST_BAD_SIZE, "gemm_tcgen05: cuTensorMapEncodeTiled refused the operands");
      return launch_pair<256, 6>(mw, mx128, a, workspace_bytes, stream);
    }

    if (!off)
      return bn == 128 ? launch_persistent<128, 5>(mw, mx, a, workspace_bytes, stream)
                       : launch_persistent<256, 4>(mw, mx, a, workspace_bytes, stream);
    a.tile_counters = nullptr;
    a.partial = nullptr;
  }
  const long long blocks = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn) * splits;
  switch (bn) {
    // stages chosen so that two or three blocks share an SM: their prologues and epilogues overlap one
    // another's streaming, and tile counts that are no multiple of 148 still keep every SM busy; at
    // 17..64 tokens a block's stream is bound by the latency of its ring, hence the deeper rings there
    // (more blocks than run at once two to an SM, 296 on 148 SMs: a ring of three stages lets a third block in;
    // gate/up of 8B sizes in 2 splits, 384 blocks: 33.0 against 34.3 us unsplit at 32 tokens, 34.2 against
    // 36.0 us at 64)
    case 16: return launch<16, 4>(mw, mx, a, splits, stream);
    case 32:
      return blocks > 2ll * device_sms() ? launch<32, 3>(mw, mx, a, splits, stream)
                                         : launch<32, 5>(mw, mx, a, splits, stream);
    case 64:
      return blocks > 2ll * device_sms() ? launch<64, 3>(mw, mx, a, splits, stream)
                                         : launch<64, 4>(mw, mx, a, splits, stream);
    case 128: return launch<128, 3>(mw, mx, a, splits, stream);
    default: return launch<256, 4>(mw, mx, a, splits, stream);
  }
}

extern "C" int srlm_gemm_tn_tcgen05(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K,
                                    long long ldx, long long ldw, long long ldc, int splits, void* workspace,
                                    long long workspace_bytes, int* err_flag, int swiglu8, cudaStream_t stream) {
  return gemm_entry(X, W, C, c_dtype, M, N, K, ldx, ldw, ldc, splits, workspace, workspace_bytes, err_flag, swiglu8,
                    nullptr, stream);
}

// The same product for 1 to 128 tokens fused with the norms around it (see GemmFuse).  scale_parts may be
// null (X is already normalised); residual may be null (the product is stored to C, possibly through
// SwiGLU); with residual C is not written and may be null.
extern "C" int srlm_gemm_tn_tcgen05_fused(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K,
                                          long long ldx, long long ldw, long long ldc, int splits, void* workspace,
                                          long long workspace_bytes, int* err_flag, int swiglu8,
                                          const float* scale_parts, int n_parts, long long ld_parts, int norm_width,
                                          float eps, float* residual, long long ldr, const float* next_w,
                                          void* xw_out, long long ldxw, float* ss_out, long long ld_ss,
                                          cudaStream_t stream) {
  if (scale_parts && (n_parts <= 0 || ld_parts < M || norm_width <= 0 || !(eps > 0.f)))
    return refuse(ST_BAD_SIZE, "gemm_tcgen05_fused: n_parts=%d ld_parts=%lld norm_width=%d eps=%g", n_parts, ld_parts,
                  norm_width, (double)eps);
  if (residual && swiglu8) return refuse(ST_BAD_SIZE, "gemm_tcgen05_fused: residual and SwiGLU epilogues exclude each other");
  if (residual && (ldr < N || (next_w && (!xw_out || !ss_out || ldxw < N || ld_ss < M))))
    return refuse(ST_BAD_SIZE, "gemm_tcgen05_fused: residual epilogue with incomplete arguments");
  if (!residual && !C) return refuse(ST_BAD_SIZE, "gemm_tcgen05_fused: no output");
  const GemmFuse fuse{scale_parts, n_parts, ld_parts, norm_width > 0 ? 1.f / (float)norm_width : 0.f, eps, residual,
                      ldr, next_w, (bf16*)xw_out, ldxw, ss_out, ld_ss};
  if (residual) {            // C is not written: the size checks of the plain entry must not trip over it
    if (!C) C = residual;
    ldc = N;
  }
  return gemm_entry(X, W, C, c_dtype, M, N, K, ldx, ldw, ldc, splits, workspace, workspace_bytes, err_flag, swiglu8,
                    &fuse, stream);
}

// Launches wait_probe_kernel: a wait of at most limit_cycles (refused beyond 2e9, about a second) that runs out
// and writes `code` to err_flag.
extern "C" int srlm_wait_probe(int* err_flag, long long limit_cycles, int code, cudaStream_t stream) {
  if (!err_flag || limit_cycles <= 0 || limit_cycles > 2000000000ll || code == 0)
    return refuse(ST_BAD_SIZE, "wait_probe: a flag, a limit of 1..2e9 cycles and a nonzero code");
  wait_probe_kernel<<<1, 32, 0, stream>>>(err_flag, limit_cycles, code);
  return launched();
}

// The width of the token tiles this file's entry point picks for a product of M tokens and N weight
// rows, and the tile count from which it picks 256 (for the host-side plans, which must agree with it).
extern "C" int srlm_gemm_tcgen05_token_tile(int M, int N, int* min_tiles_for_256) {
  if (min_tiles_for_256) *min_tiles_for_256 = BN256_MIN_TILES;
  return token_tile(M, N, device_sms());
}

// How many of the product's tiles the persistent kernel would deal out by k-blocks on the current
// device (0: whole tiles only, or another kernel serves these sizes); for tests and notes.
extern "C" int srlm_gemm_tcgen05_dealt_tiles(int M, int N, int K) {
  const int sm_count = device_sms();
  const int bn = token_tile(M, N, sm_count);
  if (bn < 128) return 0;
  if (sm_count <= 0) return 0;
  static const bool pair_off = getenv("SRLM_GEMM_PAIR") && !atoi(getenv("SRLM_GEMM_PAIR"));
  if (bn == 256 && !pair_off)                 // pairs of SMs on tiles of 256 x 256
    return dealt_pair_tiles(((N + 2 * BM - 1) / (2 * BM)) * ((M + 255) / 256), (K + BK - 1) / BK, sm_count / 2);
  return dealt_tiles(((N + BM - 1) / BM) * ((M + bn - 1) / bn), (K + BK - 1) / BK, sm_count);
}

// ---------------------------------------------------------------------------
// The same product for callers that cannot allocate device memory: the split-K
// scratch is a device array inside the library image.  See srlm_no_alloc.h.
// ---------------------------------------------------------------------------
#include "srlm_no_alloc.h"

namespace srlm {
// [0, 65536): tile counters (zero on entry to the kernel); from 65536 on: float32 partial sums.
static __device__ __align__(256) unsigned char g_static_scratch[SRLM_STATIC_SCRATCH_BYTES];
static __device__ int g_static_err_flag;

constexpr int kMaxDevices = 64;
// Device addresses of the two symbols, looked up once per device.  In host code the symbols' names
// are only handles for cudaGetSymbolAddress; a kernel must be given the looked-up pointers.
static void* g_scratch_ptr[kMaxDevices];
static int* g_err_ptr[kMaxDevices];
static std::mutex g_static_mutex;

static int static_setup(int device) {
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_scratch_ptr[device]) return ST_OK;
  void* scratch = nullptr;
  void* flag = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&scratch, g_static_scratch);
  if (e != cudaSuccess) return refuse((int)e, "gemm_static: cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
  e = cudaGetSymbolAddress(&flag, g_static_err_flag);
  if (e != cudaSuccess) return refuse((int)e, "gemm_static: cudaGetSymbolAddress(flag): %s", cudaGetErrorString(e));
  g_err_ptr[device] = static_cast<int*>(flag);
  g_scratch_ptr[device] = scratch;
  return ST_OK;
}
}  // namespace srlm

extern "C" int srlm_gemm_tn_tcgen05_static(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K,
                                           long long ldx, long long ldw, long long ldc, int splits,
                                           int* err_flag_out, cudaStream_t stream) {
  if (M <= 0) return ST_OK;
  if (N <= 0 || K <= 0 || ldx < K || ldw < K || ldc < N)
    return refuse(ST_BAD_SIZE, "gemm_static: M=%d N=%d K=%d ldx=%lld ldw=%lld ldc=%lld", M, N, K, ldx, ldw, ldc);
  if (K % 8 || ldx % 8 || ldw % 8)
    return refuse(ST_BAD_SIZE, "gemm_static: K=%d and the leading dimensions must be multiples of 8", K);
  if (((uintptr_t)X | (uintptr_t)W) & 15) return refuse(ST_BAD_ALIGN, "gemm_static: operands must be 16-byte aligned");
  if (c_dtype != DT_F32 && c_dtype != DT_BF16) return refuse(ST_BAD_DTYPE, "gemm_static: output dtype %d", c_dtype);
  const int total_kb = (K + BK - 1) / BK;
  if (splits < 1) splits = 1;
  if (splits > total_kb) splits = total_kb;
  const int kb_per_split = (total_kb + splits - 1) / splits;
  splits = (total_kb + kb_per_split - 1) / kb_per_split;
  const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const long long tiles = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
  const long long need = 65536 + (long long)splits * tiles * BM * bn * 4;      // partial sums lie in whole tiles
  if (splits > 1 && (need > SRLM_STATIC_SCRATCH_BYTES || tiles * 4 > 65536))
    return refuse(ST_BAD_SIZE, "gemm_static: %d splits of a %d x %d product need %lld bytes of scratch, the "
                  "built-in array holds %d; use fewer splits or the entry point that takes a workspace",
                  splits, M, N, need, (int)SRLM_STATIC_SCRATCH_BYTES);
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices)
    return refuse(ST_BAD_SIZE, "gemm_static: no usable current device (%s)", cudaGetErrorString(e));
  int st = static_setup(device);
  if (st != ST_OK) return st;
  unsigned char* scratch = static_cast<unsigned char*>(g_scratch_ptr[device]);
  int* err = g_err_ptr[device];
  // what has to start at zero: the error flag always, the tile counters when they are used
  e = cudaMemsetAsync(err, 0, sizeof(int), stream);
  if (e == cudaSuccess && splits > 1) e = cudaMemsetAsync(scratch, 0, (size_t)tiles * 4, stream);
  if (e != cudaSuccess) return refuse((int)e, "gemm_static: clearing the scratch: %s", cudaGetErrorString(e));
  GemmArgs a{C, c_dtype == DT_F32, M, N, K, ldc, err, kb_per_split, nullptr, nullptr};
  if (splits > 1) {
    a.tile_counters = reinterpret_cast<int*>(scratch);
    a.partial = reinterpret_cast<float*>(scratch + 65536);
  }
  CUtensorMap mw, mx;       // built on the stack: nothing is cached, nothing is allocated
  if (!make_map(&mw, W, N, K, ldw, BM, true) || !make_map(&mx, X, M, K, ldx, bn, false))
    return refuse(ST_BAD_SIZE, "gemm_static: cuTensorMapEncodeTiled refused the operands");
  switch (bn) {
    case 16: st = launch<16, 4>(&mw, &mx, a, splits, stream); break;
    case 32: st = launch<32, 3>(&mw, &mx, a, splits, stream); break;
    case 64: st = launch<64, 3>(&mw, &mx, a, splits, stream); break;
    case 128: st = launch<128, 3>(&mw, &mx, a, splits, stream); break;
    default: st = launch<256, 4>(&mw, &mx, a, splits, stream); break;
  }
  if (st != ST_OK || !err_flag_out) return st;
  e = cudaStreamSynchronize(stream);
  if (e == cudaSuccess) e = cudaMemcpy(err_flag_out, err, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return refuse((int)e, "gemm_static: reading the error flag: %s", cudaGetErrorString(e));
  return ST_OK;
}
