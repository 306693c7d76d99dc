// C[M,N] = X[M,K] . W[N,K]^T for M <= 16 tokens (decode): a weight-streaming
// kernel.  Each block owns 16 weight rows; its 8 warps split K among them and
// every lane pulls 16 bytes of a weight row straight from global memory into
// registers, many loads in flight, no shared-memory staging and no barrier in
// the loop.  The products run on the tensor cores with mma.sync m16n8k16: the
// 16 weight rows are the M side, up to 8 tokens the N side (two tiles for up to
// 16 tokens), float32 accumulation.  Because A and B may permute K in the same
// way, a lane's 8 consecutive k values serve as the fragments of two k-steps, so
// the global loads stay 16 bytes wide and whole 32-byte sectors are used.
//
// For a handful of tokens the product is bound by HBM alone; what matters is
// that all SMs stream at once with little fixed cost per launch.  The one-tile
// tcgen05 kernel with 16-token tiles and its K splits in a thread-block cluster
// (gemm_tcgen05.cu) does that better still (a decode layer's four products at 8
// tokens: 70.8 against 82.8 us), so this kernel serves no step unless
// KernelLibrary.skinny_max_tokens is raised; its tests keep it honest.
// The eight warps' partial sums are added in warp order: the same on every run.
//
// Replaces, for decode, the same reference code as gemm_tcgen05.cu
// (native/cuda/safetyraise_cuda.cu:43-63, src/artifact/mod.rs:377-405).
#include "common.cuh"

namespace srlm {

// Optional fusions with the norms around a product (decode steps, M <= 8):
//  * scale_parts: the tokens X are (residual * norm weight) in bfloat16, not yet divided by their RMS;
//    the sums of squares of each token's residual row come in n_parts partial rows [n_parts][8] and the
//    product is scaled by rsqrt(sum / norm_width + eps) per token.  Multiplying after the product is
//    the same linear map, and the division happens in float32.
//  * residual: instead of storing the product, add it to the float32 residual stream in place; and, if
//    next_w is given, also emit for the norm that follows xw_out = bf16(residual * next_w) and this
//    block's share of the row sums of squares, ss_out[blockIdx.x][token].
struct SkinnyFuse {
  const float* scale_parts;
  int n_parts;
  float inv_width, eps;
  float* residual;
  long long ldr;
  const float* next_w;
  bf16* xw_out;
  long long ldxw;
  float* ss_out;
};

constexpr int SK_WARPS = 8;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_ROWS = 16;

// The weights are read once per step: not kept in L1, and the first to leave L2, which then keeps what is
// read again between the products (tokens, block tables, norm weights, partial sums).
__device__ __forceinline__ uint4 ld_stream16(const void* p, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ uint4 ld_cached16(const void* p) {      // the tokens: read by every block
  return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, typename TO, int SK_UNROLL>     // MT token tiles of 8; SK_UNROLL groups of 32 k per batch
__global__ void __launch_bounds__(SK_THREADS, SK_UNROLL == 2 ? 3 : 1)     // the lean form: three blocks per SM
gemm_skinny_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, TO* __restrict__ C, int M, int N, int K,
                   long long ldx, long long ldw, long long ldc, int swiglu8, const SkinnyFuse fuse) {
  __shared__ float part[SK_WARPS][SK_ROWS][MT * 8 + 1];
  __shared__ float ss_warp[SK_WARPS][8];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, q = lane & 3;
  const int n0 = blockIdx.x * SK_ROWS;
  // this warp's share of K, in groups of 32
  const int groups = (K + 31) / 32;
  const int per_warp = (groups + SK_WARPS - 1) / SK_WARPS;
  const int g_lo = warp * per_warp, g_hi = min(groups, g_lo + per_warp);

  const int row_a = min(n0 + r, N - 1), row_b = min(n0 + r + 8, N - 1);      // clamped: never stored if beyond N
  const bf16* wa = W + (size_t)row_a * ldw + 8 * q;
  const bf16* wb = W + (size_t)row_b * ldw + 8 * q;
  const bf16* xs[MT];
  bool x_ok[MT];
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    const int m = t * 8 + r;                   // B fragment: column n = lane / 4 is the token
    x_ok[t] = m < M;
    xs[t] = X + (size_t)min(m, M - 1) * ldx + 8 * q;
  }
  float acc[MT][4];
#pragma unroll
  for (int t = 0; t < MT; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;

  // Two batches of weight loads are kept in flight: the next batch is requested before the current
  // one is multiplied.
  const uint4 zero = make_uint4(0, 0, 0, 0);
  const uint64_t once = l2_evict_first_policy();
  uint4 a[2][SK_UNROLL], b[2][SK_UNROLL];
  auto load_w = [&](int g, uint4 (&aa)[SK_UNROLL], uint4 (&bb)[SK_UNROLL]) {
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int k = (g + u) * 32;
      const bool in = g + u < g_hi && k + 8 * q < K;        // K is a multiple of 8: a 16-byte piece is whole
      aa[u] = in ? ld_stream16(wa + k, once) : zero;
      bb[u] = in ? ld_stream16(wb + k, once) : zero;
    }
  };
  load_w(g_lo, a[0], b[0]);
  pdl_wait();
  // the epilogue's reads of the residual stream and of the next norm's weight are requested now, so that
  // their latency passes under the main loop instead of behind it (idx = m * 16 + row, as below)
  float res_old = 0.f, next_scale = 0.f;
  {
    const int m = threadIdx.x / SK_ROWS, row = threadIdx.x % SK_ROWS;
    if (fuse.residual && threadIdx.x < SK_ROWS * MT * 8 && m < M && n0 + row < N) {
      res_old = fuse.residual[(size_t)m * fuse.ldr + n0 + row];
      if (fuse.next_w) next_scale = __ldg(fuse.next_w + n0 + row);
    }
  }
  int buf = 0;
  for (int g = g_lo; g < g_hi; g += SK_UNROLL, buf ^= 1) {
    uint4 x[SK_UNROLL][MT];
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int k = (g + u) * 32;
      const bool in = g + u < g_hi && k + 8 * q < K;
#pragma unroll
      for (int t = 0; t < MT; ++t) x[u][t] = (in && x_ok[t]) ? ld_cached16(xs[t] + k) : zero;
    }
    if (buf == 0) load_w(g + SK_UNROLL, a[1], b[1]); else load_w(g + SK_UNROLL, a[0], b[0]);
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
#pragma unroll
      for (int t = 0; t < MT; ++t) {
        // the lane's 8 consecutive k: pairs 0,1 are k-step 0 (columns c, c+8), pairs 2,3 are k-step 1
        const uint4 av = buf == 0 ? a[0][u] : a[1][u], bv = buf == 0 ? b[0][u] : b[1][u];
        mma_16816(acc[t], av.x, bv.x, av.y, bv.y, x[u][t].x, x[u][t].y);
        mma_16816(acc[t], av.z, bv.z, av.w, bv.w, x[u][t].z, x[u][t].w);
      }
    }
  }
  // D fragment: rows r and r + 8, tokens 2q and 2q + 1 of each tile
#pragma unroll
  for (int t = 0; t < MT; ++t) {
    part[warp][r][t * 8 + 2 * q] = acc[t][0];
    part[warp][r][t * 8 + 2 * q + 1] = acc[t][1];
    part[warp][r + 8][t * 8 + 2 * q] = acc[t][2];
    part[warp][r + 8][t * 8 + 2 * q + 1] = acc[t][3];
  }
  // 1 / RMS of each token's row from the partial sums of squares, behind the main loop: nothing in the
  // loop needs it, and in front of it the loads and two block-wide barriers held up every warp's stream
  // (3 us a launch, measured).  Every thread takes partial rows (8 tokens each); a warp adds its threads'
  // rows in nine shuffles (the lanes halve the tokens they keep three times, then the four lanes of a
  // token add up: lane 4 t ends with token t); the warps' sums meet in shared memory at the barrier the
  // epilogue needs anyway.  The order of the additions is fixed by the thread layout.
  if (fuse.scale_parts) {
    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = threadIdx.x; p < fuse.n_parts; p += SK_THREADS) {
      const float4 lo = __ldg(reinterpret_cast<const float4*>(fuse.scale_parts + (size_t)p * 8));
      const float4 hi = __ldg(reinterpret_cast<const float4*>(fuse.scale_parts + (size_t)p * 8 + 4));
      v[0] += lo.x; v[1] += lo.y; v[2] += lo.z; v[3] += lo.w;
      v[4] += hi.x; v[5] += hi.y; v[6] += hi.z; v[7] += hi.w;
    }
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
    float w4[4], w2[2];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      w4[j] = (b4 ? v[4 + j] : v[j]) + __shfl_xor_sync(0xffffffffu, b4 ? v[j] : v[4 + j], 16);
#pragma unroll
    for (int j = 0; j < 2; ++j)
      w2[j] = (b3 ? w4[2 + j] : w4[j]) + __shfl_xor_sync(0xffffffffu, b3 ? w4[j] : w4[2 + j], 8);
    float w1 = (b2 ? w2[1] : w2[0]) + __shfl_xor_sync(0xffffffffu, b2 ? w2[0] : w2[1], 4);
    w1 += __shfl_xor_sync(0xffffffffu, w1, 2);
    w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
    if ((lane & 3) == 0) ss_warp[warp][lane >> 2] = w1;
  }
  __syncthreads();
  auto row_scale = [&](int m) {          // the warps' sums in warp order
    float ss = 0.f;
#pragma unroll
    for (int w = 0; w < SK_WARPS; ++w) ss += ss_warp[w][m & 7];
    return rsqrtf(ss * fuse.inv_width + fuse.eps);
  };
  if (swiglu8) {
    // the block's 16 rows are 8 gate rows then the 8 up rows of the same features: out = silu(gate) * up
    for (int idx = threadIdx.x; idx < 8 * MT * 8; idx += SK_THREADS) {
      const int m = idx / 8, row = idx % 8;
      if (m < M && n0 + row + 8 < N) {
        float gsum = 0.f, usum = 0.f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) { gsum += part[w][row][m]; usum += part[w][row + 8][m]; }
        if (fuse.scale_parts) { const float sc = row_scale(m); gsum *= sc; usum *= sc; }
        const float sg = gsum >= 0.f ? gsum / (1.f + expf(-gsum)) : gsum * (expf(gsum) / (1.f + expf(gsum)));
        C[(size_t)m * ldc + (n0 >> 1) + row] = from_float<TO>(sg * usum);
      }
    }
    return;
  }
  // idx = m * 16 + row: the 16 rows of a token sit in one half-warp (MT * 8 * 16 <= 256 threads)
  {
    const int idx = threadIdx.x;
    const int m = idx / SK_ROWS, row = idx % SK_ROWS;
    const bool live = idx < SK_ROWS * MT * 8 && m < M && n0 + row < N;
    float s = 0.f;
    if (live) {
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) s += part[w][row][m];
      if (fuse.scale_parts) s *= row_scale(m);
    }
    if (!fuse.residual) {
      if (live) C[(size_t)m * ldc + n0 + row] = from_float<TO>(s);
      return;
    }
    float r = 0.f;
    if (live) {
      r = res_old + s;
      fuse.residual[(size_t)m * fuse.ldr + n0 + row] = r;
      if (fuse.next_w) fuse.xw_out[(size_t)m * fuse.ldxw + n0 + row] = __float2bfloat16_rn(r * next_scale);
    }
    if (fuse.next_w && idx < SK_ROWS * MT * 8) {       // whole half-warps, so the shuffles below are complete
      float sq = r * r;
      sq += __shfl_xor_sync(0xffffffffu, sq, 8);
      sq += __shfl_xor_sync(0xffffffffu, sq, 4);
      sq += __shfl_xor_sync(0xffffffffu, sq, 2);
      sq += __shfl_xor_sync(0xffffffffu, sq, 1);
      if (row == 0 && m < 8) fuse.ss_out[(size_t)blockIdx.x * 8 + m] = sq;
    }
  }
}

// early: the kernel may start under the tail of the kernel ahead of it in the stream (programmatic
// dependent launch): its blocks request their first weights, which no kernel writes, and only then wait
// for that kernel's results.  Measured on B200 in a decode step at 8B sizes (batch 8): worth 0.4 to 2.8 %
// of the step, depending on the machine, when every product but the one behind the attention kernel is
// launched so (3.94 -> 3.92 ms on one, 3.97 -> 3.86 ms on another); with that one too the step takes
// 5.7 ms, wherever the kernels place their triggers, with or without the attention kernel's clusters.
// A chain of these products alone gains 5 % with all of them early.  So the caller says which product
// follows a mixer's kernel, and that one is launched in plain stream order.
template <int MT, typename TO, int U>
static int launch_skinny_u(const void* X, const void* W, void* C, int M, int N, int K, long long ldx, long long ldw,
                           long long ldc, int swiglu8, const SkinnyFuse& fuse, int early, cudaStream_t stream) {
  const dim3 grid((N + SK_ROWS - 1) / SK_ROWS), block(SK_THREADS);
  if (early)
    launch_pdl(gemm_skinny_kernel<MT, TO, U>, grid, block, 0, stream, (const bf16*)X, (const bf16*)W, (TO*)C, M, N, K,
               ldx, ldw, ldc, swiglu8, fuse);
  else
    gemm_skinny_kernel<MT, TO, U><<<grid, block, 0, stream>>>((const bf16*)X, (const bf16*)W, (TO*)C, M, N, K, ldx,
                                                              ldw, ldc, swiglu8, fuse);
  return launched();
}

template <int MT, typename TO>
static int launch_skinny(const void* X, const void* W, void* C, int M, int N, int K, long long ldx, long long ldw,
                         long long ldc, int swiglu8, const SkinnyFuse& fuse, int early, cudaStream_t stream) {
  // Four groups of 32 k per batch of loads (128 registers, two blocks per SM) stream best when the blocks
  // fill whole rounds of two per SM.  A product of a little more than that -- up to three blocks per SM --
  // runs as ONE round of the leaner form (two groups per batch, 80 registers, three blocks per SM)
  // instead of a full round and a nearly empty one.  Measured on B200 (8 tokens, chains in a CUDA graph):
  // 384 blocks (QKV at 8B sizes) 13.2 -> 10.9 us; 320 blocks (the output and down projections at 14B and 32B
  // sizes) 14.9 -> 12.7, 44.3 -> 38.8, 23.1 -> 19.4, 64.6 -> 56.5 us; for every other block count the
  // form with four groups is as fast or faster (256 blocks: 7.9 against 10.1 us).
  if (MT == 1) {
    static int sms = 0;
    if (sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int blocks = (N + SK_ROWS - 1) / SK_ROWS;
    if (sms > 0 && blocks > 2 * sms && blocks <= 3 * sms)
      return launch_skinny_u<MT, TO, 2>(X, W, C, M, N, K, ldx, ldw, ldc, swiglu8, fuse, early, stream);
  }
  return launch_skinny_u<MT, TO, 4>(X, W, C, M, N, K, ldx, ldw, ldc, swiglu8, fuse, early, stream);
}

}  // namespace srlm

using namespace srlm;

static int skinny_entry(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K, long long ldx,
                        long long ldw, long long ldc, int swiglu8, const SkinnyFuse& fuse, int early,
                        cudaStream_t stream) {
  if (M <= 0) return ST_OK;
  if (swiglu8 && (N % 16 || ldc < N / 2))
    return refuse(ST_BAD_SIZE, "gemm_skinny: the SwiGLU epilogue needs N=%d a multiple of 16 and ldc >= N/2", N);
  if (M > 16) return refuse(ST_BAD_SIZE, "gemm_skinny: M=%d; this kernel takes at most 16 tokens", M);
  if (N <= 0 || K <= 0 || ldx < K || ldw < K || (!swiglu8 && !fuse.residual && ldc < N))
    return refuse(ST_BAD_SIZE, "gemm_skinny: M=%d N=%d K=%d ldx=%lld ldw=%lld ldc=%lld", M, N, K, ldx, ldw, ldc);
  if (K % 8 || ldx % 8 || ldw % 8 || (((uintptr_t)X | (uintptr_t)W) & 15))
    return refuse(ST_BAD_ALIGN, "gemm_skinny: K and the leading dimensions must be multiples of 8 and the operands "
                  "16-byte aligned (16-byte loads)");
  if ((fuse.scale_parts || fuse.residual) && M > 8)
    return refuse(ST_BAD_SIZE, "gemm_skinny: the norm fusions take at most 8 tokens, got %d", M);
  if (fuse.residual && swiglu8) return refuse(ST_BAD_SIZE, "gemm_skinny: residual and SwiGLU epilogues exclude each other");
  if (fuse.residual && (fuse.ldr < N || (fuse.next_w && (!fuse.xw_out || !fuse.ss_out || fuse.ldxw < N))))
    return refuse(ST_BAD_SIZE, "gemm_skinny: residual epilogue with incomplete arguments");
  if (c_dtype == DT_BF16)
    return M <= 8 ? launch_skinny<1, bf16>(X, W, C, M, N, K, ldx, ldw, ldc, swiglu8, fuse, early, stream)
                  : launch_skinny<2, bf16>(X, W, C, M, N, K, ldx, ldw, ldc, swiglu8, fuse, early, stream);
  if (c_dtype == DT_F32)
    return M <= 8 ? launch_skinny<1, float>(X, W, C, M, N, K, ldx, ldw, ldc, swiglu8, fuse, early, stream)
                  : launch_skinny<2, float>(X, W, C, M, N, K, ldx, ldw, ldc, swiglu8, fuse, early, stream);
  return refuse(ST_BAD_DTYPE, "gemm_skinny: output dtype %d", c_dtype);
}

extern "C" int srlm_gemm_tn_skinny(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K,
                                   long long ldx, long long ldw, long long ldc, int swiglu8, int early,
                                   cudaStream_t stream) {
  const SkinnyFuse none{};
  return skinny_entry(X, W, C, c_dtype, M, N, K, ldx, ldw, ldc, swiglu8, none, early, stream);
}

// early (both entry points): 1 lets the kernel start under the tail of the kernel ahead of it, see launch_skinny_u.
// The same product fused with the norms around it (see SkinnyFuse).  scale_parts may be null (X is already
// normalised); residual may be null (the product is stored to C as usual, possibly through SwiGLU).
extern "C" int srlm_gemm_tn_skinny_fused(const void* X, const void* W, void* C, int c_dtype, int M, int N, int K,
                                         long long ldx, long long ldw, long long ldc, int swiglu8,
                                         const float* scale_parts, int n_parts, int norm_width, float eps,
                                         float* residual, long long ldr, const float* next_w, void* xw_out,
                                         long long ldxw, float* ss_out, int early, cudaStream_t stream) {
  if (scale_parts && (n_parts <= 0 || norm_width <= 0 || !(eps > 0.f)))
    return refuse(ST_BAD_SIZE, "gemm_skinny_fused: n_parts=%d norm_width=%d eps=%g", n_parts, norm_width, (double)eps);
  const SkinnyFuse fuse{scale_parts, n_parts, norm_width > 0 ? 1.f / (float)norm_width : 0.f, eps, residual, ldr,
                        next_w, (bf16*)xw_out, ldxw, ss_out};
  return skinny_entry(X, W, C, c_dtype, M, N, K, ldx, ldw, ldc, swiglu8, fuse, early, stream);
}
