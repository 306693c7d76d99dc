// C[M,N] = A[M,K] . W[N,K]^T with float32 FMA accumulation (no tensor cores,
// no reduced-precision mode).  Every output element sums over k in the order
// 0..K-1 whatever M and N are, so a row's result does not depend on the batch.
// This is the matrix product of the float32 path and the reference twin of the
// tensor-core GEMM.  Formula: src/artifact/mod.rs:377-405.
#include "common.cuh"

namespace srlm {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_tn_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ C, int M, int N,
                    int K, long long lda, long long ldw, long long ldc) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 columns each: 1024 elements, 4 per thread
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / BK, c = idx % BK;
      const int k = k0 + c;
      As[c][r] = (m0 + r < M && k < K) ? to_float(A[(size_t)(m0 + r) * lda + k]) : 0.f;
      Ws[c][r] = (n0 + r < N && k < K) ? to_float(W[(size_t)(n0 + r) * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = As[kk][tm + i]; w[i] = Ws[kk][tn + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + tm + i, n = n0 + tn + j;
      if (m < M && n < N) C[(size_t)m * ldc + n] = from_float<TO>(acc[i][j]);
    }
}

template <typename TA, typename TW, typename TO>
static int run(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
               long long ldc, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  gemm_tn_simt_kernel<TA, TW, TO><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, (TO*)C, M, N, K,
                                                            lda, ldw, ldc);
  return launched();
}

}  // namespace srlm

using namespace srlm;

extern "C" int srlm_gemm_tn_simt(const void* A, int a_dtype, const void* W, int w_dtype, void* C,
                                 int c_dtype, int M, int N, int K, long long lda, long long ldw,
                                 long long ldc, cudaStream_t stream) {
  if (M <= 0) return ST_OK;
  if (N <= 0 || K <= 0 || lda < K || ldw < K || ldc < N)
    return refuse(ST_BAD_SIZE, "gemm_tn_simt: M=%d N=%d K=%d lda=%lld ldw=%lld ldc=%lld", M, N, K, lda,
                  ldw, ldc);
  if ((M + BM - 1) / BM > 65535)
    return refuse(ST_BAD_SIZE, "gemm_tn_simt: M=%d exceeds %d rows", M, 65535 * BM);
  if (a_dtype == DT_F32 && w_dtype == DT_F32 && c_dtype == DT_F32)
    return run<float, float, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  if (a_dtype == DT_BF16 && w_dtype == DT_BF16 && c_dtype == DT_BF16)
    return run<bf16, bf16, bf16>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  if (a_dtype == DT_BF16 && w_dtype == DT_BF16 && c_dtype == DT_F32)
    return run<bf16, bf16, float>(A, W, C, M, N, K, lda, ldw, ldc, stream);
  return refuse(ST_BAD_DTYPE, "gemm_tn_simt: dtypes (%d, %d) -> %d are not offered", a_dtype, w_dtype,
                c_dtype);
}
