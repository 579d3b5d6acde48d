// out[m, n] = sum_k A[m, k] * W[n, k] (+ bias[n]) (+ residual[m, n]) on CUDA cores with
// float32 fused multiply-adds: the matrix product of the true 32-bit path (no tensor cores,
// no reduced-precision mode), and a plain reference for the tensor-core kernels.  Each output
// element is accumulated by one thread in ascending k, so its value does not depend on how
// many rows the call has or on where a row sits among them.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, THREADS = 256;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(THREADS)
gemm_simple_kernel(const TA* __restrict__ A, const TW* __restrict__ W, const float* __restrict__ bias,
                   const float* residual, TO* out, int M, int N, int K, int lda, int ldo) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int ty = tid / 16, tx = tid % 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < (BM * BK) / THREADS; i++) {
      const int idx = tid + i * THREADS;
      const int row = idx / BK, k = idx % BK;
      const int gm = m0 + row, gn = n0 + row, gk = k0 + k;
      As[k][row] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
      Ws[k][row] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; k++) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      if (residual) v += residual[(size_t)gm * ldo + gn];
      out[(size_t)gm * ldo + gn] = from_float<TO>(v);
    }
  }
}

template <typename TA, typename TW, typename TO>
int launch(const void* A, const void* W, const float* bias, const float* residual, void* out, int M, int N,
           int K, int lda, int ldo, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  sprout_launch(gemm_simple_kernel<TA, TW, TO>, grid, dim3(THREADS), 0, stream, (const TA*)A, (const TW*)W, bias, residual,
                (TO*)out, M, N, K, lda, ldo);
  return sprout_check_launch("gemm_simple");
}

}  // namespace

// A is [M, K] with row stride lda, W is [N, K] contiguous, out (and residual) [M, N] with row
// stride ldo.  `residual` may be the same buffer as `out`.  a_dtype is also the weight's dtype.
SPROUT_API int sprout_gemm_simple(const void* A, const void* W, const float* bias, const float* residual,
                                  void* out, int a_dtype, int out_dtype, int M, int N, int K, int lda, int ldo,
                                  cudaStream_t stream) {
  SPROUT_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_simple: sizes must be positive (M=%d N=%d K=%d)", M, N, K);
  SPROUT_REQUIRE(A && W && out, "gemm_simple: null pointer");
  SPROUT_REQUIRE(lda >= K && ldo >= N, "gemm_simple: row strides smaller than the rows");
  SPROUT_REQUIRE(!residual || out_dtype == SPROUT_F32, "gemm_simple: a residual needs a float32 output");
  SPROUT_REQUIRE((M + BM - 1) / BM <= 65535, "gemm_simple: too many rows (%d)", M);
  if (a_dtype == SPROUT_F32 && out_dtype == SPROUT_F32)
    return launch<float, float, float>(A, W, bias, residual, out, M, N, K, lda, ldo, stream);
  if (a_dtype == SPROUT_BF16 && out_dtype == SPROUT_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(A, W, bias, residual, out, M, N, K, lda, ldo, stream);
  if (a_dtype == SPROUT_BF16 && out_dtype == SPROUT_F32)
    return launch<__nv_bfloat16, __nv_bfloat16, float>(A, W, bias, residual, out, M, N, K, lda, ldo, stream);
  return sprout_fail("gemm_simple: unsupported dtypes a=%d out=%d", a_dtype, out_dtype);
}
