// Plain matrix product C[M,N] = A[M,K] * W[N,K]^T (+ bias) on the CUDA cores, 32-bit
// accumulate.  This is the matrix product of the true 32-bit path (no tensor cores, no
// reduced-precision mode) and the yardstick the fast bfloat16 products are tested
// against.  Every output element adds its K products in the order k = 0, 1, 2, ... with
// one accumulator, so a row's result does not depend on how many rows the call has or
// on where the row lies in the batch.
//
// Reference counterpart: the fp32 GEMM of the CPU backend (src/flint/cpu/matmul.cc:56-259)
// and cublasGemmEx with CUBLAS_COMPUTE_32F on CUDA (src/flint/cuda/gemm_cublas.cc:160-197).
#include "common.cuh"

LLM_DEFINE_LAST_ERROR(llm_gemm_plain_last_error)

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TA *__restrict__ A, long long lda, const TW *__restrict__ W, long long ldw,
                  const float *__restrict__ bias, TC *__restrict__ C, long long ldc, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;          // 16 x 16 threads, each 4 x 4 outputs
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 x 16 tile of each operand: 1024 values, 4 per thread; k is the fast index of
    // the load so that reads of a row are contiguous.
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const int e = tid + l * 256;
      const int r = e / BK, kk = e % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      As[kk][r] = (gm < M && gk < K) ? to_float(A[(size_t)gm * lda + gk]) : 0.f;
      Ws[kk][r] = (gn < N && gk < K) ? to_float(W[(size_t)gn * ldw + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      C[(size_t)gm * ldc + gn] = from_float<TC>(v);
    }
  }
}

template <typename TA, typename TW, typename TC>
static int launch(const void *A, long long lda, const void *W, long long ldw, const float *bias, void *C,
                  long long ldc, int M, int N, int K, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  LLM_REQUIRE(grid.y <= 65535, "gemm_plain: %d rows are too many for one launch", M);
  gemm_plain_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA *)A, lda, (const TW *)W, ldw, bias,
                                                         (TC *)C, ldc, M, N, K);
  LLM_CHECK_LAUNCH("gemm_plain");
  return LLM_OK;
}

// in_dtype is the type of A and W, out_dtype that of C.  Leading dimensions in elements.
LLM_EXPORT int llm_gemm_plain(int in_dtype, int out_dtype, const void *A, long long lda, const void *W,
                              long long ldw, const float *bias, void *C, long long ldc, int M, int N,
                              int K, cudaStream_t stream) {
  if (M == 0) return LLM_OK;
  LLM_REQUIRE(M > 0 && N > 0 && K > 0 && lda >= K && ldw >= K && ldc >= N, "gemm_plain: bad sizes");
  if (in_dtype == LLM_F32 && out_dtype == LLM_F32)
    return launch<float, float, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, stream);
  if (in_dtype == LLM_BF16 && out_dtype == LLM_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(A, lda, W, ldw, bias, C, ldc, M, N, K, stream);
  if (in_dtype == LLM_BF16 && out_dtype == LLM_F32)
    return launch<__nv_bfloat16, __nv_bfloat16, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, stream);
  LLM_FAIL("gemm_plain: unsupported dtypes in %d out %d", in_dtype, out_dtype);
}
