// Small-batch matrix product for decoding: out[M, N] = x[M, K] * W[N, K]^T with M <= 64
// tokens, bfloat16 inputs, 32-bit accumulation, optional fused SwiGLU.
//
// At these sizes the product is bound by reading W once from HBM (intensity ~M flop per
// byte), so the kernel is a weight streamer: every lane keeps several 16-byte loads of W
// in flight (L1 bypassed), W's rows are the 16-row operand of mma.sync m16n8k16 and the
// tokens its 8-column operand, so that batch 1..64 costs no more instructions than batch
// 8.  K is split over the warps of a CTA and summed through shared memory in warp order;
// nothing is atomic, so a result does not depend on timing, and a token's result does
// not depend on the other tokens of the batch (each is its own MMA column).
//
// The 16 K-values of one MMA step are taken from memory in a permuted order that is the
// same for both operands (lane t holds elements 8t..8t+7 of a 32-wide block), which lets
// every lane fetch 16 contiguous bytes of a row instead of four 4-byte pieces.
//
// Reference counterpart: the one-row matrix-vector kernel (src/flint/cuda/matvec.cu:61-87)
// and cuBLAS for more rows (src/flint/cuda/gemm_cublas.cc:160-197); SwiGLU is a separate
// launch there (src/flint/cuda/swiglu.cu:29-59).
#include "common.cuh"

LLM_DEFINE_LAST_ERROR(llm_gemv_last_error)

constexpr int GEMV_WARPS = 8;

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: 8-token column tiles (M <= 8*NT).  MT: 16-row tiles per warp.  UNROLL: 32-wide K
// blocks whose loads are issued before the first MMA.  SWIGLU: W is [2*inter, K] (gate
// rows, then up rows); row r pairs with row inter + r and out is [M, inter].
template <int NT, int MT, int UNROLL, bool SWIGLU, typename TO>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_kernel(const __nv_bfloat16 *__restrict__ x, long long ldx, const __nv_bfloat16 *__restrict__ W,
            TO *__restrict__ out, long long ldo, int M, int N, int K, int k_split, int kb_per_part,
            long long part_stride) {
  constexpr int SETS = SWIGLU ? 2 : 1;
  extern __shared__ float red[];          // [k_split][row_groups][SETS*MT*NT*4][32]
  grid_dependents_launch();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int row_groups = GEMV_WARPS / k_split;
  const int ks = warp % k_split, rg = warp / k_split;
  const int n_out = SWIGLU ? N / 2 : N;                       // rows of out's N dimension
  const int row0 = (blockIdx.x * row_groups + rg) * (16 * MT);

  float acc[SETS][MT][NT][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[s][m][n][i] = 0.f;

  // Row pointers (clamped: rows beyond the matrix are read from its last row and dropped).
  const __nv_bfloat16 *wrow[SETS][MT][2];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        int r = row0 + m * 16 + g + 8 * h;
        r = r < n_out ? r : n_out - 1;
        wrow[s][m][h] = W + ((size_t)r + (size_t)s * n_out) * K;
      }
  const __nv_bfloat16 *xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int tok = n * 8 + g;
    xok[n] = tok < M;
    xrow[n] = x + (size_t)(xok[n] ? tok : 0) * ldx;
  }

  // blockIdx.y selects a part of K; each part writes its own partial result.
  const int kb_first = blockIdx.y * kb_per_part;
  const int n_kblocks = min((K + 31) / 32, kb_first + kb_per_part);
  out += (size_t)blockIdx.y * part_stride;
  uint4 a[UNROLL][SETS][MT][2];
  auto load_weights = [&](int kb0) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb0 + u) * 32 + 8 * t;
      const bool kok = k < K;                                 // K is a multiple of 8
#pragma unroll
      for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h)
            a[u][s][m][h] = kok ? ld_stream16(wrow[s][m][h] + k) : make_uint4(0, 0, 0, 0);
    }
  };
  // The weights do not depend on the kernel before this one: the first round's loads are
  // in flight while that kernel drains; the tokens are read after the wait.
  const int kb_begin = kb_first + ks * UNROLL;
  if (kb_begin < n_kblocks) load_weights(kb_begin);
  grid_dependency_wait();
  for (int kb0 = kb_begin; kb0 < n_kblocks; kb0 += k_split * UNROLL) {
    if (kb0 != kb_begin) load_weights(kb0);
    uint4 b[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb0 + u) * 32 + 8 * t;
      const bool kok = k < K;
#pragma unroll
      for (int n = 0; n < NT; ++n)
        b[u][n] = (kok && xok[n]) ? __ldg(reinterpret_cast<const uint4 *>(xrow[n] + k)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
          for (int n = 0; n < NT; ++n) {
            mma_bf16(acc[s][m][n], a[u][s][m][0].x, a[u][s][m][1].x, a[u][s][m][0].y, a[u][s][m][1].y,
                     b[u][n].x, b[u][n].y);
            mma_bf16(acc[s][m][n], a[u][s][m][0].z, a[u][s][m][1].z, a[u][s][m][0].w, a[u][s][m][1].w,
                     b[u][n].z, b[u][n].w);
          }
  }

  // Sum the K splits in split order through shared memory.
  constexpr int VALS = SETS * MT * NT * 4;
  if (k_split > 1) {
    float *mine = red + ((size_t)(ks * row_groups + rg) * VALS) * 32 + lane;
    int v = 0;
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) mine[(v++) * 32] = acc[s][m][n][i];
    __syncthreads();
    if (ks != 0) return;
    v = 0;
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
      for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float sum = acc[s][m][n][i];
            for (int o = 1; o < k_split; ++o) sum += red[((size_t)(o * row_groups + rg) * VALS + v) * 32 + lane];
            acc[s][m][n][i] = sum;
            ++v;
          }
  }

  // c0,c1: row g, tokens 2t, 2t+1; c2,c3: row g+8.
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = row0 + m * 16 + g + 8 * (i >> 1);
        const int tok = n * 8 + 2 * t + (i & 1);
        if (r < n_out && tok < M) {
          float v = acc[0][m][n][i];
          if (SWIGLU) {
            const float up = acc[SETS - 1][m][n][i];
            v = v / (1.f + expf(-v)) * up;
          }
          out[(size_t)tok * ldo + r] = from_float<TO>(v);
        }
      }
}

template <int NT, int MT, int UNROLL, bool SWIGLU, typename TO>
static int launch_gemv(const void *x, long long ldx, const void *W, void *out, long long ldo, int M, int N,
                       int K, int k_parts, long long part_stride, cudaStream_t stream) {
  constexpr int SETS = SWIGLU ? 2 : 1;
  const int n_out = SWIGLU ? N / 2 : N;
  const int kb_per_part = ((K + 31) / 32 + k_parts - 1) / k_parts;
  const int n_kblocks = kb_per_part;
  // Split K over the warps of a CTA while each warp keeps at least two rounds of loads;
  // when the matrix has too few rows to give every SM two CTAs, split further (down to
  // one round per warp), since CTAs, not warps, are what spreads over the SMs.
  int k_split = 1;
  while (k_split < GEMV_WARPS && n_kblocks / (k_split * 2) >= 4 * UNROLL) k_split *= 2;
  while (k_split < GEMV_WARPS && n_kblocks / (k_split * 2) >= UNROLL &&
         (n_out + (GEMV_WARPS / k_split) * 16 * MT - 1) / ((GEMV_WARPS / k_split) * 16 * MT) < 2 * sm_count())
    k_split *= 2;
  const int row_groups = GEMV_WARPS / k_split;
  const int rows_per_cta = row_groups * 16 * MT;
  const int grid = (n_out + rows_per_cta - 1) / rows_per_cta;
  const size_t smem = k_split > 1 ? (size_t)GEMV_WARPS * SETS * MT * NT * 4 * 32 * sizeof(float) : 0;
  auto kern = gemv_kernel<NT, MT, UNROLL, SWIGLU, TO>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "gemv attribute");
  llm_launch(kern, dim3(grid, k_parts), dim3(GEMV_WARPS * 32), smem, stream, (const __nv_bfloat16 *)x, ldx,
             (const __nv_bfloat16 *)W, (TO *)out, ldo, M, N, K, k_split, kb_per_part, part_stride);
  LLM_CHECK_LAUNCH("gemv");
  return LLM_OK;
}

template <bool SWIGLU, typename TO>
static int dispatch_gemv(const void *x, long long ldx, const void *W, void *out, long long ldo, int M, int N,
                         int K, int k_parts, long long part_stride, cudaStream_t stream) {
  if (M <= 8) return launch_gemv<1, 1, 4, SWIGLU, TO>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, stream);
  if (M <= 16) return launch_gemv<2, 1, 4, SWIGLU, TO>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, stream);
  if (M <= 32) return launch_gemv<4, 1, 2, SWIGLU, TO>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, stream);
  return launch_gemv<8, 1, 2, SWIGLU, TO>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, stream);
}

// How many parts of K a product of this shape is best cut into so that the GPU has
// about two CTAs per SM; 1 when the matrix has rows enough.  The caller adds the parts.
LLM_EXPORT int llm_gemv_suggest_parts(int M, int N, int K) {
  const int unroll = M <= 16 ? 4 : 2;
  const int ctas = (N + 15) / 16;
  const int kblocks = (K + 31) / 32;
  int parts = 1;
  while (parts < 8 && ctas * parts < 2 * sm_count() && kblocks / (parts * 2) >= GEMV_WARPS * unroll) parts *= 2;
  return parts;
}

// x [M, K] bfloat16 (row stride ldx), W [N, K] bfloat16 contiguous, out [M, N] (or
// [M, N/2] with swiglu) of out_dtype.  M <= 64, K a multiple of 8.
// With k_parts > 1 (plain product, 32-bit out only) part p covers its share of K and
// writes to out + p * part_stride; the sum over parts is the product.
LLM_EXPORT int llm_gemv_bf16(const void *x, long long ldx, const void *W, void *out, long long ldo, int out_dtype,
                             int M, int N, int K, int swiglu, int k_parts, long long part_stride,
                             cudaStream_t stream) {
  if (M == 0) return LLM_OK;
  LLM_REQUIRE(M > 0 && M <= 64, "gemv: %d tokens (1..64 are taken)", M);
  LLM_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && ldx % 8 == 0, "gemv: K=%d and the row stride must be multiples of 8", K);
  LLM_REQUIRE(!swiglu || N % 2 == 0, "gemv: a stacked gate|up matrix has an even number of rows");
  LLM_REQUIRE(k_parts >= 1 && k_parts <= 64 && (k_parts == 1 || (!swiglu && out_dtype == LLM_F32)),
              "gemv: parts of K need a plain product with 32-bit output");
  LLM_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)W % 16 == 0), "gemv: operands must be 16-byte aligned");
  if (swiglu) {
    if (out_dtype == LLM_BF16) return dispatch_gemv<true, __nv_bfloat16>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, stream);
    if (out_dtype == LLM_F32) return dispatch_gemv<true, float>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, stream);
  } else {
    if (out_dtype == LLM_BF16) return dispatch_gemv<false, __nv_bfloat16>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, stream);
    if (out_dtype == LLM_F32) return dispatch_gemv<false, float>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, stream);
  }
  LLM_FAIL("gemv: unknown output dtype %d", out_dtype);
}
