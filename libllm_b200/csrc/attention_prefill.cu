// Causal grouped-query attention for prompt steps over the paged bfloat16 cache: the
// flash-attention form (a running maximum and sum per query row, scores never stored),
// on the tensor cores.
//
// One CTA takes 64 query rows of one head of one sequence; its four warps own 16 rows
// each.  Keys and values are walked page by page: a page of the cache holds 64 tokens of
// one kv head as one contiguous [64, d] block, which is exactly one key tile, so a tile is
// fetched with plain 16-byte asynchronous copies (two tiles in flight) and no gather.
// S = Q K^T and O += P V run as mma.sync m16n8k16 with bfloat16 operands and 32-bit
// accumulators; the probabilities go from the accumulators of the first product straight
// into the operand registers of the second.  Maximum, exponentials (exp2 of pre-scaled
// scores), sums and the output accumulation are 32-bit.
//
// The step's own keys are in the cache already when this runs (the rotation kernel wrote
// them), so a sequence that brings tokens i = 0..n-1 behind `past` cached ones sees, for
// its token i, keys 0..past+i: the mask aligned to the bottom right of the reference
// (src/flint/operators.cc:119-124).  Head h reads kv head h / (heads / kv_heads)
// (src/flint/operators.cc:43-56); scores are scaled by 1/sqrt(d) unless another scale is
// given (src/flint/operators.cc:115-117).  The reference calls FlashAttention-2's forward
// kernel here (src/flint/cuda/flash_attn.cc:101-186).
//
// Rows are padded by 16 bytes in shared memory, which spreads the eight rows of an
// ldmatrix over all banks for every head size that is a multiple of 16.
#include "common.cuh"
#include "mma_tiles.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_attention_prefill_last_error)

constexpr int AP_WARPS = 4;
constexpr int AP_BM = 16 * AP_WARPS;     // query rows per CTA
constexpr int AP_BN = 64;                // keys per tile = tokens per page

template <int D>
__global__ void __launch_bounds__(AP_WARPS * 32)
attention_prefill_kernel(const __nv_bfloat16 *__restrict__ q, long long q_stride, __nv_bfloat16 *__restrict__ out,
                         long long out_stride, const __nv_bfloat16 *__restrict__ kc,
                         const __nv_bfloat16 *__restrict__ vc, const int *__restrict__ seq_start,
                         const int *__restrict__ seq_past, const int *__restrict__ page_table, int pt_stride,
                         int n_heads, int n_kv, int window, float scale_log2) {
  constexpr int LD = D + 8;                                  // padded row, in elements
  constexpr int CHUNKS = D / 8;                              // 16-byte pieces of a row
  constexpr int KS = D / 16;                                 // k-steps of Q K^T
  constexpr int NT = AP_BN / 8;                              // key tiles of 8 in S
  constexpr int DT = D / 8;                                  // channel tiles of 8 in O
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16 *sQ = reinterpret_cast<__nv_bfloat16 *>(smem_raw);
  __nv_bfloat16 *sK = sQ + AP_BM * LD;                       // [2][AP_BN][LD]
  __nv_bfloat16 *sV = sK + 2 * AP_BN * LD;                   // [2][AP_BN][LD]

  grid_dependents_launch();
  grid_dependency_wait();
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = seq_start[b], n_q = seq_start[b + 1] - q0, past = seq_past[b];
  const int tile = gridDim.x - 1 - blockIdx.x;               // long tiles first
  const int r0 = tile * AP_BM;
  if (r0 >= n_q) return;
  const int rows = min(AP_BM, n_q - r0);
  const int kvh = h / (n_heads / n_kv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  // key tiles this CTA needs: the first row's window start .. the last row's own position
  const int last_tile = (past + r0 + rows - 1) / AP_BN;
  const int first_tile = window > 0 ? max(0, past + r0 - window + 1) / AP_BN : 0;
  const int *pt = page_table + (size_t)b * pt_stride;

  auto load_kv = [&](int kt, int stage) {
    const int page = pt[kt];
    const size_t base = ((size_t)page * n_kv + kvh) * AP_BN * D;
    __nv_bfloat16 *dk = sK + stage * AP_BN * LD, *dv = sV + stage * AP_BN * LD;
    for (int c = tid; c < AP_BN * CHUNKS; c += AP_WARPS * 32) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      cp_async16(dk + r * LD + ch * 8, kc + base + (size_t)r * D + ch * 8, true);
      cp_async16(dv + r * LD + ch * 8, vc + base + (size_t)r * D + ch * 8, true);
    }
  };

  // Q tile (rows beyond the sequence are zeros) and the first key tile
  for (int c = tid; c < AP_BM * CHUNKS; c += AP_WARPS * 32) {
    const int r = c / CHUNKS, ch = c % CHUNKS;
    const bool ok = r < rows;
    cp_async16(sQ + r * LD + ch * 8, q + (size_t)(q0 + r0 + (ok ? r : 0)) * q_stride + (size_t)h * D + ch * 8, ok);
  }
  load_kv(first_tile, 0);
  cp_async_commit();

  unsigned qf[KS][4];
  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  // absolute positions of this thread's two rows
  const int pos0 = past + r0 + warp * 16 + g, pos1 = pos0 + 8;

  for (int kt = first_tile; kt <= last_tile; ++kt) {
    const int stage = (kt - first_tile) & 1;
    if (kt + 1 <= last_tile) load_kv(kt + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (kt == first_tile) {
#pragma unroll
      for (int ks = 0; ks < KS; ++ks)
        ldmatrix_x4(qf[ks], sQ + (warp * 16 + (lane & 15)) * LD + ks * 16 + (lane >> 4) * 8);
    }
    const __nv_bfloat16 *tk = sK + stage * AP_BN * LD, *tv = sV + stage * AP_BN * LD;

    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[n][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; ++n2) {
        unsigned kb[4];
        ldmatrix_x4(kb, tk + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
        mma16816(s[2 * n2], qf[ks], kb[0], kb[1]);
        mma16816(s[2 * n2 + 1], qf[ks], kb[2], kb[3]);
      }
    }

    // mask: key j is seen by the row at position p when j <= p and (no window or j > p - window)
    const int k0 = kt * AP_BN;
    const bool edge = (k0 + AP_BN - 1 > past + r0) || (window > 0 && k0 <= past + r0 + AP_BM - 1 - window);
    if (edge) {
#pragma unroll
      for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = k0 + n * 8 + 2 * t + (j & 1);
          const int p = (j & 2) ? pos1 : pos0;
          const bool seen = key <= p && (window <= 0 || key > p - window);
          if (!seen) s[n][j] = -INFINITY;
        }
    }

    // running maximum and sum per row (rows g and g + 8 of the warp's 16)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
    }
    float alpha[2], moff[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      // a row that has seen no key yet keeps m = -inf; its exponentials are taken against 0
      moff[r] = m_new == -INFINITY ? 0.f : m_new * scale_log2;
      alpha[r] = m_run[r] == -INFINITY ? 0.f : exp2f(m_run[r] * scale_log2 - moff[r]);
      m_run[r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      s[n][0] = exp2f(fmaf(s[n][0], scale_log2, -moff[0]));
      s[n][1] = exp2f(fmaf(s[n][1], scale_log2, -moff[0]));
      s[n][2] = exp2f(fmaf(s[n][2], scale_log2, -moff[1]));
      s[n][3] = exp2f(fmaf(s[n][3], scale_log2, -moff[1]));
      sum[0] += s[n][0] + s[n][1];
      sum[1] += s[n][2] + s[n][3];
    }
    l_run[0] = l_run[0] * alpha[0] + sum[0];
    l_run[1] = l_run[1] * alpha[1] + sum[1];
#pragma unroll
    for (int i = 0; i < DT; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < AP_BN / 16; ++kk) {
      unsigned pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d2 = 0; d2 < DT / 2; ++d2) {
        unsigned vb[4];
        ldmatrix_x4_trans(vb, tv + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + d2 * 16 + (lane >> 4) * 8);
        mma16816(o[2 * d2], pa, vb[0], vb[1]);
        mma16816(o[2 * d2 + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();                      // the stage is free for the copy after next
  }
  cp_async_wait<0>();

  // the row sums live spread over the four lanes of a row
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const float inv_a = 1.f / l_run[0], inv_b = 1.f / l_run[1];
  __nv_bfloat16 *oa = out + (size_t)(q0 + r0 + row_a) * out_stride + (size_t)h * D + 2 * t;
  __nv_bfloat16 *ob = out + (size_t)(q0 + r0 + row_b) * out_stride + (size_t)h * D + 2 * t;
#pragma unroll
  for (int i = 0; i < DT; ++i) {
    if (row_a < rows) *reinterpret_cast<unsigned *>(oa + i * 8) = pack_bf16(o[i][0] * inv_a, o[i][1] * inv_a);
    if (row_b < rows) *reinterpret_cast<unsigned *>(ob + i * 8) = pack_bf16(o[i][2] * inv_b, o[i][3] * inv_b);
  }
}

template <int D>
static int launch_prefill(const void *q, long long q_stride, void *out, long long out_stride, const void *kc,
                          const void *vc, const int *seq_start, const int *seq_past, const int *page_table,
                          int pt_stride, int n_seqs, int max_q_len, int n_heads, int n_kv, int window, float scale,
                          cudaStream_t stream) {
  constexpr int LD = D + 8;
  const size_t smem = (size_t)(AP_BM + 4 * AP_BN) * LD * sizeof(__nv_bfloat16);
  auto kern = attention_prefill_kernel<D>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "attention_prefill attribute");
  dim3 grid((max_q_len + AP_BM - 1) / AP_BM, n_heads, n_seqs);
  llm_launch(kern, grid, dim3(AP_WARPS * 32), smem, stream, (const __nv_bfloat16 *)q, q_stride, (__nv_bfloat16 *)out,
             out_stride, (const __nv_bfloat16 *)kc, (const __nv_bfloat16 *)vc, seq_start, seq_past, page_table,
             pt_stride, n_heads, n_kv, window, scale * 1.4426950408889634f);
  LLM_CHECK_LAUNCH("attention_prefill");
  return LLM_OK;
}

// 1 if this head size and page size have an instantiation, else 0.
LLM_EXPORT int llm_attention_prefill_supports(int d, int page_size) {
  return page_size == AP_BN && d >= 16 && d <= 128 && d % 16 == 0;
}

// q [tokens, >= heads*d] bfloat16 (rotated), out [tokens, heads*d], caches
// [pages, kv_heads, 64, d]; sequence b owns rows seq_start[b]..seq_start[b+1]-1, which
// stand at positions seq_past[b].. of the sequence; max_q_len bounds the rows of a sequence.
LLM_EXPORT int llm_attention_prefill(const void *q, long long q_stride, void *out, long long out_stride,
                                     const void *kc, const void *vc, const int *seq_start, const int *seq_past,
                                     const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads,
                                     int n_kv, int d, int page_size, int window, float scale, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return LLM_OK;
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_heads > 0 && n_heads <= 65535 && n_kv > 0 && n_heads % n_kv == 0,
              "attention_prefill: bad sizes (%d sequences, %d heads, %d kv heads)", n_seqs, n_heads, n_kv);
  LLM_REQUIRE(llm_attention_prefill_supports(d, page_size),
              "attention_prefill: head size %d with pages of %d tokens is not built (multiples of 16 up to 128, pages of 64)",
              d, page_size);
  LLM_REQUIRE(q_stride % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)kc % 16 == 0 && (uintptr_t)vc % 16 == 0,
              "attention_prefill: rows must be 16-byte aligned");
  LLM_REQUIRE(out_stride % 2 == 0 && (uintptr_t)out % 4 == 0, "attention_prefill: output rows must be 4-byte aligned");
#define AP_CASE(DD)                                                                                                  \
  if (d == DD)                                                                                                       \
    return launch_prefill<DD>(q, q_stride, out, out_stride, kc, vc, seq_start, seq_past, page_table, pt_stride,      \
                              n_seqs, max_q_len, n_heads, n_kv, window, scale, stream);
  AP_CASE(16) AP_CASE(32) AP_CASE(48) AP_CASE(64) AP_CASE(80) AP_CASE(96) AP_CASE(112) AP_CASE(128)
#undef AP_CASE
  LLM_FAIL("attention_prefill: no kernel for head size %d", d);
}
