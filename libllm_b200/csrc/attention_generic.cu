// Causal grouped-query attention over the paged cache, any head size up to 256, any
// number of heads and groups, optional sliding window; element type float or bfloat16,
// arithmetic in 32-bit.  One warp serves one (token, head): lanes take 32 keys at a time
// for the scores, then 32 channels at a time for the weighted sum, with a running
// maximum and sum (the online form of softmax, src/flint/cpu/softmax.cc:31-60).
//
// This is the attention of the true 32-bit path and of head sizes the fast bfloat16
// kernels do not take.  It serves prompts and single tokens alike: the keys of the
// step's own tokens are already in the cache when it runs, and the token at position p
// reads keys 0..p (or the last `window` of them), which is the bottom-right aligned
// causal mask of the reference (src/flint/operators.cc:119-124).  Head h reads
// key/value head h / (heads / kv_heads) (src/flint/operators.cc:43-56); scores are
// scaled by 1/sqrt(d) (src/flint/operators.cc:115-117).
//
// A token's result depends only on its own sequence: the order of additions is fixed by
// the position, not by the batch.
#include "common.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_attention_generic_last_error)

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

__device__ __forceinline__ float dot_row(const float *q, const float *k, int d) {
  float acc = 0.f;
  for (int c = 0; c < d; c += 4) {
    const float4 v = *reinterpret_cast<const float4 *>(k + c);
    acc = fmaf(q[c], v.x, acc);
    acc = fmaf(q[c + 1], v.y, acc);
    acc = fmaf(q[c + 2], v.z, acc);
    acc = fmaf(q[c + 3], v.w, acc);
  }
  return acc;
}
__device__ __forceinline__ float dot_row(const float *q, const __nv_bfloat16 *k, int d) {
  float acc = 0.f;
  for (int c = 0; c < d; c += 8) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(k + c);
    const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      acc = fmaf(q[c + 2 * i], f.x, acc);
      acc = fmaf(q[c + 2 * i + 1], f.y, acc);
    }
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T *__restrict__ q, long long q_stride, T *__restrict__ out,
                         long long out_stride, const T *__restrict__ kcache,
                         const T *__restrict__ vcache, const int *__restrict__ tok_seq,
                         const int *__restrict__ tok_pos, const int *__restrict__ page_table,
                         int pt_stride, int n_tokens, int n_heads, int n_kv, int d, int page_size,
                         int window, float scale) {
  __shared__ __align__(16) float q_s[WARPS][MAX_D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long w = (long long)blockIdx.x * WARPS + warp;
  const int token = (int)(w / n_heads), h = (int)(w % n_heads);
  if (token >= n_tokens) return;
  const int p = tok_pos[token];
  const int *pt = page_table + (size_t)tok_seq[token] * pt_stride;
  const int kvh = h / (n_heads / n_kv);
  const T *qrow = q + (size_t)token * q_stride + (size_t)h * d;
  for (int c = lane; c < d; c += 32) q_s[warp][c] = to_float(qrow[c]);
  __syncwarp();

  const int kstart = window > 0 ? max(0, p - window + 1) : 0;
  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) acc[i] = 0.f;

  for (int kb = kstart; kb <= p; kb += 32) {
    const int j = kb + lane;
    const bool valid = j <= p;
    float s = -INFINITY;
    if (valid) {
      const int page = pt[j / page_size];
      const T *krow = kcache + (((size_t)page * n_kv + kvh) * page_size + (j % page_size)) * d;
      s = dot_row(q_s[warp], krow, d) * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));          // finite: lane 0 always holds a key
    const float pj = valid ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);                // 0 on the first block (m = -inf)
    l = l * alpha + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < MAX_D / 32; ++i) acc[i] *= alpha;
    const int nvalid = min(32, p - kb + 1);
    for (int jj = 0; jj < nvalid; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const int key = kb + jj;
      const int page = pt[key / page_size];
      const T *vrow = vcache + (((size_t)page * n_kv + kvh) * page_size + (key % page_size)) * d;
#pragma unroll
      for (int i = 0; i < MAX_D / 32; ++i) {
        const int c = lane + 32 * i;
        if (c < d) acc[i] = fmaf(pv, to_float(vrow[c]), acc[i]);
      }
    }
    m = m_new;
  }
  T *orow = out + (size_t)token * out_stride + (size_t)h * d;
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < MAX_D / 32; ++i) {
    const int c = lane + 32 * i;
    if (c < d) orow[c] = from_float<T>(acc[i] * inv);
  }
}

LLM_EXPORT int llm_attention_generic(int dtype, const void *q, long long q_stride, void *out,
                                     long long out_stride, const void *kcache, const void *vcache,
                                     const int *tok_seq, const int *tok_pos, const int *page_table,
                                     int pt_stride, int n_tokens, int n_heads, int n_kv, int d,
                                     int page_size, int window, float scale, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0, "attention: bad head counts %d/%d", n_heads, n_kv);
  LLM_REQUIRE(d > 0 && d <= MAX_D && d % 8 == 0, "attention: head size %d is not supported (a multiple of 8 up to %d)", d, MAX_D);
  LLM_REQUIRE(q_stride % 4 == 0, "attention: q rows must be 16-byte aligned");
  const long long warps = (long long)n_tokens * n_heads;
  const long long blocks = (warps + WARPS - 1) / WARPS;
  LLM_REQUIRE(blocks < 2147483647LL, "attention: too many tokens for one launch");
  if (dtype == LLM_F32) {
    LLM_REQUIRE(d % 4 == 0, "attention: head size");
    attention_generic_kernel<float><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
        (const float *)q, q_stride, (float *)out, out_stride, (const float *)kcache, (const float *)vcache,
        tok_seq, tok_pos, page_table, pt_stride, n_tokens, n_heads, n_kv, d, page_size, window, scale);
  } else if (dtype == LLM_BF16) {
    attention_generic_kernel<__nv_bfloat16><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
        (const __nv_bfloat16 *)q, q_stride, (__nv_bfloat16 *)out, out_stride, (const __nv_bfloat16 *)kcache,
        (const __nv_bfloat16 *)vcache, tok_seq, tok_pos, page_table, pt_stride, n_tokens, n_heads, n_kv, d,
        page_size, window, scale);
  } else {
    LLM_FAIL("attention: unknown dtype %d", dtype);
  }
  LLM_CHECK_LAUNCH("attention_generic");
  return LLM_OK;
}
