// Rotary position encoding of q and k and the append of k and v to the paged cache,
// in one pass over the stacked q|k|v rows of a step.
//
// The reference rotates with about fourteen elementwise launches per layer
// (src/libllm/llama.cc:151-176) and appends by re-allocating and copying the whole
// cache (src/libllm/llama.cc:203-212, src/flint/functional.cc:126-144).  The rotation
// pairs element i with i + d/2 (src/libllm/llama.cc:151-164):
//   out[i]       = x[i] * cos - x[i + d/2] * sin
//   out[i + d/2] = x[i + d/2] * cos + x[i] * sin
// cos and sin come from a 32-bit table [positions, d] (d/2 cosines, then d/2 sines) that
// is computed in 64-bit on the host side; the arithmetic here is 32-bit, rounded once.
//
// Cache layout per layer: [pages, kv_heads, page_size, d]; a token at position p of a
// sequence lies in page page_table[seq][p / page_size] at row p % page_size.
#include "common.cuh"

LLM_DEFINE_LAST_ERROR(llm_rope_last_error)

// TI: type of the stacked q|k|v rows (the product's output, 32-bit when the product can
// give that, so that q and k are rounded once, after the rotation); T: type of the
// rotated queries and of the cache.
template <typename TI, typename T>
__global__ void rope_cache_write_kernel(const TI *__restrict__ qkv, long long row_stride,
                                        T *__restrict__ q_out, long long q_stride, int n_heads,
                                        int n_kv, int d, const float *__restrict__ table,
                                        int table_rows, int rot_dim, const int *__restrict__ tok_seq,
                                        const int *__restrict__ tok_pos, const int *__restrict__ page_table,
                                        int pt_stride, T *__restrict__ kcache, T *__restrict__ vcache,
                                        int page_size) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int slot = blockIdx.y;                 // 0..n_heads-1: q, then k heads, then v heads
  const int pos = tok_pos[t];
  const TI *row = qkv + (size_t)t * row_stride + (size_t)slot * d;
  const int half = rot_dim / 2;
  const bool is_v = slot >= n_heads + n_kv;
  const bool is_k = !is_v && slot >= n_heads;
  T *dst;
  if (is_k || is_v) {
    const int kvh = is_k ? slot - n_heads : slot - n_heads - n_kv;
    const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
    T *base = is_k ? kcache : vcache;
    dst = base + (((size_t)page * n_kv + kvh) * page_size + (pos % page_size)) * d;
  } else {
    dst = q_out + (size_t)t * q_stride + (size_t)slot * d;
  }
  if (is_v) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = from_float<T>(to_float(row[i]));
    return;
  }
  const int p = pos < table_rows ? pos : table_rows - 1;   // the host refuses longer sequences
  const float *cs = table + (size_t)p * rot_dim;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float c = cs[i], s = cs[half + i];
    const float a = to_float(row[i]), b = to_float(row[i + half]);
    dst[i] = from_float<T>(a * c - b * s);
    dst[i + half] = from_float<T>(b * c + a * s);
  }
  // Channels beyond the rotated ones (rot_dim < d) pass through unchanged.
  for (int i = rot_dim + threadIdx.x; i < d; i += blockDim.x) dst[i] = from_float<T>(to_float(row[i]));
}

// The same with four channel pairs per thread and one CTA per token, for head sizes that are
// a multiple of 8 and rotate all of their channels: 16-byte loads, and the position and the
// page are looked up once per token.
template <typename TI, typename T>
__global__ void __launch_bounds__(256)
rope_cache_write_vec_kernel(const TI *__restrict__ qkv, long long row_stride, T *__restrict__ q_out,
                            long long q_stride, int n_heads, int n_kv, int d, const float *__restrict__ table,
                            int table_rows, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos,
                            const int *__restrict__ page_table, int pt_stride, T *__restrict__ kcache,
                            T *__restrict__ vcache, int page_size, int n_slots) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = d / 2, groups = half / 4;
  size_t cache_row = 0;
  if (n_slots > n_heads) {
    const int page = page_table[(size_t)tok_seq[t] * pt_stride + pos / page_size];
    cache_row = (size_t)page * n_kv * page_size + (pos % page_size);
  }
  const float *cs = table + (size_t)(pos < table_rows ? pos : table_rows - 1) * d;
  for (int item = threadIdx.x; item < n_slots * groups; item += blockDim.x) {
    const int slot = item / groups, j = (item % groups) * 4;
    const TI *row = qkv + (size_t)t * row_stride + (size_t)slot * d;
    const float4 a = ld4(row + j), b = ld4(row + j + half);
    const bool is_v = slot >= n_heads + n_kv;
    T *dst;
    if (slot < n_heads) {
      dst = q_out + (size_t)t * q_stride + (size_t)slot * d;
    } else {
      const int kvh = is_v ? slot - n_heads - n_kv : slot - n_heads;
      dst = (is_v ? vcache : kcache) + (cache_row + (size_t)kvh * page_size) * d;
    }
    if (is_v) {
      st4(dst + j, a);
      st4(dst + j + half, b);
    } else {
      const float4 c = ld4(cs + j), s = ld4(cs + half + j);
      st4(dst + j, make_float4(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y, a.z * c.z - b.z * s.z, a.w * c.w - b.w * s.w));
      st4(dst + j + half, make_float4(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y, b.z * c.z + a.z * s.z, b.w * c.w + a.w * s.w));
    }
  }
}

// in_dtype: type of qkv; dtype: type of q_out and of the cache.  With write_cache == 0
// only the query heads are processed (the layer reads another layer's keys and values).
LLM_EXPORT int llm_rope_cache_write(int in_dtype, int dtype, const void *qkv, long long row_stride,
                                    void *q_out, long long q_stride, int n_tokens, int n_heads,
                                    int n_kv, int d, const float *table, int table_rows, int rot_dim,
                                    const int *tok_seq, const int *tok_pos, const int *page_table,
                                    int pt_stride, void *kcache, void *vcache, int page_size,
                                    int write_cache, cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && n_heads > 0 && n_kv > 0 && d > 0, "rope: bad sizes");
  // rot_dim 0: nothing is rotated (a mixer without a position encoding); queries pass through and
  // keys and values are appended as they are
  LLM_REQUIRE(rot_dim % 2 == 0 && rot_dim <= d && rot_dim >= 0 && (rot_dim == 0 || table != nullptr),
              "rope: rotated width %d does not fit head size %d", rot_dim, d);
  LLM_REQUIRE(n_heads + 2 * n_kv <= 65535, "rope: too many heads for one launch");
  const int n_slots = write_cache ? n_heads + 2 * n_kv : n_heads;
  const bool vec = d % 8 == 0 && rot_dim == d && row_stride % 4 == 0 && q_stride % 4 == 0 &&
                   (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && (uintptr_t)table % 16 == 0 &&
                   (uintptr_t)kcache % 16 == 0 && (uintptr_t)vcache % 16 == 0;
  if (vec) {
    const int items = n_slots * (d / 8);
    const int vthreads = items >= 256 ? 256 : (items + 31) / 32 * 32;
#define ROPE_VEC(TI, T)                                                                                  \
  llm_launch(rope_cache_write_vec_kernel<TI, T>, dim3(n_tokens), dim3(vthreads), 0, stream, (const TI *)qkv, \
             row_stride, (T *)q_out, q_stride, n_heads, n_kv, d, table, table_rows, tok_seq, tok_pos,    \
             page_table, pt_stride, (T *)kcache, (T *)vcache, page_size, n_slots)
    if (in_dtype == LLM_F32 && dtype == LLM_F32) ROPE_VEC(float, float);
    else if (in_dtype == LLM_F32 && dtype == LLM_BF16) ROPE_VEC(float, __nv_bfloat16);
    else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) ROPE_VEC(__nv_bfloat16, __nv_bfloat16);
    else LLM_FAIL("rope: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef ROPE_VEC
    LLM_CHECK_LAUNCH("rope_cache_write");
    return LLM_OK;
  }
  dim3 grid(n_tokens, n_slots);
  int threads = d / 2 >= 64 ? 64 : 32;
#define ROPE_LAUNCH(TI, T)                                                                              \
  llm_launch(rope_cache_write_kernel<TI, T>, grid, dim3(threads), 0, stream,                           \
      (const TI *)qkv, row_stride, (T *)q_out, q_stride, n_heads, n_kv, d, table, table_rows, rot_dim,  \
      tok_seq, tok_pos, page_table, pt_stride, (T *)kcache, (T *)vcache, page_size)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) ROPE_LAUNCH(float, float);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) ROPE_LAUNCH(float, __nv_bfloat16);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) ROPE_LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else LLM_FAIL("rope: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef ROPE_LAUNCH
  LLM_CHECK_LAUNCH("rope_cache_write");
  return LLM_OK;
}
