// Embedding gather, residual-add + RMSNorm, and SwiGLU.  Element type T is float (the
// true 32-bit path) or bfloat16; all arithmetic is in 32-bit.
//
// Reference counterparts: lookup (src/flint/cuda/lookup.cu:30-43), rmsNorm
// (src/flint/cuda/rms_norm.cu:31-84) followed by a separate add
// (src/flint/cuda/binary.cu:48-88), swiglu (src/flint/cuda/swiglu.cu:29-59).  Here the
// residual stream is kept in 32-bit and the add is part of the norm kernel, so one
// pass over the row does what three launches do there.
#include "common.cuh"

LLM_DEFINE_LAST_ERROR(llm_elementwise_last_error)

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const T *__restrict__ table, const int *__restrict__ tokens,
                                 const int *__restrict__ fed_tokens, const int *__restrict__ fed_rows,
                                 float *__restrict__ out, int hidden, int vocab) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int t = blockIdx.x;
  // A token either comes with the step (tokens[t]) or is the one the previous step sampled for
  // row fed_rows[t] of its batch, still on the device (fed_tokens): the host can then start this
  // step before it has read that token back.
  int id = tokens[t];
  if (fed_rows != nullptr && fed_rows[t] >= 0) id = fed_tokens[fed_rows[t]];
  // Token ids are checked on the host before they are uploaded; ids that the sampler
  // wrote on the device are below the vocabulary size by construction.  The clamp keeps
  // the read inside the table whatever happens.
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T *row = table + (size_t)id * hidden;
  float *o = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_float(row[i]);
}

LLM_EXPORT int llm_embedding(int dtype, const void *table, const int *tokens, const int *fed_tokens,
                             const int *fed_rows, float *out, int n_tokens, int hidden, int vocab,
                             cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
  LLM_REQUIRE((fed_tokens == nullptr) == (fed_rows == nullptr), "embedding: fed tokens come with their rows");
  int threads = hidden >= 1024 ? 256 : 128;
  // A step's first kernel after its descriptor has arrived, and launched so that it starts only
  // when that is complete: the kernels after it read positions and page tables from the descriptor
  // before they wait for their own predecessors, which is safe because none of them can start before
  // this one has.  (Inside a single-token step's graph the descriptor comes by a kernel just before
  // this one; with an overlapping launch here, a later kernel could in rare runs read the positions
  // of the step before last.)
  if (dtype == LLM_F32)
    llm_launch_after(embedding_kernel<float>, n_tokens, threads, 0, stream, (const float *)table, tokens, fed_tokens, fed_rows, out, hidden, vocab);
  else if (dtype == LLM_BF16)
    llm_launch_after(embedding_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream, (const __nv_bfloat16 *)table, tokens, fed_tokens, fed_rows, out, hidden, vocab);
  else
    LLM_FAIL("embedding: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("embedding");
  return LLM_OK;
}

// ---------------------------------------------------------------- small copies as kernels
// n 32-bit words from src to dst, either of which may be pinned host memory (which the device
// reaches by the same address).  A step's descriptor comes in and its tokens go out this way inside
// the step's graph: a copy of the copy engine there costs 8 to 15 us of hand-over on either side,
// a kernel two or three.
// The kernels behind it may start only when the words are written: later kernels of a step read
// the descriptor before they wait for their predecessors.
__global__ void copy_words_kernel(const int *__restrict__ src, int *__restrict__ dst, int n) {
  grid_dependency_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = src[i];
  __threadfence();
  grid_dependents_launch();
}

LLM_EXPORT int llm_copy_words(const int *src, int *dst, int n, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && src != nullptr && dst != nullptr, "copy_words: bad arguments");
  const int blocks = n <= 1024 ? 1 : (n + 1023) / 1024 > 64 ? 64 : (n + 1023) / 1024;
  llm_launch(copy_words_kernel, blocks, n < 256 ? 64 : 256, 0, stream, src, dst, n);
  LLM_CHECK_LAUNCH("copy_words");
  return LLM_OK;
}

// n1 words from src1 followed by n2 words from src2, to dst (which may be pinned host memory): a
// step's sampled tokens and the status word of its tensor-core kernels leave the device together.
__global__ void gather_words_kernel(const int *__restrict__ src1, int n1, const int *__restrict__ src2, int n2,
                                    int *__restrict__ dst) {
  grid_dependency_wait();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n1 + n2; i += gridDim.x * blockDim.x)
    dst[i] = i < n1 ? src1[i] : src2[i - n1];
  __threadfence_system();
  grid_dependents_launch();
}

LLM_EXPORT int llm_gather_words(const int *src1, int n1, const int *src2, int n2, int *dst, cudaStream_t stream) {
  if (n1 + n2 == 0) return LLM_OK;
  LLM_REQUIRE(n1 >= 0 && n2 >= 0 && dst != nullptr && (n1 == 0 || src1) && (n2 == 0 || src2), "gather_words: bad arguments");
  const int n = n1 + n2;
  const int blocks = n <= 1024 ? 1 : (n + 1023) / 1024 > 64 ? 64 : (n + 1023) / 1024;
  llm_launch(gather_words_kernel, blocks, n < 256 ? 64 : 256, 0, stream, src1, n1, src2, n2, dst);
  LLM_CHECK_LAUNCH("gather_words");
  return LLM_OK;
}

// ---------------------------------------------------------------- add + rmsnorm
// For each output row i (source row r = rows ? rows[i] : i):
//   v = resid[r] + sum_p delta[p][r]      (32-bit; parts added in index order)
//   if (!rows) resid[r] = v               (the residual stream moves on)
//   out[i] = v * w * rsqrt(mean(v^2) + eps)   (skipped when out is null)
template <typename TD, typename TO, int THREADS>
__global__ void add_rmsnorm_kernel(float *__restrict__ resid, const TD *__restrict__ delta,
                                   int n_parts, size_t part_stride, const float *__restrict__ weight,
                                   float eps, TO *__restrict__ out, const int *__restrict__ rows,
                                   int hidden) {
  extern __shared__ float row_buf[];   // hidden floats
  __shared__ float scratch[THREADS / 32 + 1];
  grid_dependents_launch();
  grid_dependency_wait();
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float *x = resid + (size_t)r * hidden;
  float ss = 0.f;
  for (int c = threadIdx.x; c < hidden; c += THREADS) {
    float v = x[c];
    for (int p = 0; p < n_parts; ++p) v += to_float(delta[p * part_stride + (size_t)r * hidden + c]);
    row_buf[c] = v;
    if (!rows && n_parts > 0) x[c] = v;
    ss += v * v;
  }
  if (!out) return;
  const float total = block_sum<THREADS>(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  TO *o = out + (size_t)i * hidden;
  for (int c = threadIdx.x; c < hidden; c += THREADS) o[c] = from_float<TO>(row_buf[c] * weight[c] * inv);
}

// The same for rows whose width is a multiple of 4 and at most 4 * VPT * THREADS, with up
// to MAXP parts: every thread issues all its loads (the row, every part, the weight) before
// it uses one, so the kernel waits for memory once and not once per part.  The values,
// the order of the additions and the order of the sum of squares within a thread differ
// from the general kernel's only in which thread owns which columns; like it, a row's
// result does not depend on the other rows of the launch.
template <typename TD, typename TO, int THREADS, int VPT, int MAXP>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_vec_kernel(float *__restrict__ resid, const TD *__restrict__ delta, int n_parts,
                       size_t part_stride, const float *__restrict__ weight, float eps,
                       TO *__restrict__ out, const int *__restrict__ rows, int hidden) {
  __shared__ float scratch[THREADS / 32 + 1];
  grid_dependents_launch();
  const int i = blockIdx.x;
  const int n4 = hidden / 4;
  float4 v[VPT], w[VPT], d[VPT][MAXP];
  if (out) {                             // the norm's weight does not depend on the kernel before
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int c4 = threadIdx.x + j * THREADS;
      if (c4 < n4) w[j] = ld4(weight + 4 * c4);
    }
  }
  grid_dependency_wait();
  const int r = rows ? rows[i] : i;
  float *x = resid + (size_t)r * hidden;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
      v[j] = ld4(x + 4 * c4);
#pragma unroll
      for (int p = 0; p < MAXP; ++p)
        if (p < n_parts) d[j][p] = ld4(delta + p * part_stride + (size_t)r * hidden + 4 * c4);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4) {
#pragma unroll
      for (int p = 0; p < MAXP; ++p)
        if (p < n_parts) {
          v[j].x += d[j][p].x;
          v[j].y += d[j][p].y;
          v[j].z += d[j][p].z;
          v[j].w += d[j][p].w;
        }
      if (!rows && n_parts > 0) st4(x + 4 * c4, v[j]);
      ss += v[j].x * v[j].x;
      ss += v[j].y * v[j].y;
      ss += v[j].z * v[j].z;
      ss += v[j].w * v[j].w;
    }
  }
  if (!out) return;
  const float total = block_sum<THREADS>(ss, scratch);
  const float inv = rsqrtf(total / (float)hidden + eps);
  TO *o = out + (size_t)i * hidden;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c4 = threadIdx.x + j * THREADS;
    if (c4 < n4)
      st4(o + 4 * c4, make_float4(v[j].x * w[j].x * inv, v[j].y * w[j].y * inv, v[j].z * w[j].z * inv,
                                  v[j].w * w[j].w * inv));
  }
}

template <typename TD, typename TO>
static int launch_add_rmsnorm(float *resid, const void *delta, int n_parts, size_t part_stride,
                              const float *weight, float eps, void *out, const int *rows, int n_rows,
                              int hidden, cudaStream_t stream) {
  constexpr int THREADS = 256;
  constexpr int VPT = 4;
  const bool aligned = hidden % 4 == 0 && (uintptr_t)resid % 16 == 0 && (uintptr_t)delta % 16 == 0 &&
                       (uintptr_t)weight % 16 == 0 && (uintptr_t)out % 16 == 0 && part_stride % 4 == 0;
  if (aligned && hidden <= 4 * VPT * THREADS && n_parts <= 8) {
    // one instantiation per bound on the parts: registers for eight parts cost a prompt step
    // (one part, thousands of rows) a third of its speed
    // A thread per four columns where the row allows it (up to 4,096 columns): with many parts the
    // loads of a row are in flight from more warps at once.
#define ADDNORM_GO2(T_, V_, MAXP)                                                                        \
  llm_launch(add_rmsnorm_vec_kernel<TD, TO, T_, V_, MAXP>, n_rows, T_, 0, stream, resid,                 \
             (const TD *)delta, n_parts, part_stride, weight, eps, (TO *)out, rows, hidden)
#define ADDNORM_GO(MAXP)                                                                                 \
  do {                                                                                                   \
    if (hidden <= 2048) ADDNORM_GO2(512, 1, MAXP);                                                       \
    else if (hidden <= 4096) ADDNORM_GO2(1024, 1, MAXP);                                                 \
    else ADDNORM_GO2(THREADS, VPT, MAXP);                                                                \
  } while (0)
    if (n_parts <= 1) ADDNORM_GO(1);
    else if (n_parts <= 4) ADDNORM_GO(4);
    else ADDNORM_GO(8);
#undef ADDNORM_GO
#undef ADDNORM_GO2
    LLM_CHECK_LAUNCH("add_rmsnorm");
    return LLM_OK;
  }
  size_t smem = (size_t)hidden * sizeof(float);
  auto kern = add_rmsnorm_kernel<TD, TO, THREADS>;
  if (smem > 48 * 1024) {
    LLM_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: a row of %d values does not fit shared memory", hidden);
    LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "add_rmsnorm attribute");
  }
  llm_launch(kern, n_rows, THREADS, smem, stream, resid, (const TD *)delta, n_parts, part_stride, weight, eps,
             (TO *)out, rows, hidden);
  LLM_CHECK_LAUNCH("add_rmsnorm");
  return LLM_OK;
}

// delta_dtype: type of delta; out_dtype: type of out.  delta may be null (n_parts 0),
// out may be null (add only), rows may be null (all rows, residual written back).
LLM_EXPORT int llm_add_rmsnorm(float *resid, const void *delta, int delta_dtype, int n_parts,
                               long long part_stride, const float *weight, float eps, void *out,
                               int out_dtype, const int *rows, int n_rows, int hidden,
                               cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 0, "add_rmsnorm: bad sizes");
  LLM_REQUIRE(out == nullptr || weight != nullptr, "add_rmsnorm: a norm needs its weight");
  if (!delta) n_parts = 0;
  if (delta_dtype == LLM_F32 && out_dtype == LLM_F32)
    return launch_add_rmsnorm<float, float>(resid, delta, n_parts, part_stride, weight, eps, out, rows, n_rows, hidden, stream);
  if (delta_dtype == LLM_F32 && out_dtype == LLM_BF16)
    return launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, n_parts, part_stride, weight, eps, out, rows, n_rows, hidden, stream);
  if (delta_dtype == LLM_BF16 && out_dtype == LLM_BF16)
    return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, n_parts, part_stride, weight, eps, out, rows, n_rows, hidden, stream);
  if (delta_dtype == LLM_BF16 && out_dtype == LLM_F32)
    return launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, n_parts, part_stride, weight, eps, out, rows, n_rows, hidden, stream);
  LLM_FAIL("add_rmsnorm: unknown dtypes %d, %d", delta_dtype, out_dtype);
}

// ---------------------------------------------------------------- rows of the stream picked out
// out[i] = resid[rows[i]] + sum_p delta[p][rows[i]] (32-bit, parts in index order): the residual
// stream of the rows that anything still reads, when the others are done with.
template <typename TD>
__global__ void gather_rows_add_kernel(const float *__restrict__ resid, const TD *__restrict__ delta, int n_parts,
                                       size_t part_stride, const int *__restrict__ rows, float *__restrict__ out, int hidden) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int i = blockIdx.x;
  const size_t r = (size_t)rows[i];
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = resid[r * hidden + c];
    for (int p = 0; p < n_parts; ++p) v += to_float(delta[p * part_stride + r * hidden + c]);
    out[(size_t)i * hidden + c] = v;
  }
}

LLM_EXPORT int llm_gather_rows_add(const float *resid, const void *delta, int delta_dtype, int n_parts, long long part_stride,
                                   const int *rows, int n_rows, float *out, int hidden, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && hidden > 0 && n_parts >= 0 && rows != nullptr && out != nullptr, "gather_rows_add: bad arguments");
  if (!delta) n_parts = 0;
  if (delta_dtype == LLM_BF16 && n_parts > 0)
    LLM_CHECK_CUDA(llm_launch(gather_rows_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(256), 0, stream, resid, (const __nv_bfloat16 *)delta,
                              n_parts, (size_t)part_stride, rows, out, hidden), "gather_rows_add launch");
  else
    LLM_CHECK_CUDA(llm_launch(gather_rows_add_kernel<float>, dim3(n_rows), dim3(256), 0, stream, resid, (const float *)delta, n_parts,
                              (size_t)part_stride, rows, out, hidden), "gather_rows_add launch");
  return LLM_OK;
}

// ---------------------------------------------------------------- swiglu
// out[t, i] = silu(gu[t, i]) * gu[t, inter + i], silu(a) = a / (1 + exp(-a)).  TI is the
// type of the stacked gate|up product (32-bit when the product gives that), T of out.
template <typename TI, typename T>
__global__ void swiglu_kernel(const TI *__restrict__ gu, T *__restrict__ out, int inter, size_t total) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter;
    const int i = (int)(idx - t * inter);
    const float g = to_float(gu[t * 2 * inter + i]);
    const float u = to_float(gu[t * 2 * inter + inter + i]);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

// Four values per thread (widths that are a multiple of 4, 16-byte aligned rows).
template <typename TI, typename T>
__global__ void swiglu_vec_kernel(const TI *__restrict__ gu, T *__restrict__ out, int inter4, size_t total4) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / inter4;
    const int i = (int)(idx - t * inter4) * 4;
    const TI *row = gu + t * 8 * (size_t)inter4;
    const float4 g = ld4(row + i), u = ld4(row + 4 * (size_t)inter4 + i);
    st4(out + idx * 4, make_float4(g.x / (1.f + expf(-g.x)) * u.x, g.y / (1.f + expf(-g.y)) * u.y,
                                   g.z / (1.f + expf(-g.z)) * u.z, g.w / (1.f + expf(-g.w)) * u.w));
  }
}

LLM_EXPORT int llm_swiglu(int in_dtype, int dtype, const void *gu, void *out, int n_tokens, int inter,
                          cudaStream_t stream) {
  if (n_tokens == 0) return LLM_OK;
  LLM_REQUIRE(n_tokens > 0 && inter > 0, "swiglu: bad sizes");
  const int threads = 256;
  const bool vec = inter % 4 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0;
  const size_t total = vec ? (size_t)n_tokens * (inter / 4) : (size_t)n_tokens * inter;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
#define SWIGLU_GO(TI, T)                                                                                     \
  do {                                                                                                       \
    if (vec)                                                                                                 \
      llm_launch(swiglu_vec_kernel<TI, T>, (unsigned)blocks, threads, 0, stream, (const TI *)gu, (T *)out, inter / 4, total); \
    else                                                                                                     \
      llm_launch(swiglu_kernel<TI, T>, (unsigned)blocks, threads, 0, stream, (const TI *)gu, (T *)out, inter, total); \
  } while (0)
  if (in_dtype == LLM_F32 && dtype == LLM_F32) SWIGLU_GO(float, float);
  else if (in_dtype == LLM_F32 && dtype == LLM_BF16) SWIGLU_GO(float, __nv_bfloat16);
  else if (in_dtype == LLM_BF16 && dtype == LLM_BF16) SWIGLU_GO(__nv_bfloat16, __nv_bfloat16);
  else LLM_FAIL("swiglu: unsupported dtypes in %d out %d", in_dtype, dtype);
#undef SWIGLU_GO
  LLM_CHECK_LAUNCH("swiglu");
  return LLM_OK;
}

// ---------------------------------------------------------------- scaling of rows and logits
// x *= scale over n values: the token rows of an architecture that scales its embedding.
__global__ void scale_rows_kernel(float *__restrict__ x, long long n, float scale) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] *= scale;
}

LLM_EXPORT int llm_scale_rows(float *x, long long n, float scale, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && x != nullptr, "scale_rows: bad arguments");
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
  llm_launch(scale_rows_kernel, (unsigned)blocks, 256, 0, stream, x, n, scale);
  LLM_CHECK_LAUNCH("scale_rows");
  return LLM_OK;
}

// logit = logit * scale, then, with a positive cap, cap * tanh(logit / cap), in 32-bit.
__global__ void logit_transform_kernel(float *__restrict__ x, long long n, float scale, float cap) {
  grid_dependents_launch();
  grid_dependency_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float v = x[i] * scale;
    if (cap > 0.f) v = cap * tanhf(v / cap);
    x[i] = v;
  }
}

LLM_EXPORT int llm_logit_transform(float *x, long long n, float scale, float cap, cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && x != nullptr, "logit_transform: bad arguments");
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)sm_count() * 16) blocks = (long long)sm_count() * 16;
  llm_launch(logit_transform_kernel, (unsigned)blocks, 256, 0, stream, x, n, scale, cap);
  LLM_CHECK_LAUNCH("logit_transform");
  return LLM_OK;
}

// ---------------------------------------------------------------- random weights on the device
// Element i is a pure function of (seed, i): two SplitMix64 outputs give two uniform numbers;
// law 0 turns them into a normal number with mean a and deviation b (Box-Muller), law 1 into a
// uniform number in [a, b).  The random-weights mode of a benchmark fills its tensors here
// instead of drawing a billion numbers on the host.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T>
__global__ void random_fill_kernel(T *__restrict__ out, long long n, unsigned long long seed, int law, float a, float b) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const unsigned long long h1 = splitmix64(seed ^ splitmix64((unsigned long long)i));
    const unsigned long long h2 = splitmix64(h1);
    const float u1 = ((float)(h1 >> 40) + 1.0f) * (1.0f / 16777216.0f);      // (0, 1]
    const float u2 = (float)(h2 >> 40) * (1.0f / 16777216.0f);               // [0, 1)
    float v;
    if (law == 0) v = a + b * sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
    else v = a + (b - a) * u2;
    out[i] = from_float<T>(v);
  }
}

LLM_EXPORT int llm_random_fill(void *out, int dtype, long long n, unsigned long long seed, int law, float a, float b,
                               cudaStream_t stream) {
  if (n == 0) return LLM_OK;
  LLM_REQUIRE(n > 0 && out != nullptr && (law == 0 || law == 1), "random_fill: bad arguments");
  long long blocks = (n + 255) / 256;
  if (blocks > (long long)sm_count() * 32) blocks = (long long)sm_count() * 32;
  if (dtype == LLM_F32) random_fill_kernel<float><<<(unsigned)blocks, 256, 0, stream>>>((float *)out, n, seed, law, a, b);
  else if (dtype == LLM_BF16) random_fill_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, stream>>>((__nv_bfloat16 *)out, n, seed, law, a, b);
  else LLM_FAIL("random_fill: unknown dtype %d", dtype);
  LLM_CHECK_LAUNCH("random_fill");
  return LLM_OK;
}
