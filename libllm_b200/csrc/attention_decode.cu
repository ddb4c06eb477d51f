// Attention for decoding steps: every sequence brings one query token, keys and values
// come from the paged bfloat16 cache.  Split over the keys (flash-decoding): CTA
// (split, kv head, sequence) reduces `chunk` keys for all query heads of its group with a
// running maximum and sum, then a second kernel joins the splits in split order.
//
// The kernel is bound by reading K and V once (4 flop per byte with 4 query heads per kv
// head), so it is written for loads: D/8 lanes share a key, each lane fetching 16 bytes of
// K and of V for its 8 channels, four keys per lane group in flight, consecutive lane
// groups on consecutive keys so that a CTA reads 2 KB runs of a page.  Scores, softmax and
// the weighted sum are 32-bit; exp is taken as exp2 of pre-scaled scores.
//
// Reference counterpart: FlashAttention-2's split-KV forward and its combine kernel as the
// reference calls them for one query token (src/flint/cuda/flash_attn.cc:165-180); head h
// reads kv head h / (heads / kv_heads), scores are scaled by 1/sqrt(d), and one query sees
// every cached key (src/flint/operators.cc:43-56, 115-124).
#include "common.cuh"
#include "attention_decode.h"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_attention_decode_last_error)

constexpr int AD_THREADS = 128;
constexpr int AD_KB = 4;              // keys per lane group per iteration

__device__ __forceinline__ void unpack8(const uint4 &raw, float (&f)[8]) {
  const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

template <int D, int G>
__global__ void __launch_bounds__(AD_THREADS)
attention_decode_kernel(const __nv_bfloat16 *__restrict__ q, long long q_stride,
                        const __nv_bfloat16 *__restrict__ kc, const __nv_bfloat16 *__restrict__ vc,
                        const int *__restrict__ tok_pos, const int *__restrict__ page_table, int pt_stride,
                        int n_kv, int page_size, int chunk, int window, float scale_log2,
                        float *__restrict__ ws_o, float *__restrict__ ws_ml, int n_splits,
                        __nv_bfloat16 *__restrict__ out, long long out_stride) {
  constexpr int LPK = D / 8;                 // lanes per key
  constexpr int GPW = 32 / LPK;              // lane groups per warp
  constexpr int GROUPS = (AD_THREADS / 32) * GPW;
  __shared__ float sm_o[AD_THREADS / 32][G][D];
  __shared__ float sm_m[AD_THREADS / 32][G], sm_l[AD_THREADS / 32][G];

  // Positions and page tables come from the step's descriptor, which is copied to the device
  // before the step's first kernel starts.  So this CTA looks up its pages before the wait;
  // the queries and the newest token's key and value (written by the rotation kernel) are
  // read after it.
  grid_dependents_launch();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int len = tok_pos[b] + 1;
  const int kstart = window > 0 ? max(0, len - window) : 0;
  const int c0 = split * chunk;
  const int c1 = min(c0 + chunk, len);
  if (c0 >= len || c1 <= kstart) {
    grid_dependency_wait();
    return;
  }

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPK, grp = warp * GPW + lane / LPK;
  const int n_heads = n_kv * G;

  // The chunk's page numbers, once, so that no load address waits on another load.
  extern __shared__ int s_pages[];
  {
    const int *pt = page_table + (size_t)b * pt_stride + c0 / page_size;
    const int n_pg = (c1 - c0 + page_size - 1) / page_size;
    for (int i = threadIdx.x; i < n_pg; i += AD_THREADS) s_pages[i] = pt[i];
  }
  grid_dependency_wait();
  __syncthreads();

  float qr[G][8];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(q + (size_t)b * q_stride + (size_t)(kvh * G + h) * D + sub * 8);
    unpack8(raw, qr[h]);
#pragma unroll
    for (int c = 0; c < 8; ++c) qr[h][c] *= scale_log2;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[h][c] = 0.f;
  }

  constexpr int STEP = GROUPS * AD_KB;
  auto load = [&](int base, uint4 (&kr)[AD_KB], uint4 (&vr)[AD_KB]) {
#pragma unroll
    for (int u = 0; u < AD_KB; ++u) {
      const int key = base + u * GROUPS + grp;
      // A key that exists and lies inside the window (its weight is zero): pages before
      // the window may have been given back, and their table entries are not page numbers.
      int kk = key < c1 ? key : c1 - 1;
      kk = kk < kstart ? kstart : kk;
      const int page = s_pages[(kk - c0) / page_size];
      const size_t off = (((size_t)page * n_kv + kvh) * page_size + (kk % page_size)) * D + sub * 8;
      kr[u] = *reinterpret_cast<const uint4 *>(kc + off);
      vr[u] = *reinterpret_cast<const uint4 *>(vc + off);
    }
  };
  auto consume = [&](int base, const uint4 (&kraw)[AD_KB], const uint4 (&vraw)[AD_KB]) {
    bool ok[AD_KB];
#pragma unroll
    for (int u = 0; u < AD_KB; ++u) {
      const int key = base + u * GROUPS + grp;
      ok[u] = key < c1 && key >= kstart;
    }
    float s[AD_KB][G];
#pragma unroll
    for (int u = 0; u < AD_KB; ++u) {
      float kf[8];
      unpack8(kraw[u], kf);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float d = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) d = fmaf(qr[h][c], kf[c], d);
        s[u][h] = d;
      }
    }
#pragma unroll
    for (int o = 1; o < LPK; o <<= 1)
#pragma unroll
      for (int u = 0; u < AD_KB; ++u)
#pragma unroll
        for (int h = 0; h < G; ++h) s[u][h] += __shfl_xor_sync(0xffffffffu, s[u][h], o);
    float vf[AD_KB][8];
#pragma unroll
    for (int u = 0; u < AD_KB; ++u) unpack8(vraw[u], vf[u]);
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float mx = -INFINITY;
#pragma unroll
      for (int u = 0; u < AD_KB; ++u) mx = fmaxf(mx, ok[u] ? s[u][h] : -INFINITY);
      const float m_new = fmaxf(m[h], mx);
      if (m_new == -INFINITY) continue;                       // this group has seen no key yet
      const float alpha = exp2f(m[h] - m_new);                // 0 when m was -inf
      l[h] *= alpha;
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[h][c] *= alpha;
#pragma unroll
      for (int u = 0; u < AD_KB; ++u) {
        const float p = ok[u] ? exp2f(s[u][h] - m_new) : 0.f;
        l[h] += p;
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[h][c] = fmaf(p, vf[u][c], acc[h][c]);
      }
      m[h] = m_new;
    }
  };

  // Two register buffers: the loads of the next round are issued before this round's math.
  uint4 ka[AD_KB], va[AD_KB], kb[AD_KB], vb[AD_KB];
  load(c0, ka, va);
  for (int base = c0; base < c1; base += 2 * STEP) {
    const bool more = base + STEP < c1;
    if (more) load(base + STEP, kb, vb);
    consume(base, ka, va);
    if (!more) break;
    if (base + 2 * STEP < c1) load(base + 2 * STEP, ka, va);
    consume(base + STEP, kb, vb);
  }

  // Join the lane groups of a warp (fixed order: partner at distance LPK, 2 LPK, ...).
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[h], o);
      const float lo = __shfl_xor_sync(0xffffffffu, l[h], o);
      const float m_new = fmaxf(m[h], mo);
      const float sa = m[h] == -INFINITY ? 0.f : exp2f(m[h] - m_new);
      const float sb = mo == -INFINITY ? 0.f : exp2f(mo - m_new);
      l[h] = l[h] * sa + lo * sb;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[h][c], o);
        acc[h][c] = acc[h][c] * sa + ao * sb;
      }
      m[h] = m_new;
    }
  }
  if (lane < LPK) {
#pragma unroll
    for (int h = 0; h < G; ++h) {
#pragma unroll
      for (int c = 0; c < 8; ++c) sm_o[warp][h][sub * 8 + c] = acc[h][c];
      if (sub == 0) {
        sm_m[warp][h] = m[h];
        sm_l[warp][h] = l[h];
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += AD_THREADS) {
    const int h = idx / D, c = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < AD_THREADS / 32; ++w) M = fmaxf(M, sm_m[w][h]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < AD_THREADS / 32; ++w) {
      const float f = sm_m[w][h] == -INFINITY ? 0.f : exp2f(sm_m[w][h] - M);
      L += sm_l[w][h] * f;
      O += sm_o[w][h][c] * f;
    }
    const int head = kvh * G + h;
    if (n_splits == 1) {
      out[(size_t)b * out_stride + (size_t)head * D + c] = __float2bfloat16_rn(O / L);
    } else {
      const size_t slot = ((size_t)b * n_heads + head) * n_splits + split;
      ws_o[slot * D + c] = O;
      if (c == 0) {
        ws_ml[slot * 2] = M;
        ws_ml[slot * 2 + 1] = L;
      }
    }
  }
}

// Joins the splits of one (sequence, head): out = sum_s o_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
__global__ void attention_decode_combine_kernel(const float *__restrict__ ws_o, const float *__restrict__ ws_ml,
                                                const int *__restrict__ tok_pos, int n_heads, int D, int chunk,
                                                int window, int n_splits, __nv_bfloat16 *__restrict__ out,
                                                long long out_stride) {
  grid_dependents_launch();
  grid_dependency_wait();
  const int head = blockIdx.x, b = blockIdx.y;
  const int len = tok_pos[b] + 1;
  const int kstart = window > 0 ? max(0, len - window) : 0;
  // Splits beyond n_splits do not exist (the caller's n_splits * chunk should cover the longest
  // sequence; keys beyond it were not attended to): never read another head's scratch.
  const int first = min(kstart / chunk, n_splits - 1), last = min((len - 1) / chunk, n_splits - 1);
  const size_t slot0 = ((size_t)b * n_heads + head) * n_splits;
  float M = -INFINITY;
  for (int s = first; s <= last; ++s) M = fmaxf(M, ws_ml[(slot0 + s) * 2]);
  float L = 0.f;
  for (int s = first; s <= last; ++s) L += ws_ml[(slot0 + s) * 2 + 1] * exp2f(ws_ml[(slot0 + s) * 2] - M);
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float O = 0.f;
    for (int s = first; s <= last; ++s) O += ws_o[(slot0 + s) * D + c] * exp2f(ws_ml[(slot0 + s) * 2] - M);
    out[(size_t)b * out_stride + (size_t)head * D + c] = __float2bfloat16_rn(O / L);
  }
}

template <int D, int G>
static int launch_decode(const void *q, long long q_stride, const void *kc, const void *vc, const int *tok_pos,
                         const int *page_table, int pt_stride, int n_seqs, int n_kv, int page_size, int chunk,
                         int n_splits, int window, float scale, float *ws_o, float *ws_ml, void *out,
                         long long out_stride, cudaStream_t stream) {
  dim3 grid(n_splits, n_kv, n_seqs);
  const size_t smem = (size_t)((chunk + page_size - 1) / page_size) * sizeof(int);
  LLM_REQUIRE(smem <= 16 * 1024, "attention_decode: a chunk of %d keys spans too many pages", chunk);
  llm_launch(attention_decode_kernel<D, G>, grid, dim3(AD_THREADS), smem, stream,
      (const __nv_bfloat16 *)q, q_stride, (const __nv_bfloat16 *)kc, (const __nv_bfloat16 *)vc, tok_pos, page_table,
      pt_stride, n_kv, page_size, chunk, window, scale * 1.4426950408889634f, ws_o, ws_ml, n_splits,
      (__nv_bfloat16 *)out, out_stride);
  LLM_CHECK_LAUNCH("attention_decode");
  if (n_splits > 1) {
    dim3 cgrid(n_kv * G, n_seqs);
    llm_launch(attention_decode_combine_kernel, cgrid, dim3(D < 64 ? 32 : 64), 0, stream, (const float *)ws_o,
               (const float *)ws_ml, tok_pos, n_kv * G, D, chunk, window, n_splits, (__nv_bfloat16 *)out, out_stride);
    LLM_CHECK_LAUNCH("attention_decode_combine");
  }
  return LLM_OK;
}

// 1 if the (head size, group size) pair has an instantiation, else 0.
LLM_EXPORT int llm_attention_decode_supports(int d, int group) {
  const bool d_ok = d == 16 || d == 32 || d == 64 || d == 128;
  const bool g_ok = group == 1 || group == 2 || group == 3 || group == 4 || group == 8;
  return d_ok && g_ok;
}

// q [B, heads*d] bfloat16 (rotated), caches [pages, kv_heads, page_size, d], tok_pos[b] =
// position of sequence b's query (it sees keys 0..tok_pos[b]).  ws_o needs
// B*heads*n_splits*d floats and ws_ml B*heads*n_splits*2 when n_splits > 1.
LLM_EXPORT int llm_attention_decode(const void *q, long long q_stride, void *out, long long out_stride,
                                    const void *kc, const void *vc, const int *tok_pos, const int *page_table,
                                    int pt_stride, int n_seqs, int n_heads, int n_kv, int d, int page_size,
                                    int chunk, int n_splits, int window, float scale, float *ws_o, float *ws_ml,
                                    cudaStream_t stream) {
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_kv > 0 && n_kv <= 65535 && n_heads % n_kv == 0, "attention_decode: bad sizes");
  const int group = n_heads / n_kv;
  LLM_REQUIRE(llm_attention_decode_supports(d, group), "attention_decode: head size %d with %d query heads per kv head is not built", d, group);
  LLM_REQUIRE(chunk > 0 && chunk % page_size == 0 && n_splits >= 1, "attention_decode: chunk %d must be a positive multiple of the page size", chunk);
  LLM_REQUIRE(n_splits == 1 || (ws_o && ws_ml), "attention_decode: splits need scratch memory");
  LLM_REQUIRE(q_stride % 8 == 0 && (uintptr_t)q % 16 == 0, "attention_decode: q rows must be 16-byte aligned");
#define AD_CASE(DD, GG)                                                                                         \
  if (d == DD && group == GG)                                                                                   \
    return launch_decode<DD, GG>(q, q_stride, kc, vc, tok_pos, page_table, pt_stride, n_seqs, n_kv, page_size, \
                                 chunk, n_splits, window, scale, ws_o, ws_ml, out, out_stride, stream);
#define AD_CASES(DD) AD_CASE(DD, 1) AD_CASE(DD, 2) AD_CASE(DD, 3) AD_CASE(DD, 4) AD_CASE(DD, 8)
  AD_CASES(16) AD_CASES(32) AD_CASES(64) AD_CASES(128)
#undef AD_CASES
#undef AD_CASE
  LLM_FAIL("attention_decode: no kernel for head size %d, group %d", d, group);
}


// ---------------------------------------------------------------- the entry point that allocates nothing
// Scratch of llm_attention_decode_static: the splits' unnormalised outputs, then their maxima and
// sums.  It is part of the library's image on every GPU that loads it, until the process ends.
static __device__ __align__(256) float g_decode_scratch[LLM_ATTENTION_DECODE_STATIC_FLOATS];

// Device address of the scratch, looked up once per device.  In host code the array's name is
// only a stand-in: the address a kernel may use comes from cudaGetSymbolAddress, asked with that
// device current.
static int static_scratch(float **out) {
  constexpr int MAX_DEVICES = 64;
  static float *ptrs[MAX_DEVICES] = {};
  int dev = -1;
  LLM_CHECK_CUDA(cudaGetDevice(&dev), "attention_decode_static: cudaGetDevice");
  LLM_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "attention_decode_static: device %d is beyond the %d this entry point keeps track of", dev, MAX_DEVICES);
  if (!ptrs[dev]) {
    float *p = nullptr;
    LLM_CHECK_CUDA(cudaGetSymbolAddress((void **)&p, g_decode_scratch), "attention_decode_static: cudaGetSymbolAddress");
    LLM_REQUIRE(p != nullptr, "attention_decode_static: no device address for the scratch array");
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return LLM_OK;
}

LLM_EXPORT long long llm_attention_decode_static_floats_needed(int n_seqs, int n_heads, int d, int n_splits) {
  return n_splits <= 1 ? 0 : (long long)n_seqs * n_heads * n_splits * (d + 2);
}

LLM_EXPORT int llm_attention_decode_static(const void *q, long long q_stride, void *out, long long out_stride,
                                           const void *kc, const void *vc, const int *tok_pos, const int *page_table,
                                           int pt_stride, int n_seqs, int n_heads, int n_kv, int d, int page_size,
                                           int chunk, int n_splits, int window, float scale, cudaStream_t stream) {
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(n_seqs > 0 && n_heads > 0 && d > 0 && n_splits >= 1, "attention_decode_static: bad sizes");
  const long long need = llm_attention_decode_static_floats_needed(n_seqs, n_heads, d, n_splits);
  LLM_REQUIRE(need <= (long long)LLM_ATTENTION_DECODE_STATIC_FLOATS,
              "attention_decode_static: %d sequences x %d heads x %d splits x (%d + 2) = %lld floats of scratch, the built-in "
              "array holds %lld; use fewer splits or sequences per call, or llm_attention_decode with scratch of your own",
              n_seqs, n_heads, n_splits, d, need, (long long)LLM_ATTENTION_DECODE_STATIC_FLOATS);
  float *ws_o = nullptr, *ws_ml = nullptr;
  if (n_splits > 1) {
    // The array that is looked up is the current device's; a stream of another device would make
    // the kernels run there with this device's address.
    if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread) {
      int cur = -1, sdev = -1;
      LLM_CHECK_CUDA(cudaGetDevice(&cur), "attention_decode_static: cudaGetDevice");
      if (cudaStreamGetDevice(stream, &sdev) == cudaSuccess)
        LLM_REQUIRE(sdev == cur, "attention_decode_static: the stream belongs to device %d, the current device is %d; make "
                    "the stream's device current before the call", sdev, cur);
      else
        cudaGetLastError();
    }
    float *base = nullptr;
    const int rc = static_scratch(&base);
    if (rc != LLM_OK) return rc;
    ws_o = base;
    ws_ml = base + (size_t)n_seqs * n_heads * n_splits * d;
  }
  return llm_attention_decode(q, q_stride, out, out_stride, kc, vc, tok_pos, page_table, pt_stride, n_seqs, n_heads, n_kv,
                              d, page_size, chunk, n_splits, window, scale, ws_o, ws_ml, stream);
}
