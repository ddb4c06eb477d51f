// Sampling on the device from 32-bit logits: greedy, and temperature with top-k / top-p.
//
// The draw follows the reference's CPU sampler step by step (src/libllm/generator.cc:47-129,
// 197-214): logits * (1/temperature), softmax over the whole vocabulary, the top_k most
// probable tokens in falling order, the shortest prefix of them whose probabilities reach
// top_p, then r = u * (sum of that prefix) and the first candidate whose running sum
// exceeds r.  The reference's CUDA sampler picks from the same candidate set with an
// exponential race over top_k random numbers (src/flint/cuda/sampling.cu:121-163); one
// uniform number per draw is used here instead so that a draw is a pure function of
// (logits, u) and can be checked against a plain implementation.
//
// Additions with no counterpart there: temperature 0 is greedy (lowest index wins a tie),
// and top_k = 0 draws from the whole vocabulary in index order (top_p must then be 1).
//
// One block of 1024 threads per row; no scratch memory outside shared memory; every
// reduction has a fixed order, so a row's result does not depend on the other rows.
#include "common.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_sampling_last_error)

constexpr int ST = 1024;         // threads per row
constexpr int MAX_TOP_K = 1024;
constexpr int MAX_CAND = 2048;   // candidates the quick selection sorts; more: the radix selection
constexpr int SEL_BINS = 256;    // bins of the quick selection, 1/32 wide in (max - logit) / temperature

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgMax warp_argmax(ArgMax a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = better(a, b);
  }
  return a;
}

__device__ ArgMax block_argmax(const float *row, int V, float *sv, int *si) {
  ArgMax a{-INFINITY, 0x7fffffff};
  if (((uintptr_t)row & 15) == 0) {
    // Four values a load and four loads in flight: a row of 128,256 logits is 125 dependent
    // scalar loads a thread otherwise, and the step waits for the slowest row.  The candidates meet
    // in `better`, which does not depend on the order they come in (ties go to the lower index).
    const int n4 = V >> 2;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);
    int i = threadIdx.x;
    for (; i + 3 * ST < n4; i += 4 * ST) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = row4[i + u * ST];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = 4 * (i + u * ST);
        a = better(a, ArgMax{v[u].x, c});
        a = better(a, ArgMax{v[u].y, c + 1});
        a = better(a, ArgMax{v[u].z, c + 2});
        a = better(a, ArgMax{v[u].w, c + 3});
      }
    }
    for (; i < n4; i += ST) {
      const float4 v = row4[i];
      a = better(a, ArgMax{v.x, 4 * i});
      a = better(a, ArgMax{v.y, 4 * i + 1});
      a = better(a, ArgMax{v.z, 4 * i + 2});
      a = better(a, ArgMax{v.w, 4 * i + 3});
    }
    for (int j = 4 * n4 + threadIdx.x; j < V; j += ST) a = better(a, ArgMax{row[j], j});
  } else {
    for (int i = threadIdx.x; i < V; i += ST) {
      ArgMax b{row[i], i};
      a = better(a, b);
    }
  }
  a = warp_argmax(a);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { sv[warp] = a.v; si[warp] = a.i; }
  __syncthreads();
  if (warp == 0) {
    ArgMax b{sv[lane], si[lane]};
    b = warp_argmax(b);
    if (lane == 0) { sv[0] = b.v; si[0] = b.i; }
  }
  __syncthreads();
  ArgMax r{sv[0], si[0]};
  __syncthreads();
  if (r.i == 0x7fffffff) r.i = 0;    // a row of NaN or -inf: still a valid index
  return r;
}

__global__ void __launch_bounds__(ST) argmax_kernel(const float *__restrict__ logits, long long stride,
                                                    int V, int *__restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  grid_dependents_launch();
  grid_dependency_wait();
  const ArgMax r = block_argmax(logits + (size_t)blockIdx.x * stride, V, sv, si);
  if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

__device__ __forceinline__ unsigned ordered_key(float x) {
  const unsigned b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Inclusive scan over the block's threads in thread order; returns this thread's
// exclusive prefix, *total the sum of all.
__device__ float block_exclusive_scan(float v, float *warp_tot /*33*/, float *total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    float w = warp_tot[lane];
    float winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    warp_tot[lane] = winc - w;       // exclusive prefix of each warp
    if (lane == 31) warp_tot[32] = winc;
  }
  __syncthreads();
  const float res = warp_tot[warp] + inc - v;
  *total = warp_tot[32];
  __syncthreads();
  return res;
}
__device__ int block_exclusive_scan_int(int v, int *warp_tot /*33*/, int *total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += n;
  }
  __syncthreads();
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tot[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += n;
    }
    warp_tot[lane] = winc - w;
    if (lane == 31) warp_tot[32] = winc;
  }
  __syncthreads();
  const int res = warp_tot[warp] + inc - v;
  *total = warp_tot[32];
  __syncthreads();
  return res;
}

__global__ void __launch_bounds__(ST)
sample_kernel(const float *__restrict__ logits, long long stride, int V, float temperature, int top_k,
              float top_p, const float *__restrict__ uniforms, int *__restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float fscan[33];
  __shared__ int iscan[33];
  __shared__ unsigned hist[256];
  __shared__ unsigned sel_prefix, sel_mask;
  __shared__ int sel_remaining, n_greater, result;
  __shared__ unsigned long long cand[MAX_CAND];
  __shared__ int sel_bin, n_cand;
  grid_dependents_launch();
  grid_dependency_wait();

  const float *row = logits + (size_t)blockIdx.x * stride;
  const int tid = threadIdx.x;
  const ArgMax top = block_argmax(row, V, sv, si);
  if (temperature <= 0.f) {
    if (tid == 0) out[blockIdx.x] = top.i;
    return;
  }
  const float inv_t = 1.f / temperature;
  const float mx = top.v;
  const float u = uniforms[blockIdx.x];
  // Contiguous chunk per thread: sums and scans follow the vocabulary's order.
  const int chunk = (V + ST - 1) / ST;
  const int c0 = min(V, tid * chunk), c1 = min(V, c0 + chunk);

  // With top_k the sum is only the normaliser: one pass with every thread striding over the row
  // (four values a load when the row allows) sums the exponentials and counts, in bins of
  // (max - logit) / temperature, the logits within 8 of the maximum.  The candidates are then the
  // logits in the bins up to the one where the count reaches top_k; sorted, their first top_k are
  // the top_k of the row.  Seven passes of one block over half a megabyte become three.  Flat rows
  // (more than MAX_CAND candidates, or fewer than top_k logits within 8 of the maximum) take the
  // radix selection below, which is exact for any row.
  float part = 0.f;
  const int k = min(top_k, V);
  bool quick = false;
  if (top_k > 0) {
    if (tid < SEL_BINS) hist[tid] = 0u;
    __syncthreads();
    auto take = [&](float x) {
      const float d = (mx - x) * inv_t;
      part += expf((x - mx) * inv_t);
      const int bin = (int)(d * 32.f);
      if (d >= 0.f && bin < SEL_BINS) atomicAdd(&hist[bin], 1u);
    };
    if (((uintptr_t)row & 15) == 0) {
      const int n4 = V >> 2;
      const float4 *row4 = reinterpret_cast<const float4 *>(row);
      for (int i = tid; i < n4; i += ST) {
        const float4 v = row4[i];
        take(v.x);
        take(v.y);
        take(v.z);
        take(v.w);
      }
      for (int j = 4 * n4 + tid; j < V; j += ST) take(row[j]);
    } else {
      for (int i = tid; i < V; i += ST) take(row[i]);
    }
  } else {
    for (int i = c0; i < c1; ++i) part += expf((row[i] - mx) * inv_t);
  }
  float Z;
  const float before = block_exclusive_scan(part, fscan, &Z);     // also a barrier: the counts are complete

  if (top_k == 0) {
    const float r = u * Z;
    if (tid == 0) result = 0;
    __syncthreads();
    // The owner of r is the last thread whose running sum before its chunk is <= r
    // (thread 0 always qualifies); taking the maximum keeps the choice unique even where
    // rounding makes two neighbouring prefixes equal or out of order by one ulp.
    if (before <= r && c1 > c0) atomicMax(&result, tid);
    __syncthreads();
    const int owner = result;
    __syncthreads();
    if (tid == owner) {
      float acc = before;
      int pick = c1 - 1;
      for (int i = c0; i < c1; ++i) {
        acc += expf((row[i] - mx) * inv_t);
        if (r < acc) { pick = i; break; }
      }
      out[blockIdx.x] = pick;
    }
    return;
  }

  // ---- the quick selection: the bin where the count reaches top_k, and what lies up to it
  if (tid == 0) {
    int cum = 0, b = 0;
    for (; b < SEL_BINS; ++b) {
      cum += (int)hist[b];
      if (cum >= k) break;
    }
    sel_bin = (b < SEL_BINS && cum <= MAX_CAND) ? b : -1;
    n_cand = 0;
  }
  __syncthreads();
  quick = sel_bin >= 0;
  int n_sort = k;
  if (quick) {
    const int last = sel_bin;
    auto keep = [&](float x, int i) {
      const float d = (mx - x) * inv_t;
      if (d >= 0.f && (int)(d * 32.f) <= last) {
        const int s = atomicAdd(&n_cand, 1);
        cand[s] = ((unsigned long long)ordered_key(x) << 32) | (unsigned)(0xffffffffu - (unsigned)i);
      }
    };
    if (((uintptr_t)row & 15) == 0) {
      const int n4 = V >> 2;
      const float4 *row4 = reinterpret_cast<const float4 *>(row);
      for (int i = tid; i < n4; i += ST) {
        const float4 v = row4[i];
        keep(v.x, 4 * i);
        keep(v.y, 4 * i + 1);
        keep(v.z, 4 * i + 2);
        keep(v.w, 4 * i + 3);
      }
      for (int j = 4 * n4 + tid; j < V; j += ST) keep(row[j], j);
    } else {
      for (int i = tid; i < V; i += ST) keep(row[i], i);
    }
    __syncthreads();
    n_sort = n_cand;
  }
  // ---- otherwise the top_k-th largest logit by radix selection over order-preserving keys
  if (!quick) {
  if (tid == 0) { sel_prefix = 0u; sel_mask = 0u; sel_remaining = k; }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned prefix = sel_prefix, mask = sel_mask;
    for (int i = tid; i < V; i += ST) {
      const unsigned key = ordered_key(row[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      int remaining = sel_remaining;
      int b = 255;
      for (; b > 0; --b) {
        const int h = (int)hist[b];
        if (remaining <= h) break;
        remaining -= h;
      }
      sel_remaining = remaining;
      sel_prefix = prefix | ((unsigned)b << shift);
      sel_mask = mask | (0xffu << shift);
    }
    __syncthreads();
  }
  const unsigned kth = sel_prefix;
  const int need_ties = sel_remaining;            // how many keys equal to kth are taken
  const int greater = k - need_ties;              // keys above kth: all taken
  if (tid == 0) n_greater = 0;
  __syncthreads();
  int my_ties = 0;
  for (int i = c0; i < c1; ++i) {
    const unsigned key = ordered_key(row[i]);
    if (key > kth) {
      const int s = atomicAdd(&n_greater, 1);
      cand[s] = ((unsigned long long)key << 32) | (unsigned)(0xffffffffu - (unsigned)i);
    } else if (key == kth) {
      ++my_ties;
    }
  }
  int total_ties;
  int tie_rank = block_exclusive_scan_int(my_ties, iscan, &total_ties);
  if (my_ties > 0 && tie_rank < need_ties) {
    for (int i = c0; i < c1 && tie_rank < need_ties; ++i) {
      if (ordered_key(row[i]) == kth) {
        cand[greater + tie_rank] = ((unsigned long long)kth << 32) | (unsigned)(0xffffffffu - (unsigned)i);
        ++tie_rank;
      }
    }
  }
  }  // radix selection
  // ---- sort the candidates: value falling, index rising on ties (bitonic, padded)
  int n = 1;
  while (n < n_sort) n <<= 1;
  for (int i = n_sort + tid; i < n; i += ST) cand[i] = 0ull;
  __syncthreads();
  for (int size = 2; size <= n; size <<= 1) {
    for (int strd = size >> 1; strd > 0; strd >>= 1) {
      for (int i = tid; i < n; i += ST) {
        const int j = i ^ strd;
        if (j > i) {
          const bool desc = (i & size) == 0;
          const unsigned long long a = cand[i], b = cand[j];
          if ((a < b) == desc) { cand[i] = b; cand[j] = a; }
        }
      }
      __syncthreads();
    }
  }
  // ---- top_p prefix and the draw (sequential over at most top_k candidates)
  if (tid == 0) {
    float sum = 0.f;
    int count = 0;
    for (int i = 0; i < k; ++i) {
      const int idx = (int)(0xffffffffu - (unsigned)(cand[i] & 0xffffffffull));
      sum += expf((row[idx] - mx) * inv_t) / Z;
      ++count;
      if (sum >= top_p) break;
    }
    const float r = u * sum;
    float acc = 0.f;
    int pick = (int)(0xffffffffu - (unsigned)(cand[count - 1] & 0xffffffffull));
    for (int i = 0; i < count; ++i) {
      const int idx = (int)(0xffffffffu - (unsigned)(cand[i] & 0xffffffffull));
      acc += expf((row[idx] - mx) * inv_t) / Z;
      if (r < acc) { pick = idx; break; }
    }
    out[blockIdx.x] = pick;
  }
}

LLM_EXPORT int llm_argmax(const float *logits, long long stride, int n_rows, int vocab, int *out,
                          cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && vocab > 0 && stride >= vocab, "argmax: bad sizes");
  llm_launch(argmax_kernel, n_rows, ST, 0, stream, logits, stride, vocab, out);
  LLM_CHECK_LAUNCH("argmax");
  return LLM_OK;
}

LLM_EXPORT int llm_sample(const float *logits, long long stride, int n_rows, int vocab, float temperature,
                          int top_k, float top_p, const float *uniforms, int *out, cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && vocab > 0 && stride >= vocab, "sample: bad sizes");
  LLM_REQUIRE(temperature >= 0.f, "sample: temperature must not be negative");
  LLM_REQUIRE(top_k >= 0 && top_k <= MAX_TOP_K, "sample: top_k %d is outside 0..%d", top_k, MAX_TOP_K);
  LLM_REQUIRE(top_p > 0.f, "sample: top_p must be positive");
  LLM_REQUIRE(top_k > 0 || top_p >= 1.f, "sample: top_p below 1 needs a top_k");
  llm_launch(sample_kernel, n_rows, ST, 0, stream, logits, stride, vocab, temperature, top_k, top_p, uniforms, out);
  LLM_CHECK_LAUNCH("sample");
  return LLM_OK;
}
