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
__device__ __forceinline__ float from_ordered_key(unsigned key) {
  return __uint_as_float((key & 0x80000000u) ? (key ^ 0x80000000u) : ~key);
}
// The tail of a draw: `cand` holds the sorted candidates (key << 32 | ~index); their probabilities
// exp((x - mx) / t) / Z come from the keys themselves, all at once (a thread that fetched the
// logits one by one from memory, stopping at top_p, waited for memory up to a hundred times, longer
// than the passes over the row take); then one thread walks the shortest prefix that reaches top_p
// and draws from it.  Called by all threads of the block; `probs` has MAX_TOP_K floats.
__device__ __forceinline__ void draw_from_sorted(const unsigned long long *cand, float *probs, int k, float mx, float inv_t,
                                                 float Z, float top_p, float u, int *out) {
  for (int i = threadIdx.x; i < k; i += ST) probs[i] = expf((from_ordered_key((unsigned)(cand[i] >> 32)) - mx) * inv_t) / Z;
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = 0.f;
    int count = 0;
    for (int i = 0; i < k; ++i) {
      sum += probs[i];
      ++count;
      if (sum >= top_p) break;
    }
    const float r = u * sum;
    float acc = 0.f;
    int pick = (int)(0xffffffffu - (unsigned)(cand[count - 1] & 0xffffffffull));
    for (int i = 0; i < count; ++i) {
      acc += probs[i];
      if (r < acc) {
        pick = (int)(0xffffffffu - (unsigned)(cand[i] & 0xffffffffull));
        break;
      }
    }
    *out = pick;
  }
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
              float top_p, const float *__restrict__ uniforms, int *__restrict__ out, int only_marked) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float fscan[33];
  __shared__ int iscan[33];
  __shared__ unsigned hist[256];
  __shared__ unsigned sel_prefix, sel_mask;
  __shared__ int sel_remaining, n_greater, result;
  __shared__ unsigned long long cand[MAX_CAND];
  __shared__ float probs[MAX_TOP_K];
  __shared__ int sel_bin, n_cand;
  grid_dependents_launch();
  grid_dependency_wait();
  // after the kernel that gives a row to several blocks: only the rows it handed on (marked -1)
  if (only_marked && out[blockIdx.x] != -1) return;

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
  // ---- top_p prefix and the draw
  draw_from_sorted(cand, probs, k, mx, inv_t, Z, top_p, u, out + blockIdx.x);
}

// ---------------------------------------------------------------- a row over a cluster of blocks
// One block's three passes over a row of 128,256 logits are three times half a megabyte against
// L2's latency, 12 us each.  Here the eight blocks of a thread-block cluster take an eighth of the
// row each and meet through distributed shared memory: the maximum (every block reads the eight
// partial ones), then the sum of the exponentials and the counts per bin (block 0 adds the eight up,
// in block order, and finds the bin where the count reaches top_k), then the candidates, which every
// block appends to block 0's list; block 0 sorts and draws as the single block does.  A row that
// the quick selection does not settle (see sample_kernel) is marked -1 and taken by a launch of
// sample_kernel that follows and looks at marked rows only.  Every block of a cluster passes the
// same cluster barriers: the branches between them depend on values all of them read alike.
constexpr int SC = 8;

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in this block's generic address space, of the same shared variable in block `rank`.
template <typename T>
__device__ __forceinline__ T *in_block(T *p, unsigned rank) {
  unsigned long long out;
  asm volatile("mapa.u64 %0, %1, %2;" : "=l"(out) : "l"((unsigned long long)p), "r"(rank));
  return reinterpret_cast<T *>(out);
}

__global__ void __cluster_dims__(SC, 1, 1) __launch_bounds__(ST)
argmax_cluster_kernel(const float *__restrict__ logits, long long stride, int V, int *__restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float xmax;
  __shared__ int xidx;
  grid_dependents_launch();
  grid_dependency_wait();
  const unsigned rank = cluster_rank();
  const int r = blockIdx.x / SC;
  const float *row = logits + (size_t)r * stride;
  const int per = (((V + SC - 1) / SC) + 3) & ~3;
  const int lo = min(V, (int)rank * per), hi = min(V, lo + per);
  ArgMax a = block_argmax(row + lo, hi - lo, sv, si);
  if (threadIdx.x == 0) {
    xmax = hi > lo ? a.v : -INFINITY;
    xidx = a.i + lo;
  }
  cluster_sync_all();
  if (rank == 0 && threadIdx.x == 0) {
    ArgMax top{-INFINITY, 0x7fffffff};
    for (unsigned q = 0; q < SC; ++q) top = better(top, ArgMax{*in_block(&xmax, q), *in_block(&xidx, q)});
    out[r] = top.i == 0x7fffffff ? 0 : top.i;
  }
  cluster_sync_all();             // nobody's shared memory goes away while block 0 reads it
}

__global__ void __cluster_dims__(SC, 1, 1) __launch_bounds__(ST)
sample_cluster_kernel(const float *__restrict__ logits, long long stride, int V, float temperature, int top_k,
                      float top_p, const float *__restrict__ uniforms, int *__restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float fscan[33];
  __shared__ unsigned hist[SEL_BINS];
  __shared__ unsigned long long cand[MAX_CAND];
  __shared__ float probs[MAX_TOP_K];
  __shared__ float xmax, xz, row_z;
  __shared__ int xidx, sel_bin, n_cand;
  grid_dependents_launch();
  grid_dependency_wait();
  const unsigned rank = cluster_rank();
  const int r = blockIdx.x / SC;
  const int tid = threadIdx.x;
  const float *row = logits + (size_t)r * stride;
  const int per = (((V + SC - 1) / SC) + 3) & ~3;
  const int lo = min(V, (int)rank * per), hi = min(V, lo + per);
  const float *mine = row + lo;
  const int n_mine = hi - lo;

  // ---- the row's maximum
  {
    const ArgMax a = block_argmax(mine, n_mine, sv, si);
    if (tid == 0) {
      xmax = n_mine > 0 ? a.v : -INFINITY;
      xidx = a.i + lo;
    }
  }
  cluster_sync_all();
  ArgMax top{-INFINITY, 0x7fffffff};
  for (unsigned q = 0; q < SC; ++q) top = better(top, ArgMax{*in_block(&xmax, q), *in_block(&xidx, q)});
  if (top.i == 0x7fffffff) top.i = 0;
  if (temperature <= 0.f) {
    if (rank == 0 && tid == 0) out[r] = top.i;
    cluster_sync_all();
    return;
  }
  const float inv_t = 1.f / temperature;
  const float mx = top.v;
  const int k = min(top_k, V);

  // ---- exponentials' sum and counts per bin over this block's share
  if (tid < SEL_BINS) hist[tid] = 0u;
  __syncthreads();
  float part = 0.f;
  auto take = [&](float x) {
    const float d = (mx - x) * inv_t;
    part += expf((x - mx) * inv_t);
    const int bin = (int)(d * 32.f);
    if (d >= 0.f && bin < SEL_BINS) atomicAdd(&hist[bin], 1u);
  };
  const bool wide = ((uintptr_t)mine & 15) == 0;
  if (wide) {
    const int n4 = n_mine >> 2;
    const float4 *row4 = reinterpret_cast<const float4 *>(mine);
    for (int i = tid; i < n4; i += ST) {
      const float4 v = row4[i];
      take(v.x);
      take(v.y);
      take(v.z);
      take(v.w);
    }
    for (int j = 4 * n4 + tid; j < n_mine; j += ST) take(mine[j]);
  } else {
    for (int i = tid; i < n_mine; i += ST) take(mine[i]);
  }
  float z_mine;
  block_exclusive_scan(part, fscan, &z_mine);
  if (tid == 0) xz = z_mine;
  cluster_sync_all();
  if (rank == 0) {
    if (tid < SEL_BINS) {
      unsigned h = 0;
      for (unsigned q = 0; q < SC; ++q) h += in_block(hist, q)[tid];
      hist[tid] = h;
    }
    __syncthreads();
    if (tid == 0) {
      float z = 0.f;
      for (unsigned q = 0; q < SC; ++q) z += *in_block(&xz, q);
      int cum = 0, b = 0;
      for (; b < SEL_BINS; ++b) {
        cum += (int)hist[b];
        if (cum >= k) break;
      }
      sel_bin = (b < SEL_BINS && cum <= MAX_CAND) ? b : -1;
      row_z = z;
      n_cand = 0;
    }
  }
  cluster_sync_all();
  const int last = *in_block(&sel_bin, 0);
  const float Z = *in_block(&row_z, 0);
  if (last < 0) {                       // not settled here: the single block's kernel takes the row
    if (rank == 0 && tid == 0) out[r] = -1;
    cluster_sync_all();
    return;
  }

  // ---- the candidates, appended to block 0's list
  {
    unsigned long long *cand0 = in_block(cand, 0);
    int *n0 = in_block(&n_cand, 0);
    auto keep = [&](float x, int i) {
      const float d = (mx - x) * inv_t;
      if (d >= 0.f && (int)(d * 32.f) <= last) {
        const int s = atomicAdd(n0, 1);
        cand0[s] = ((unsigned long long)ordered_key(x) << 32) | (unsigned)(0xffffffffu - (unsigned)i);
      }
    };
    if (wide) {
      const int n4 = n_mine >> 2;
      const float4 *row4 = reinterpret_cast<const float4 *>(mine);
      for (int i = tid; i < n4; i += ST) {
        const float4 v = row4[i];
        keep(v.x, lo + 4 * i);
        keep(v.y, lo + 4 * i + 1);
        keep(v.z, lo + 4 * i + 2);
        keep(v.w, lo + 4 * i + 3);
      }
      for (int j = 4 * n4 + tid; j < n_mine; j += ST) keep(mine[j], lo + j);
    } else {
      for (int i = tid; i < n_mine; i += ST) keep(mine[i], lo + i);
    }
  }
  cluster_sync_all();
  if (rank != 0) return;

  // ---- block 0: sort (value falling, index rising on ties), top_p prefix, the draw
  const int n_sort = n_cand;
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
  draw_from_sorted(cand, probs, k, mx, inv_t, Z, top_p, uniforms[r], out + r);
}

LLM_EXPORT int llm_argmax(const float *logits, long long stride, int n_rows, int vocab, int *out,
                          cudaStream_t stream) {
  if (n_rows == 0) return LLM_OK;
  LLM_REQUIRE(n_rows > 0 && vocab > 0 && stride >= vocab, "argmax: bad sizes");
  if (vocab >= 8 * ST) {            // rows long enough to share out
    LLM_REQUIRE((long long)n_rows * SC < (1ll << 31), "argmax: too many rows");
    llm_launch(argmax_cluster_kernel, n_rows * SC, ST, 0, stream, logits, stride, vocab, out);
  } else {
    llm_launch(argmax_kernel, n_rows, ST, 0, stream, logits, stride, vocab, out);
  }
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
  if (top_k > 0 && vocab >= 8 * ST) {
    // the row over a cluster of blocks; what that leaves undecided (flat rows) to the single block
    LLM_REQUIRE((long long)n_rows * SC < (1ll << 31), "sample: too many rows");
    llm_launch(sample_cluster_kernel, n_rows * SC, ST, 0, stream, logits, stride, vocab, temperature, top_k, top_p, uniforms, out);
    LLM_CHECK_LAUNCH("sample");
    llm_launch(sample_kernel, n_rows, ST, 0, stream, logits, stride, vocab, temperature, top_k, top_p, uniforms, out, 1);
  } else {
    llm_launch(sample_kernel, n_rows, ST, 0, stream, logits, stride, vocab, temperature, top_k, top_p, uniforms, out, 0);
  }
  LLM_CHECK_LAUNCH("sample");
  return LLM_OK;
}
