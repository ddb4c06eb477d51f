// Attention for decoding steps on the tensor cores, with the rotation of q and k, the append
// of k and v to the paged cache and the joining of the key splits in the same launch.
//
// Every sequence brings one token.  CTA (split, kv head, sequence) takes `chunk` cached keys
// for all query heads of the kv head's group: the group's heads are the rows of one 16-row
// MMA tile (rows beyond the group are zeros), so S = Q K^T and O += P V are mma.sync m16n8k16
// products and the issue slots stay free for the loads, which is what this kernel is bound
// by (it reads K and V once; a kernel that computes the scores on the FMA pipe spends its
// time issuing).  Key tiles are pages of the cache ([64, d] contiguous) fetched by 16-byte
// asynchronous copies, two to four in flight (issued before the dependency on the previous kernel is
// waited for); each of the four warps takes 16 keys of a tile with a
// running maximum and sum of its own, and the four are joined at the end.
//
// What the reference does in some twenty launches per layer (fourteen for the rotation,
// src/libllm/llama.cc:151-176; two re-allocating appends, :203-212; the split-KV attention and
// its combine kernel, src/flint/cuda/flash_attn.cc:165-180) is one launch here:
//  * q's heads are rotated from the 32-bit q|k|v row into the MMA tile; the CTA whose keys
//    include the new token rotates k, writes k and v to the cache and puts them into its tile;
//  * each CTA writes its split's unnormalised output, maximum and sum to scratch, and the
//    CTA that finishes last for a (sequence, kv head) joins the splits in split order, so the
//    result does not depend on which one that is.
// Head h reads kv head h / (heads / kv_heads); scores are scaled by `scale` (1/sqrt(d),
// src/flint/operators.cc:43-56, 115-117); one query sees every cached key or the last `window`.
#include "common.cuh"
#include "mma_tiles.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_attention_decode_tc_last_error)

constexpr int DT_BN = 64;      // keys per tile = tokens per page
constexpr int DT_ROWS = 16;    // rows of the MMA tile: query heads of one group

// Key/value tiles kept in flight per CTA.  Two, so that a CTA is small and several share an SM (five
// at head size 64, three at 128): the loads in flight per SM come from the number of CTAs, and a
// step's CTAs all fit on the GPU at once instead of running in one and a bit waves.
__host__ __device__ constexpr int decode_tc_stages(int d) { return 2; }

// DT_WARPS warps share a tile's 64 keys (64 / DT_WARPS each, a running maximum and sum per warp,
// joined at the end).  Four warps run: with one warp per CTA (no waiting for other warps at a
// tile) 64 sequences take as long, and 1 or 8 take up to twice as long (measured), because the
// rotation, the copies' issue and the joining are then one warp's work.
// exp2 of a number that is never above zero here: one instruction (-inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// A pair of 32-bit floats from L2, issued where it stands (the split join issues many before it uses any).
__device__ __forceinline__ float2 ld_l2_pair(const float *p) {
  float2 v;
  asm volatile("ld.global.cg.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
  return v;
}

template <int D, int DT_WARPS>
__global__ void __launch_bounds__(DT_WARPS * 32, D <= 64 ? 5 : 3)
attention_decode_tc_kernel(const float *__restrict__ qkv, long long qkv_stride, int qkv_parts,
                           long long qkv_part_stride, const float *__restrict__ table,
                           int table_rows, int rot_dim, const int *__restrict__ tok_pos,
                           const int *__restrict__ page_table, int pt_stride, __nv_bfloat16 *__restrict__ kc,
                           __nv_bfloat16 *__restrict__ vc, int write_cache, int n_heads, int n_kv, int G, int chunk,
                           int window, float scale_log2, float *__restrict__ ws_o, float *__restrict__ ws_ml,
                           int *__restrict__ counters, int n_splits, __nv_bfloat16 *__restrict__ out,
                           long long out_stride) {
  constexpr int LD = D + 8;
  constexpr int CHUNKS = D / 8;
  constexpr int KS = D / 16;
  constexpr int DT = D / 8;
  constexpr int NS = decode_tc_stages(D);                    // key tiles in flight
  constexpr int KW = DT_BN / DT_WARPS;                       // keys of a tile per warp
  constexpr int NTW = KW / 8;                                // its score tiles of 8 keys
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16 *sQ = reinterpret_cast<__nv_bfloat16 *>(smem_raw);           // [16][LD]
  __nv_bfloat16 *sNew = sQ + DT_ROWS * LD;                                    // [2][LD]: new k, new v
  __nv_bfloat16 *sK = sNew + 2 * LD;                                          // [NS][64][LD]
  __nv_bfloat16 *sV = sK + NS * DT_BN * LD;                                   // [NS][64][LD]
  int *s_pages = reinterpret_cast<int *>(sV + NS * DT_BN * LD);
  __shared__ float sm_m[DT_WARPS][DT_ROWS], sm_l[DT_WARPS][DT_ROWS];
  __shared__ int s_last;

  grid_dependents_launch();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int pos = tok_pos[b];
  const int len = pos + 1;
  const int kstart = window > 0 ? max(0, len - window) : 0;
  // chunk 0: the sequence's own length cut into n_splits runs of whole pages, so that every split
  // has work whatever bound on the length the launch was shaped for
  if (chunk <= 0) chunk = max(DT_BN, ((len + n_splits - 1) / n_splits + DT_BN - 1) / DT_BN * DT_BN);
  const int c0 = split * chunk;
  const int c1 = min(c0 + chunk, len);
  if (c0 >= len || c1 <= kstart) {
    grid_dependency_wait();
    return;
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int first_tile = max(c0, kstart) / DT_BN, last_tile = (c1 - 1) / DT_BN;
  {
    const int *pt = page_table + (size_t)b * pt_stride;
    for (int i = first_tile + tid; i <= last_tile; i += DT_WARPS * 32) s_pages[i - first_tile] = pt[i];
  }
  const bool owns_new = write_cache && pos >= c0 && pos < c1;     // c1 = len here
  const int half = rot_dim / 2;
  const float *cs = table + (size_t)(pos < table_rows ? pos : table_rows - 1) * rot_dim;
  __syncthreads();

  auto load_kv = [&](int kt, int stage) {
    const int page = s_pages[kt - first_tile];
    const size_t base = ((size_t)page * n_kv + kvh) * DT_BN * D;
    __nv_bfloat16 *dk = sK + stage * DT_BN * LD, *dv = sV + stage * DT_BN * LD;
    for (int c = tid; c < DT_BN * CHUNKS; c += DT_WARPS * 32) {
      const int r = c / CHUNKS, ch = c % CHUNKS;
      cp_async16(dk + r * LD + ch * 8, kc + base + (size_t)r * D + ch * 8, true);
      cp_async16(dv + r * LD + ch * 8, vc + base + (size_t)r * D + ch * 8, true);
    }
  };
  // The cached keys and values of earlier tokens do not depend on the kernel before this one
  // (positions and page tables come from the step's descriptor, copied before the step's first
  // kernel): the first NS tiles are on their way while that kernel, the q|k|v product, still
  // runs.  The new token's row is put into its tile by hand further down.
  // A run that reads another run's cache (write_cache == 0) finds the new token's row written by
  // that run's kernel, a few launches earlier in this same step.  Overlapping launches do not
  // order such a kernel before this one's prologue (each kernel only waits for the one directly
  // before it), so this form fetches nothing before the wait.
  if (write_cache) {
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      if (first_tile + i <= last_tile) load_kv(first_tile + i, i);
      cp_async_commit();
    }
  }
  grid_dependency_wait();
  if (!write_cache) {
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      if (first_tile + i <= last_tile) load_kv(first_tile + i, i);
      cp_async_commit();
    }
  }

  // The group's queries, rotated, as rows of the MMA tile (rows beyond the group are zeros), and
  // the new token's key (rotated) and value: into the cache, and kept for this CTA's own tile.
  const float *row = qkv + (size_t)b * qkv_stride;
  size_t new_dst = 0;
  if (owns_new) {
    const int page = s_pages[pos / DT_BN - first_tile];
    new_dst = (((size_t)page * n_kv + kvh) * DT_BN + (pos % DT_BN)) * D;
  }
  constexpr int MAXP = 8;
  const bool vec = rot_dim == D && qkv_parts <= MAXP && (qkv_stride % 4 == 0) && (qkv_part_stride % 4 == 0) &&
                   ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)table % 16 == 0);
  if (vec) {
    // Four channel pairs per item; an item issues the loads of all parts before it adds them (in
    // order), so the CTA waits for memory once.  Items: G heads of q, then k, then v (two halves).
    constexpr int GROUPS = D / 8;                          // items per head
    const int n_items = (G + (owns_new ? 2 : 0)) * GROUPS;
    for (int i = tid; i < DT_ROWS * D / 8; i += DT_WARPS * 32)      // rows beyond the group
      if (i / (D / 8) >= G) *reinterpret_cast<uint4 *>(sQ + (i / (D / 8)) * LD + (i % (D / 8)) * 8) = make_uint4(0, 0, 0, 0);
    for (int item = tid; item < n_items; item += DT_WARPS * 32) {
      const int h = item / GROUPS, j = (item % GROUPS) * 4;
      const bool is_k = h == G, is_v = h == G + 1;
      const float *src = row + (size_t)(is_v ? n_heads + n_kv + kvh : (is_k ? n_heads + kvh : kvh * G + h)) * D;
      float4 a[MAXP], bb[MAXP];
#pragma unroll
      for (int p = 0; p < MAXP; ++p)
        if (p < qkv_parts) {
          a[p] = ld4(src + (size_t)p * qkv_part_stride + j);
          bb[p] = ld4(src + (size_t)p * qkv_part_stride + j + D / 2);
        }
      const float4 c = ld4(cs + j), sn = ld4(cs + D / 2 + j);
      float4 x = a[0], y = bb[0];
#pragma unroll
      for (int p = 1; p < MAXP; ++p)
        if (p < qkv_parts) {
          x.x += a[p].x; x.y += a[p].y; x.z += a[p].z; x.w += a[p].w;
          y.x += bb[p].x; y.y += bb[p].y; y.z += bb[p].z; y.w += bb[p].w;
        }
      float4 lo, hi;
      if (is_v) {
        lo = x;
        hi = y;
      } else {
        lo = make_float4(x.x * c.x - y.x * sn.x, x.y * c.y - y.y * sn.y, x.z * c.z - y.z * sn.z, x.w * c.w - y.w * sn.w);
        hi = make_float4(y.x * c.x + x.x * sn.x, y.y * c.y + x.y * sn.y, y.z * c.z + x.z * sn.z, y.w * c.w + x.w * sn.w);
      }
      if (h < G) {
        st4(sQ + h * LD + j, lo);
        st4(sQ + h * LD + j + D / 2, hi);
      } else {
        __nv_bfloat16 *keep = sNew + (is_v ? LD : 0);
        st4(keep + j, lo);
        st4(keep + j + D / 2, hi);
        __nv_bfloat16 *dstc = (is_v ? vc : kc) + new_dst;
        st4(dstc + j, lo);
        st4(dstc + j + D / 2, hi);
      }
    }
  } else {
    // one value of the stacked row: the product's parts over K added in order
    auto val = [&](const float *p) {
      float v = p[0];
      for (int i = 1; i < qkv_parts; ++i) v += p[(size_t)i * qkv_part_stride];
      return v;
    };
    for (int i = tid; i < DT_ROWS * D; i += DT_WARPS * 32) {
      const int h = i / D, c = i % D;
      float v = 0.f;
      if (h < G) {
        const float *qh = row + (size_t)(kvh * G + h) * D;
        if (c < half) v = val(qh + c) * cs[c] - val(qh + c + half) * cs[half + c];
        else if (c < rot_dim) v = val(qh + c) * cs[c - half] + val(qh + c - half) * cs[c];
        else v = val(qh + c);
      }
      sQ[h * LD + c] = __float2bfloat16_rn(v);
    }
    if (owns_new) {
      const float *kh = row + (size_t)(n_heads + kvh) * D, *vh = row + (size_t)(n_heads + n_kv + kvh) * D;
      for (int c = tid; c < D; c += DT_WARPS * 32) {
        float kv;
        if (c < half) kv = val(kh + c) * cs[c] - val(kh + c + half) * cs[half + c];
        else if (c < rot_dim) kv = val(kh + c) * cs[c - half] + val(kh + c - half) * cs[c];
        else kv = val(kh + c);
        const __nv_bfloat16 kb = __float2bfloat16_rn(kv), vb = __float2bfloat16_rn(val(vh + c));
        sNew[c] = kb;
        sNew[LD + c] = vb;
        kc[new_dst + c] = kb;
        vc[new_dst + c] = vb;
      }
    }
  }

  unsigned qf[KS][4];
  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  __syncthreads();                       // sQ and sNew are written
  for (int kt = first_tile; kt <= last_tile; ++kt) {
    const int stage = (kt - first_tile) % NS;
    cp_async_wait<NS - 1>();             // one group per tile, NS - 1 newer ones may be in flight
    __syncthreads();
    __nv_bfloat16 *tk = sK + stage * DT_BN * LD, *tv = sV + stage * DT_BN * LD;
    if (owns_new && kt == pos / DT_BN) {
      // the copy may have fetched this row before the new token was written: put it in by hand
      const int r = pos % DT_BN;
      for (int c = tid; c < D; c += DT_WARPS * 32) {
        tk[r * LD + c] = sNew[c];
        tv[r * LD + c] = sNew[LD + c];
      }
      __syncthreads();
    }
    if (kt == first_tile) {
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) ldmatrix_x4(qf[ks], sQ + (lane & 15) * LD + ks * 16 + (lane >> 4) * 8);
    }
    // this warp's keys of the tile
    const int k0 = kt * DT_BN + warp * KW;
    if (k0 < c1 && k0 + KW > kstart) {
      float s[NTW][4];
#pragma unroll
      for (int n = 0; n < NTW; ++n)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[n][j] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
        for (int n2 = 0; n2 < NTW / 2; ++n2) {
          unsigned kb[4];
          ldmatrix_x4(kb, tk + (warp * KW + n2 * 16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
          mma16816(s[2 * n2], qf[ks], kb[0], kb[1]);
          mma16816(s[2 * n2 + 1], qf[ks], kb[2], kb[3]);
        }
      }
      if (k0 + KW > c1 || k0 < kstart) {
#pragma unroll
        for (int n = 0; n < NTW; ++n)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int key = k0 + n * 8 + 2 * t + (j & 1);
            if (key >= c1 || key < kstart) s[n][j] = -INFINITY;
          }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int n = 0; n < NTW; ++n) {
        mx[0] = fmaxf(mx[0], fmaxf(s[n][0], s[n][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[n][2], s[n][3]));
      }
      float alpha[2], moff[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        moff[r] = m_new == -INFINITY ? 0.f : m_new * scale_log2;
        alpha[r] = m_run[r] == -INFINITY ? 0.f : fast_exp2(m_run[r] * scale_log2 - moff[r]);
        m_run[r] = m_new;
      }
      float sum[2] = {0.f, 0.f};
#pragma unroll
      for (int n = 0; n < NTW; ++n) {
        s[n][0] = fast_exp2(fmaf(s[n][0], scale_log2, -moff[0]));
        s[n][1] = fast_exp2(fmaf(s[n][1], scale_log2, -moff[0]));
        s[n][2] = fast_exp2(fmaf(s[n][2], scale_log2, -moff[1]));
        s[n][3] = fast_exp2(fmaf(s[n][3], scale_log2, -moff[1]));
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
#pragma unroll
      for (int kk = 0; kk < KW / 16; ++kk) {
        unsigned pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d2 = 0; d2 < DT / 2; ++d2) {
          unsigned vb[4];
          ldmatrix_x4_trans(vb, tv + (warp * KW + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + d2 * 16 + (lane >> 4) * 8);
          mma16816(o[2 * d2], pa, vb[0], vb[1]);
          mma16816(o[2 * d2 + 1], pa, vb[2], vb[3]);
        }
      }
    }
    __syncthreads();                     // every warp is done with the stage
    if (kt + NS <= last_tile) load_kv(kt + NS, stage);
    cp_async_commit();
  }
  cp_async_wait<0>();
  __syncthreads();

  // Join the warps (each saw other keys): through shared memory, in warp order.
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  float *sm_o = reinterpret_cast<float *>(sK);                 // [4][16][D], over the tiles (no longer read)
  {
    const int ra = g, rb = g + 8;
    if (t == 0) {
      sm_m[warp][ra] = m_run[0] == -INFINITY ? -INFINITY : m_run[0] * scale_log2;
      sm_m[warp][rb] = m_run[1] == -INFINITY ? -INFINITY : m_run[1] * scale_log2;
      sm_l[warp][ra] = l_run[0];
      sm_l[warp][rb] = l_run[1];
    }
#pragma unroll
    for (int i = 0; i < DT; ++i) {
      float *pa = sm_o + ((size_t)(warp * DT_ROWS + ra) * D + i * 8 + 2 * t);
      float *pb = sm_o + ((size_t)(warp * DT_ROWS + rb) * D + i * 8 + 2 * t);
      pa[0] = o[i][0];
      pa[1] = o[i][1];
      pb[0] = o[i][2];
      pb[1] = o[i][3];
    }
  }
  __syncthreads();
  const int n_active_first = kstart / chunk, n_active_last = (len - 1) / chunk;
  const int n_active = n_active_last - n_active_first + 1;
  for (int idx = tid; idx < G * D; idx += DT_WARPS * 32) {
    const int h = idx / D, c = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) M = fmaxf(M, sm_m[w][h]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) {
      const float f = sm_m[w][h] == -INFINITY ? 0.f : fast_exp2(sm_m[w][h] - M);
      L += sm_l[w][h] * f;
      O += sm_o[(size_t)(w * DT_ROWS + h) * D + c] * f;
    }
    const int head = kvh * G + h;
    if (n_active == 1) {
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
  if (n_active == 1) return;

  // The CTA that is last to finish for this (sequence, kv head) joins the splits.
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int old = atomicAdd(&counters[b * n_kv + kvh], 1);
    s_last = old == n_active - 1;
    if (s_last) counters[b * n_kv + kvh] = 0;          // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // The splits' results come from L2, which answers slowly while the next product's CTAs fill their
  // rings: every thread issues all loads of a batch of splits for its two channels before it uses
  // any, and the (maximum, sum) pairs of the batch, which all channels of a head share, come into
  // shared memory once.  A thread waits for memory once a batch; the sums keep the split order.
  constexpr int JB = 16;
  float2 *s_ml = reinterpret_cast<float2 *>(sK) + (size_t)DT_WARPS * DT_ROWS * D / 2;   // [G][JB], behind sm_o
  for (int base = 0; base < G * D / 2; base += DT_WARPS * 32) {      // a channel pair per thread (one round for a group of 4 heads of 64)
    const int idx = base + tid;
    const bool mine = idx < G * D / 2;
    const int h = mine ? idx / (D / 2) : 0, c = mine ? (idx % (D / 2)) * 2 : 0;
    const size_t my_slot0 = ((size_t)b * n_heads + kvh * G + h) * n_splits;
    float M = -INFINITY, L = 0.f, O0 = 0.f, O1 = 0.f;
    for (int s0 = n_active_first; s0 <= n_active_last; s0 += JB) {
      float2 ov[JB];
#pragma unroll
      for (int j = 0; j < JB; ++j)
        ov[j] = ld_l2_pair(ws_o + (my_slot0 + min(s0 + j, n_active_last)) * D + c);
      for (int i = tid; i < G * JB; i += DT_WARPS * 32) {
        const int hh = i / JB, j = i % JB;
        const size_t slot0 = ((size_t)b * n_heads + kvh * G + hh) * n_splits;
        float2 ml = ld_l2_pair(ws_ml + (slot0 + min(s0 + j, n_active_last)) * 2);
        if (s0 + j > n_active_last) ml = make_float2(-INFINITY, 0.f);
        s_ml[i] = ml;
      }
      __syncthreads();
      float Mb = M;
#pragma unroll
      for (int j = 0; j < JB; ++j) Mb = fmaxf(Mb, s_ml[h * JB + j].x);
      const float keep = M == -INFINITY ? 0.f : fast_exp2(M - Mb);      // what was summed so far, to the new maximum
      L *= keep;
      O0 *= keep;
      O1 *= keep;
      M = Mb;
#pragma unroll
      for (int j = 0; j < JB; ++j) {
        const float2 ml = s_ml[h * JB + j];
        const float f = ml.x == -INFINITY ? 0.f : fast_exp2(ml.x - Mb);
        L += ml.y * f;
        O0 += ov[j].x * f;
        O1 += ov[j].y * f;
      }
      __syncthreads();
    }
    if (mine)
      *reinterpret_cast<__nv_bfloat162 *>(out + (size_t)b * out_stride + (size_t)(kvh * G + h) * D + c) =
          __floats2bfloat162_rn(O0 / L, O1 / L);
  }
}

template <int D>
static int launch_decode_tc(const float *qkv, long long qkv_stride, int qkv_parts, long long qkv_part_stride,
                            const float *table, int table_rows, int rot_dim,
                            const int *tok_pos, const int *page_table, int pt_stride, void *kc, void *vc,
                            int write_cache, int n_seqs, int n_heads, int n_kv, int chunk, int max_len, int n_splits,
                            int window, float scale, float *ws_o, float *ws_ml, int *counters, void *out, long long out_stride,
                            cudaStream_t stream) {
  constexpr int LD = D + 8;
  const size_t tiles = (size_t)(DT_ROWS + 2 + 2 * decode_tc_stages(D) * DT_BN) * LD * sizeof(__nv_bfloat16);
  const int widest = chunk > 0 ? chunk : ((max_len + n_splits - 1) / n_splits + 2 * DT_BN);
  const size_t smem = tiles + (size_t)(widest / DT_BN + 2) * sizeof(int);
  LLM_REQUIRE(smem <= 200 * 1024, "attention_decode_tc: a chunk of %d keys spans too many pages", chunk);
  constexpr int DT_WARPS = 4;
  auto kern = attention_decode_tc_kernel<D, DT_WARPS>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, smem), "attention_decode_tc attribute");
  dim3 grid(n_splits, n_kv, n_seqs);
  LLM_CHECK_CUDA(llm_launch(kern, grid, dim3(DT_WARPS * 32), smem, stream, qkv, qkv_stride, qkv_parts, qkv_part_stride, table, table_rows,
                            rot_dim,
                            tok_pos, page_table, pt_stride, (__nv_bfloat16 *)kc, (__nv_bfloat16 *)vc, write_cache,
                            n_heads, n_kv, n_heads / n_kv, chunk, window, scale * 1.4426950408889634f, ws_o, ws_ml,
                            counters, n_splits, (__nv_bfloat16 *)out, out_stride),
                 "attention_decode_tc launch");
  return LLM_OK;
}

// CTAs of this kernel that fit one SM at head size d (shared memory and registers), for choosing
// how many key splits fill the GPU once.
LLM_EXPORT int llm_attention_decode_tc_ctas_per_sm(int d) {
  const size_t smem = (size_t)(DT_ROWS + 2 + 2 * decode_tc_stages(d) * DT_BN) * (d + 8) * sizeof(__nv_bfloat16) + 2048;
  const int by_smem = (int)((227 * 1024) / smem);
  const int by_regs = d <= 64 ? 5 : 3;
  return by_smem < by_regs ? (by_smem < 1 ? 1 : by_smem) : by_regs;
}

// 1 if this head size, page size and group size have an instantiation, else 0.
LLM_EXPORT int llm_attention_decode_tc_supports(int d, int page_size, int group) {
  return page_size == DT_BN && d >= 16 && d <= 128 && d % 16 == 0 && group >= 1 && group <= DT_ROWS;
}

// qkv [B, (heads + 2 kv_heads) * d] 32-bit (the stacked product, not rotated; with qkv_parts > 1 it
// is the sum of that many partial products qkv_part_stride floats apart), table
// [positions, rot_dim] (cosines, then sines), caches [pages, kv_heads, 64, d] bfloat16, tok_pos[b]
// the position of sequence b's token.  With write_cache the token's k and v are appended.  Keys are
// cut into n_splits runs of `chunk`, or, with chunk 0, each sequence's own length into n_splits runs of
// whole pages (max_len then bounds the lengths: it sizes the CTA's list of pages).
// ws_o needs B*heads*n_splits*d floats, ws_ml B*heads*n_splits*2, counters B*kv_heads ints that are
// zero before the first launch (the kernel leaves them zero).
LLM_EXPORT int llm_attention_decode_tc(const float *qkv, long long qkv_stride, int qkv_parts,
                                       long long qkv_part_stride, const float *table, int table_rows,
                                       int rot_dim, const int *tok_pos, const int *page_table, int pt_stride,
                                       void *kc, void *vc, int write_cache, int n_seqs, int n_heads, int n_kv, int d,
                                       int page_size, int chunk, int max_len, int n_splits, int window, float scale,
                                       float *ws_o,
                                       float *ws_ml, int *counters, void *out, long long out_stride,
                                       cudaStream_t stream) {
  if (n_seqs == 0) return LLM_OK;
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_kv > 0 && n_kv <= 65535 && n_heads % n_kv == 0,
              "attention_decode_tc: bad sizes");
  LLM_REQUIRE(llm_attention_decode_tc_supports(d, page_size, n_heads / n_kv),
              "attention_decode_tc: head size %d, pages of %d, %d query heads per kv head is not built", d, page_size,
              n_heads / n_kv);
  LLM_REQUIRE(chunk >= 0 && chunk % page_size == 0 && n_splits >= 1 && (chunk > 0 || max_len > 0),
              "attention_decode_tc: chunk %d must be a multiple of the page size (0: cut each sequence's own length, "
              "then a bound on the lengths is needed)", chunk);
  LLM_REQUIRE(rot_dim > 0 && rot_dim % 2 == 0 && rot_dim <= d, "attention_decode_tc: rotated width %d does not fit head size %d", rot_dim, d);
  LLM_REQUIRE(n_splits == 1 || (ws_o && ws_ml && counters), "attention_decode_tc: splits need scratch memory");
  LLM_REQUIRE(qkv_parts >= 1 && qkv_parts <= 64, "attention_decode_tc: %d parts of the stacked product", qkv_parts);
  LLM_REQUIRE((uintptr_t)kc % 16 == 0 && (uintptr_t)vc % 16 == 0 && (uintptr_t)out % 4 == 0 && out_stride % 2 == 0,
              "attention_decode_tc: caches must be 16-byte aligned");
#define DT_CASE(DD)                                                                                                 \
  if (d == DD)                                                                                                      \
    return launch_decode_tc<DD>(qkv, qkv_stride, qkv_parts, qkv_part_stride, table, table_rows, rot_dim, tok_pos, page_table, pt_stride, kc, vc, \
                                write_cache, n_seqs, n_heads, n_kv, chunk, max_len, n_splits, window, scale, ws_o,  \
                                ws_ml,                                                                              \
                                counters, out, out_stride, stream);
  DT_CASE(16) DT_CASE(32) DT_CASE(48) DT_CASE(64) DT_CASE(80) DT_CASE(96) DT_CASE(112) DT_CASE(128)
#undef DT_CASE
  LLM_FAIL("attention_decode_tc: no kernel for head size %d", d);
}
