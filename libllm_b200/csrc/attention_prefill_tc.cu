// Causal grouped-query attention for prompt steps on the 5th-generation tensor cores: the flash
// form (running maximum and sum per query row, scores never stored) with both products as
// tcgen05.mma, their accumulators in tensor memory and all operands brought by TMA.
//
// One CTA takes 128 query rows of one head of one sequence.  Its warps:
//   warp 8    one lane loads the Q tile once and then, page by page, the K and V tiles (a page of
//             the cache is a [64, d] block = one key tile) into a ring of shared-memory stages;
//   warp 9    one lane issues S = Q K^T (operands K-major, 128-byte swizzle) into one of two score
//             buffers in tensor memory;
//   warp 10   one lane issues, when the probabilities are ready, O += P V_j: P is the A operand
//             straight from tensor memory, V the MN-major B operand (it lies [key][channel] in the
//             cache and is used as it is); the output row stays in tensor memory from the first
//             tile to the last;
//   warps 0-7 two threads per query row (warp w and w + 4 reach the same 32 lanes of tensor memory),
//             each with half of the tile's keys: reads its half of the row of S (no shuffles: a row
//             is one lane), masks, exchanges the maximum with its partner through shared memory,
//             exponentials and their sum in 32-bit, and writes its half of the row of P as packed
//             bfloat16 over the scores it has just consumed.  Neither P nor O passes through
//             shared memory, whose bandwidth the two products' other operands need.
// The exponent's reference per row is not every tile's maximum: it moves only when a new maximum
// exceeds it by more than 2^8 (in the exponent), and then, tile finished, the threads rescale the
// output row in tensor memory and their sums.  P stays below 2^8, which bfloat16 and the 32-bit
// accumulators hold as well as they hold [0, 1]; after the first tiles of a row the reference
// seldom moves, so the output is seldom touched.
// With two score buffers the scores of tile j + 1 are computed while the row threads work on tile j;
// a buffer is written again when the output product has read the probabilities that lay over it.  A
// second CTA on the same SM fills the rest.  Exponentials are exp2 of scores pre-scaled by
// log2(e) / sqrt(d).
//
// Semantics as the other attention kernels: token i of a sequence that stands behind `past` cached
// ones sees keys 0..past+i (src/flint/operators.cc:119-124), head h reads kv head h / (heads /
// kv_heads) (:43-56), optional window.  Head sizes 64 and 128, pages of 64 tokens.  Every wait has
// a time limit (see tc_common.cuh).  The reference calls FlashAttention-2's sm_80 kernel here
// (src/flint/cuda/flash_attn.cc:101-186).
#include "common.cuh"
#include "tc_common.cuh"
#include <math.h>

LLM_DEFINE_LAST_ERROR(llm_attention_prefill_tc_last_error)

namespace {

constexpr int FT_THREADS = 384;   // warps 0-7: two threads per query row; 8: loader; 9, 10: tensor-core issue; 11: none
constexpr int FT_BM = 128;          // query rows per CTA
constexpr int FT_BN = 64;           // keys per tile = tokens per page

template <int D>
struct FtShape {
  static constexpr int KB = D / 64;                         // 64-wide blocks of the head size
  static constexpr int Q_BYTES = FT_BM * D * 2;
  static constexpr int KV_BYTES = FT_BN * D * 2;            // one of K or V
  static constexpr int X_BYTES = 2 * 2 * FT_BM * 4;          // the partners' maxima, two tiles deep
  static constexpr int STAGES = D == 64 ? 4 : 2;
  static constexpr int TMEM_COLS = 256;                     // two S buffers (64 columns each) + O (D columns)
  static constexpr size_t SMEM = Q_BYTES + X_BYTES + (size_t)STAGES * 2 * KV_BYTES + 256;   // two CTAs per SM
  // Registers move from the third warpgroup (loader, issuer) to the row threads.  The CTA is launched
  // with 80 registers a thread (2 CTAs x 384 threads on an SM), and what the row threads take must
  // be what the third warpgroup gives up inside the same CTA: a request beyond that waits for ever.
  static constexpr int REGS_LAUNCH = 80, REGS_FEW = 48, REGS_MANY = 96;
  static_assert(128 * REGS_FEW + 256 * REGS_MANY <= FT_THREADS * REGS_LAUNCH, "register moves must balance within the CTA");
};


// V as the MN-major operand: a tile lies [key][64 channels] in 128-byte swizzled rows, 8 keys per
// 1024 bytes (checked on the device: 16 keys further = 2048 bytes further); a second block of 64
// channels lies a whole tile (64 keys x 128 bytes) further on, which the descriptor's leading offset says.
__host__ __device__ constexpr unsigned instr_desc_mn(int m, int n) { return instr_desc(m, n) | (1u << 16); }

// the largest of three in one instruction
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// exp2 of a number that is never far above zero here: one instruction (inputs of -inf give 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(FT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16 *__restrict__ out,
                            long long out_stride, const int *__restrict__ seq_start, const int *__restrict__ seq_past,
                            const int *__restrict__ page_table, int pt_stride, int n_heads, int n_kv, int window,
                            float scale_log2, int *status) {
  using S = FtShape<D>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char *sQ = smem, *sKV = smem + S::Q_BYTES;
  float *xch = reinterpret_cast<float *>(sKV + (size_t)STAGES * 2 * S::KV_BYTES);       // [2][2][128]
  unsigned long long *bars = (unsigned long long *)(xch + 4 * FT_BM);
  // full[STAGES], empty[STAGES], q_full, s_full[2], p_full[2] (one per score buffer each), o_full, pv_done[2]
  const unsigned bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const unsigned bar_q = smem_u32(bars + 2 * STAGES), bar_sfull = bar_q + 8,
                 bar_pfull = bar_q + 24, bar_ofull = bar_q + 40, bar_pvdone = bar_q + 48;
  unsigned *tmem_slot = (unsigned *)(bars + 2 * STAGES + 9);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  // out of a shuffle, so that the compiler knows the number to be the same in all lanes of a warp
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  grid_dependents_launch();
  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_q);
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
  }
  if (smem_u32(smem) & 1023u) {                               // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, 21);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_q, 1);
    mbar_init(bar_sfull, 1);
    mbar_init(bar_sfull + 8, 1);
    mbar_init(bar_pfull, 8);
    mbar_init(bar_pfull + 8, 8);
    mbar_init(bar_ofull, 1);
    mbar_init(bar_pvdone, 1);
    mbar_init(bar_pvdone + 8, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((unsigned)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;
  const unsigned tmem_s = tmem_base, tmem_o = tmem_base + 2 * FT_BN;

  // every thread: the previous kernel wrote the queries and this step's keys and values
  grid_dependency_wait();
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = seq_start[b], n_q = seq_start[b + 1] - q0, past = seq_past[b];
  const int tile = gridDim.x - 1 - blockIdx.x;               // long tiles first
  const int r0 = tile * FT_BM;
  const bool active = r0 < n_q;
  const int rows = active ? min(FT_BM, n_q - r0) : 0;
  const int kvh = h / (n_heads / n_kv);
  const int last_tile = active ? (past + r0 + rows - 1) / FT_BN : -1;
  const int first_tile = window > 0 ? max(0, past + r0 - window + 1) / FT_BN : 0;
  const int n_tiles = last_tile - first_tile + 1;             // <= 0: nothing to do
  const int *pt = page_table + (size_t)b * pt_stride;

  // The loader's and the issuers' loops run in all lanes of their warps (waits, addresses and
  // descriptors in the uniform datapath); lane 0 issues the copies, products and commits.
  // Everything the third warpgroup runs stands behind its release of registers, so that the
  // compiler holds that code to what is left (what it used beyond would be the row threads' by then).
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(S::REGS_FEW));
  if (warp == 8) {
    // ------------------------------------------------------------ loader
    const bool leader = elect_one();
    if (n_tiles > 0) {
      if (leader) {
        mbar_expect_tx(bar_q, S::Q_BYTES);
        for (int kb = 0; kb < S::KB; ++kb) {
          tma_load_2d(smem_u32(sQ) + kb * (FT_BM * 128), &map_q, h * D + kb * 64, q0 + r0, bar_q);
          tma_load_2d(smem_u32(sQ) + kb * (FT_BM * 128) + 64 * 128, &map_q, h * D + kb * 64, q0 + r0 + 64, bar_q);
        }
      }
      int stage = 0;
      unsigned phase = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, status, 11));
        if (!ok) break;
        const int row = (pt[first_tile + j] * n_kv + kvh) * FT_BN;
        const unsigned dk = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES), dv = dk + S::KV_BYTES;
        if (leader) {
          mbar_expect_tx(bar_full + 8 * stage, 2 * S::KV_BYTES);
          for (int kb = 0; kb < S::KB; ++kb) {
            tma_load_2d(dk + kb * (FT_BN * 128), &map_k, kb * 64, row, bar_full + 8 * stage);
            tma_load_2d(dv + kb * (FT_BN * 128), &map_v, kb * 64, row, bar_full + 8 * stage);
          }
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (leader && (!ok || *abort_flag)) {
        const unsigned long long t0 = globaltimer();
        for (int s = 0; s < STAGES; ++s)
          while (!mbar_try(bar_full + 8 * s, 0) && !mbar_try(bar_full + 8 * s, 1) && globaltimer() - t0 < 2000000ull) {
          }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ tensor-core issue: scores
    // The two products have an issuing warp each.
    const bool leader = elect_one();
    if (n_tiles > 0) {
      constexpr unsigned IDESC_S = instr_desc(FT_BM, FT_BN);          // S[128 x 64 keys], both operands K-major
      bool ok = __all_sync(0xffffffffu, mbar_wait(bar_q, 0, abort_flag, status, 12));
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stage = j % STAGES;
        ok = mbar_wait(bar_full + 8 * stage, (j / STAGES) & 1, abort_flag, status, 13);
        // buffer j & 1 last held the scores of tile j - 2 and then its probabilities, which the
        // other warp's product has to have read
        if (ok && j >= 2) ok = mbar_wait(bar_pvdone + 8 * (j & 1), ((j >> 1) - 1) & 1, abort_flag, status, 14);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const unsigned ka = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES);
        if (leader) {
#pragma unroll
          for (int kb = 0; kb < S::KB; ++kb)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              tc_mma(tmem_s + (j & 1) * FT_BN, smem_desc(smem_u32(sQ) + kb * (FT_BM * 128) + kk * 32),
                     smem_desc(ka + kb * (FT_BN * 128) + kk * 32), IDESC_S, (kb > 0 || kk > 0) ? 1u : 0u);
          tc_commit(bar_sfull + 8 * (j & 1));
        }
        __syncwarp();
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------ tensor-core issue: output
    const bool leader = elect_one();
    if (n_tiles > 0) {
      constexpr unsigned IDESC_O = instr_desc_mn(FT_BM, D);           // O[128 x D channels], V MN-major
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stage = j % STAGES;
        ok = mbar_wait(bar_full + 8 * stage, (j / STAGES) & 1, abort_flag, status, 15) &&
             mbar_wait(bar_pfull + 8 * (j & 1), (j >> 1) & 1, abort_flag, status, 16);   // and the output row rescaled, if it had to be
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const unsigned va = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES) + S::KV_BYTES;
        // 16 keys to a product: 8 columns of P (it lies over the scores' first columns), 16 rows of
        // V; all D channels at once, the second block of 64 channels FT_BN rows further on
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < FT_BN / 16; ++kk)
            tc_mma_ts(tmem_o, tmem_s + (j & 1) * FT_BN + kk * 8, smem_desc_lbo(va + kk * 2048, FT_BN * 128), IDESC_O,
                      (j > 0 || kk > 0) ? 1u : 0u);
          tc_commit(bar_ofull);
          tc_commit(bar_pvdone + 8 * (j & 1));
          tc_commit(bar_empty + 8 * stage);
        }
        __syncwarp();
      }
    }
  }
  } else {
    // ------------------------------------------------------------ two threads per query row
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(S::REGS_MANY));
    const int quarter = warp & 3, half = warp >> 2;
    const int row = quarter * 32 + lane;                       // row of the tile = lane of tensor memory
    const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
    const int pos = past + r0 + row;                           // the row's position in its sequence
    constexpr int HD = D / 2;                                  // this thread's channels of the output row
    const unsigned o_addr = tmem_o + lane_addr + half * HD;
    float ref = -INFINITY;            // the exponent's reference, already times log2(e) / sqrt(d)
    float l_run = 0.f;                // sum of this thread's exponentials, relative to ref
    bool ok = n_tiles > 0;
    // Partners meet at a hardware barrier in every tile, so neither leaves the loop early: a thread
    // whose wait ran out goes on through the barriers without working.
    for (int j = 0; j < n_tiles; ++j) {
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_sfull + 8 * (j & 1), (j >> 1) & 1, abort_flag, status, 18));
      const unsigned s_addr = tmem_s + (j & 1) * FT_BN + lane_addr;
      const int k0 = (first_tile + j) * FT_BN + half * 32;    // this thread's first key
      float own[2][16];
      float *xrow = xch + (j & 1) * 2 * FT_BM + row;
      if (ok) {
        tc_fence_after();
        tc_ld16_issue(s_addr + half * 32, own[0]);
        tc_ld16_issue(s_addr + half * 32 + 16, own[1]);
        tc_ld_wait();
        tc_ld_ready(own[0]);
        tc_ld_ready(own[1]);
        if ((k0 + 31 > past + r0) || (window > 0 && k0 <= past + r0 + FT_BM - 1 - window)) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int key = k0 + c * 16 + i;
              if (!(key <= pos && (window <= 0 || key > pos - window))) own[c][i] = -INFINITY;
            }
        }
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, not one of sixteen
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 16; i += 2) m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], own[c][i], own[c][i + 1]);
        xrow[half * FT_BM] = fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]);
        tc_fence_before();
      }
      // Past this barrier the partner has its maximum in shared memory and its scores in registers,
      // so the probabilities may be written over them.
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      if (!ok) continue;
      const float mxs = fmaxf(xrow[0], xrow[FT_BM]) * scale_log2;
      if (__any_sync(0xffffffffu, mxs > ref + 8.f)) {          // a warp decides as one: the loads below are its own
        const float new_ref = fmaxf(ref, mxs);
        const float alpha = new_ref == -INFINITY ? 1.f : fast_exp2(ref - new_ref);
        if (j > 0) {
          // the output row may be touched when the tensor core has finished the previous tile's product
          ok = __all_sync(0xffffffffu, mbar_wait(bar_ofull, (j - 1) & 1, abort_flag, status, 19));
          if (!ok) continue;
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 32) {
            float t[2][16];
            tc_ld16_issue(o_addr + c0, t[0]);
            tc_ld16_issue(o_addr + c0 + 16, t[1]);
            tc_ld_wait();
            tc_ld_ready(t[0]);
            tc_ld_ready(t[1]);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
              for (int i = 0; i < 16; ++i) t[c][i] *= alpha;
              tc_st16(o_addr + c0 + c * 16, t[c]);
            }
          }
        }
        l_run *= alpha;
        ref = new_ref;
      }
      const float moff = ref == -INFINITY ? 0.f : ref;
      // two scores to an instruction for the scaling and for the sum (packed 32-bit pairs)
      float2 sum4[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 scale2 = make_float2(scale_log2, scale_log2), off2 = make_float2(-moff, -moff);
      unsigned pk[16];                                        // the half row of P: two keys to a column
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float (&v)[16] = own[c];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          const float2 t = __ffma2_rn(make_float2(v[i], v[i + 1]), scale2, off2);
          const float e0 = fast_exp2(t.x), e1 = fast_exp2(t.y);
          sum4[(i >> 1) & 3] = __fadd2_rn(sum4[(i >> 1) & 3], make_float2(e0, e1));
          const __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
          pk[c * 8 + (i >> 1)] = *reinterpret_cast<const unsigned *>(&b2);
        }
      }
      const float2 sum2 = __fadd2_rn(__fadd2_rn(sum4[0], sum4[1]), __fadd2_rn(sum4[2], sum4[3]));
      l_run += sum2.x + sum2.y;
      // The probabilities' barrier is one per score buffer: a pair of warps may be a tile ahead of
      // the others (nothing holds it back but the scores), and on a single barrier its arrival for
      // the next tile would complete this tile's phase in a slower warp's place.
      tc_st16(s_addr + half * 16, pk);
      tc_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull + 8 * (j & 1));
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_ofull, (n_tiles - 1) & 1, abort_flag, status, 20));
    // The row's sum is the two threads' sums, first half first.  Every row warp comes here, whatever
    // happened above.
    asm volatile("bar.sync 5, 256;" ::: "memory");          // the last tile's maxima have been read
    xch[half * FT_BM + row] = l_run;
    asm volatile("bar.sync 5, 256;" ::: "memory");
    const float l_row = xch[row] + xch[FT_BM + row];
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l_row;
      __nv_bfloat16 *dst = out + (size_t)(q0 + r0 + row) * out_stride + (size_t)h * D + half * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        float t[2][16];
        tc_ld16_issue(o_addr + c0, t[0]);
        tc_ld16_issue(o_addr + c0 + 16, t[1]);
        tc_ld_wait();
        tc_ld_ready(t[0]);
        tc_ld_ready(t[1]);
        if (row < rows) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int h8 = 0; h8 < 2; ++h8) {
              uint4 v;
              __nv_bfloat162 t0 = __floats2bfloat162_rn(t[c][h8 * 8] * inv, t[c][h8 * 8 + 1] * inv),
                             t1 = __floats2bfloat162_rn(t[c][h8 * 8 + 2] * inv, t[c][h8 * 8 + 3] * inv),
                             t2 = __floats2bfloat162_rn(t[c][h8 * 8 + 4] * inv, t[c][h8 * 8 + 5] * inv),
                             t3 = __floats2bfloat162_rn(t[c][h8 * 8 + 6] * inv, t[c][h8 * 8 + 7] * inv);
              v.x = *reinterpret_cast<unsigned *>(&t0);
              v.y = *reinterpret_cast<unsigned *>(&t1);
              v.z = *reinterpret_cast<unsigned *>(&t2);
              v.w = *reinterpret_cast<unsigned *>(&t3);
              *reinterpret_cast<uint4 *>(dst + c0 + c * 16 + h8 * 8) = v;
            }
        }
      }
      tc_fence_before();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)S::TMEM_COLS)
                 : "memory");
  }
}

template <int D>
int launch_prefill_tc(const void *q, long long q_stride, long long n_tokens, void *out, long long out_stride,
                      const void *kc, const void *vc, long long n_pages, const int *seq_start, const int *seq_past,
                      const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads, int n_kv, int window,
                      float scale, int *status, cudaStream_t stream) {
  using S = FtShape<D>;
  CUtensorMap map_q, map_k, map_v;
  int rc = get_map(q, n_tokens, (long long)n_heads * D, q_stride, 64, &map_q);
  if (rc != LLM_OK) return rc;
  rc = get_map(kc, n_pages * n_kv * FT_BN, D, D, 64, &map_k);
  if (rc != LLM_OK) return rc;
  rc = get_map(vc, n_pages * n_kv * FT_BN, D, D, 64, &map_v);
  if (rc != LLM_OK) return rc;
  auto kern = attention_prefill_tc_kernel<D>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, S::SMEM), "attention_prefill_tc attribute");
  dim3 grid((max_q_len + FT_BM - 1) / FT_BM, n_heads, n_seqs);
  LLM_CHECK_CUDA(llm_launch(kern, grid, dim3(FT_THREADS), S::SMEM, stream, map_q, map_k, map_v, (__nv_bfloat16 *)out,
                            out_stride, seq_start, seq_past, page_table, pt_stride, n_heads, n_kv, window,
                            scale * 1.4426950408889634f, status),
                 "attention_prefill_tc launch");
  return LLM_OK;
}

}  // namespace

// 1 if this head size and page size have an instantiation, else 0.
LLM_EXPORT int llm_attention_prefill_tc_supports(int d, int page_size) {
  return page_size == FT_BN && (d == 64 || d == 128);
}

// q [n_tokens, >= heads*d] bfloat16 (rotated; row stride q_stride elements), out [n_tokens, heads*d],
// caches [n_pages, kv_heads, 64, d]; sequence b owns rows seq_start[b]..seq_start[b+1]-1, which stand at
// positions seq_past[b].. of the sequence; max_q_len bounds the rows of a sequence.  `status` (device
// int, may be null) receives a non-zero code if a wait inside the kernel ran out of time.
LLM_EXPORT int llm_attention_prefill_tc(const void *q, long long q_stride, long long n_tokens, void *out,
                                        long long out_stride, const void *kc, const void *vc, long long n_pages,
                                        const int *seq_start, const int *seq_past, const int *page_table,
                                        int pt_stride, int n_seqs, int max_q_len, int n_heads, int n_kv, int d,
                                        int page_size, int window, float scale, int *status, cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return LLM_OK;
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_heads > 0 && n_heads <= 65535 && n_kv > 0 && n_heads % n_kv == 0,
              "attention_prefill_tc: bad sizes (%d sequences, %d heads, %d kv heads)", n_seqs, n_heads, n_kv);
  LLM_REQUIRE(llm_attention_prefill_tc_supports(d, page_size),
              "attention_prefill_tc: head size %d with pages of %d tokens is not built (64 or 128, pages of 64)", d, page_size);
  LLM_REQUIRE(q_stride % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)kc % 16 == 0 && (uintptr_t)vc % 16 == 0 &&
                  out_stride % 8 == 0 && (uintptr_t)out % 16 == 0,
              "attention_prefill_tc: rows must be 16-byte aligned");
  LLM_REQUIRE(n_pages * n_kv * FT_BN < (1ll << 31), "attention_prefill_tc: the cache has too many rows for one tensor map");
  if (d == 64)
    return launch_prefill_tc<64>(q, q_stride, n_tokens, out, out_stride, kc, vc, n_pages, seq_start, seq_past, page_table,
                                 pt_stride, n_seqs, max_q_len, n_heads, n_kv, window, scale, status, stream);
  return launch_prefill_tc<128>(q, q_stride, n_tokens, out, out_stride, kc, vc, n_pages, seq_start, seq_past, page_table,
                                pt_stride, n_seqs, max_q_len, n_heads, n_kv, window, scale, status, stream);
}
