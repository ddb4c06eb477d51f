// Causal grouped-query attention for prompt steps on the 5th-generation tensor cores: the flash
// form (running maximum and sum per query row, scores never stored) with both products as
// tcgen05.mma, their accumulators in tensor memory and all operands brought by TMA.  Two forms: the
// first, described here, for short prompts; the second ("the wide form", further down) for long ones.
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
  // The grid is [heads, sequences, query tiles]: blocks are handed out with x fastest, so every
  // head's longest (last) tile starts before anyone's second longest.  Under a causal mask a tile's
  // work grows with its index; handing out head by head left the last heads' long tiles for the end.
  const int b = blockIdx.y, h = blockIdx.x;
  const int q0 = seq_start[b], n_q = seq_start[b + 1] - q0, past = seq_past[b];
  const int tile = gridDim.z - 1 - blockIdx.z;               // long tiles first
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

// ------------------------------------------------------------------ the wide form
// For prompts of more than 128 tokens: one CTA to an SM takes 256 query rows as two tiles of 128, A
// and B, and tiles of 128 keys (two pages).  Its warps:
//   warps 0-3 / 4-7   a thread per row of tile A / B with all 128 scores of the row: no partner, no
//                     exchange of maxima; otherwise as above (lazy exponent reference, P written
//                     over the scores, the output row in tensor memory);
//   warp 8            loader: both Q tiles once, then K and V tiles, which serve both query tiles;
//   warp 9            issues all products, in the order S_A(0) S_B(0), then for every key tile j:
//                     O_A += P_A(j) V_j, S_A(j+1), O_B += P_B(j) V_j, S_B(j+1).  The tensor core
//                     works for one query tile while the other's rows compute exponentials.  A
//                     score buffer needs no second copy: products issued by one thread run in
//                     order, so S_X(j+1) cannot overtake the product that reads P_X(j).
// Tensor memory: S_A, S_B (128 columns each), O_A, O_B (D each): all 512 columns at head size 128.
// At head size 64 there is room for P_A and P_B (64 columns each) beside the scores.  Then the scores
// of tile j + 1 are asked for as soon as the rows hold tile j's in registers, and are there when the
// rows come back: what is left of the chain between two tiles of a row is its own work (the products
// take 770 of 3,400 cycles otherwise, the hand-overs to and from the issuing thread 900).
// The S product has N = 128 (the tensor core's full rate; N = 64 runs at half), and the fixed costs
// of a tile (waits, loads from tensor memory, hand-overs) are paid once for 128 keys.
constexpr int FW_THREADS = 384;
constexpr int FW_BM = 256;          // query rows per CTA
constexpr int FW_BN = 128;          // keys per tile = two pages

template <int D>
struct FwShape {
  static constexpr int KB = D / 64;
  static constexpr int Q_BYTES = FW_BM * D * 2;
  static constexpr int KV_BYTES = FW_BN * D * 2;            // one of K or V
  static constexpr int STAGES = D == 64 ? 4 : 2;
  static constexpr int TMEM_COLS = 512;
  static constexpr size_t SMEM = Q_BYTES + (size_t)STAGES * 2 * KV_BYTES + 256;   // one CTA per SM
  static constexpr int REGS_LAUNCH = 168, REGS_FEW = 56, REGS_MANY = 216;
  static_assert(128 * REGS_FEW + 256 * REGS_MANY <= FW_THREADS * REGS_LAUNCH, "register moves must balance within the CTA");
  static constexpr bool SEP_P = 2 * FW_BN + 2 * (FW_BN / 2) + 2 * D <= TMEM_COLS;    // probabilities beside the scores
  static constexpr int P_COL = SEP_P ? 2 * FW_BN : 0, P_STEP = SEP_P ? FW_BN / 2 : FW_BN;   // P of query tile x at P_COL + x * P_STEP
  static constexpr int O_COL = SEP_P ? 3 * FW_BN : 2 * FW_BN;
};

template <int D>
__global__ void __launch_bounds__(FW_THREADS, 1)
attention_prefill_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v, __nv_bfloat16 *__restrict__ out,
                              long long out_stride, const int *__restrict__ seq_start, const int *__restrict__ seq_past,
                              const int *__restrict__ page_table, int pt_stride, int n_heads, int n_kv, int window,
                              float scale_log2, int *status) {
  using S = FwShape<D>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char *sQ = smem, *sKV = smem + S::Q_BYTES;
  unsigned long long *bars = (unsigned long long *)(sKV + (size_t)STAGES * 2 * S::KV_BYTES);
  // full[STAGES], empty[STAGES], q_full, then one for each query tile: s_full[2], p_full[2], o_full[2], s_free[2]
  const unsigned bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const unsigned bar_q = smem_u32(bars + 2 * STAGES), bar_sfull = bar_q + 8, bar_pfull = bar_q + 24, bar_ofull = bar_q + 40,
                 bar_sfree = bar_q + 56;
  unsigned *tmem_slot = (unsigned *)(bars + 2 * STAGES + 9);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  grid_dependents_launch();
  if (threadIdx.x == 0) {
    tma_prefetch_map(&map_q);
    tma_prefetch_map(&map_k);
    tma_prefetch_map(&map_v);
  }
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, 21);
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_q, 1);
    for (int x = 0; x < 2; ++x) {
      mbar_init(bar_sfull + 8 * x, 1);
      mbar_init(bar_pfull + 8 * x, 4);          // the four warps of a query tile
      mbar_init(bar_ofull + 8 * x, 1);
      mbar_init(bar_sfree + 8 * x, 4);
    }
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

  grid_dependency_wait();
  // The grid is [heads, sequences, query tiles]: blocks are handed out with x fastest, so every
  // head's longest (last) tile starts before anyone's second longest.  Under a causal mask a tile's
  // work grows with its index; handing out head by head left the last heads' long tiles for the end.
  const int b = blockIdx.y, h = blockIdx.x;
  const int q0 = seq_start[b], n_q = seq_start[b + 1] - q0, past = seq_past[b];
  const int tile = gridDim.z - 1 - blockIdx.z;               // long tiles first
  const int r0 = tile * FW_BM;
  const bool active = r0 < n_q;
  const int rows = active ? min(FW_BM, n_q - r0) : 0;
  const int kvh = h / (n_heads / n_kv);
  // Key tiles of the two query tiles: A works on tiles [0, n_a) of the CTA's range, B on [j_b0, n_tiles).
  const bool has_b = rows > 128;
  const int first_tile = window > 0 ? max(0, past + r0 - window + 1) / FW_BN : 0;
  const int n_a = active ? (past + r0 + min(rows, 128) - 1) / FW_BN - first_tile + 1 : 0;
  const int n_tiles = has_b ? (past + r0 + rows - 1) / FW_BN - first_tile + 1 : n_a;
  const int j_b0 = has_b ? (window > 0 ? max(0, past + r0 + 128 - window + 1) / FW_BN : 0) - first_tile : n_tiles;
  const int *pt = page_table + (size_t)b * pt_stride;

  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(S::REGS_FEW));
  if (warp == 8) {
    // ------------------------------------------------------------ loader
    const bool leader = elect_one();
    if (n_tiles > 0) {
      if (leader) {
        mbar_expect_tx(bar_q, S::Q_BYTES);
        for (int x = 0; x < 2; ++x)
          for (int kb = 0; kb < S::KB; ++kb)
            for (int hf = 0; hf < 2; ++hf)
              tma_load_2d(smem_u32(sQ) + x * (128 * D * 2) + kb * (128 * 128) + hf * (64 * 128), &map_q, h * D + kb * 64,
                          q0 + r0 + x * 128 + hf * 64, bar_q);
      }
      const int last_page = (past + n_q - 1) / 64;            // the sequence's last page with keys
      int stage = 0;
      unsigned phase = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, status, 31));
        if (!ok) break;
        // A tile's second page may lie behind the sequence's end: the first is loaded in its place
        // (finite numbers, all masked).
        const int p0 = 2 * (first_tile + j), p1 = min(p0 + 1, last_page);
        const int row0 = (pt[p0] * n_kv + kvh) * 64, row1 = (pt[p1] * n_kv + kvh) * 64;
        const unsigned dk = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES), dv = dk + S::KV_BYTES;
        if (leader) {
          mbar_expect_tx(bar_full + 8 * stage, 2 * S::KV_BYTES);
          for (int kb = 0; kb < S::KB; ++kb) {
            tma_load_2d(dk + kb * (FW_BN * 128), &map_k, kb * 64, row0, bar_full + 8 * stage);
            tma_load_2d(dk + kb * (FW_BN * 128) + 64 * 128, &map_k, kb * 64, row1, bar_full + 8 * stage);
          }
          for (int kb = 0; kb < S::KB; ++kb) {
            tma_load_2d(dv + kb * (FW_BN * 128), &map_v, kb * 64, row0, bar_full + 8 * stage);
            tma_load_2d(dv + kb * (FW_BN * 128) + 64 * 128, &map_v, kb * 64, row1, bar_full + 8 * stage);
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
    // ------------------------------------------------------------ tensor-core issue
    const bool leader = elect_one();
    if (n_tiles > 0) {
      constexpr unsigned IDESC_S = instr_desc(128, FW_BN);            // S[128 rows x 128 keys], both operands K-major
      constexpr unsigned IDESC_O = instr_desc_mn(128, D);             // O[128 rows x D channels], V MN-major
      bool ok = __all_sync(0xffffffffu, mbar_wait(bar_q, 0, abort_flag, status, 32));
      // scores of query tile x against the key tile in `stage`
      auto scores = [&](int x, int stage) {
        const unsigned qa = smem_u32(sQ) + x * (128 * D * 2), ka = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES);
        if (leader) {
#pragma unroll
          for (int kb = 0; kb < S::KB; ++kb)
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              tc_mma(tmem_base + x * FW_BN, smem_desc(qa + kb * (128 * 128) + kk * 32),
                     smem_desc(ka + kb * (FW_BN * 128) + kk * 32), IDESC_S, (kb > 0 || kk > 0) ? 1u : 0u);
          tc_commit(bar_sfull + 8 * x);
        }
      };
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar_full, 0, abort_flag, status, 33));
      if (ok) {
        tc_fence_after();
        scores(0, 0);
        if (j_b0 == 0) scores(1, 0);
        __syncwarp();
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int stage = j % STAGES, next_stage = (j + 1) % STAGES;
        const unsigned va = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES) + S::KV_BYTES;
        if constexpr (S::SEP_P) {
          // the next tile's scores first: they need only that the rows hold this tile's in registers
#pragma unroll
          for (int x = 0; x < 2; ++x) {
            const int c = x ? j - j_b0 : j;
            const bool act = x ? j >= j_b0 : j < n_a;
            const bool act_next = j + 1 < n_tiles && (x ? j + 1 >= j_b0 : j + 1 < n_a);
            if (act_next) {
              if (act) ok = mbar_wait(bar_sfree + 8 * x, c & 1, abort_flag, status, 40);
              if (ok) ok = mbar_wait(bar_full + 8 * next_stage, ((j + 1) / STAGES) & 1, abort_flag, status, 35);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              tc_fence_after();
              scores(x, next_stage);
            }
          }
          if (!ok) break;
        }
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          const int c = x ? j - j_b0 : j;                     // how many tiles this query tile has behind it
          const bool act = x ? j >= j_b0 : j < n_a;
          const bool act_next = !S::SEP_P && j + 1 < n_tiles && (x ? j + 1 >= j_b0 : j + 1 < n_a);
          if (act) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_pfull + 8 * x, c & 1, abort_flag, status, 34));   // and the output row rescaled, if it had to be
            if (!ok) break;
            tc_fence_after();
            // 16 keys to a product: 8 columns of P (it lies over the scores' first columns), 16 rows of
            // V; all D channels at once, the second block of 64 channels a tile's rows further on
            if (leader) {
#pragma unroll
              for (int kk = 0; kk < FW_BN / 16; ++kk)
                tc_mma_ts(tmem_base + S::O_COL + x * D, tmem_base + S::P_COL + x * S::P_STEP + kk * 8,
                          smem_desc_lbo(va + kk * 2048, FW_BN * 128), IDESC_O, (c > 0 || kk > 0) ? 1u : 0u);
              tc_commit(bar_ofull + 8 * x);
            }
          }
          if (act_next) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * next_stage, ((j + 1) / STAGES) & 1, abort_flag, status, 35));
            if (!ok) break;
            tc_fence_after();
            scores(x, next_stage);
          }
        }
        if (!ok) break;
        if (leader) tc_commit(bar_empty + 8 * stage);
        __syncwarp();
      }
    }
  }
  } else {
    // ------------------------------------------------------------ a thread per query row
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(S::REGS_MANY));
    const int x = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;                       // row of the query tile = lane of tensor memory
    const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
    const int pos_lo = past + r0 + x * 128 + quarter * 32;     // the warp's first position
    const int pos = pos_lo + lane;
    const unsigned s_addr = tmem_base + x * FW_BN + lane_addr;
    const unsigned p_addr = tmem_base + S::P_COL + x * S::P_STEP + lane_addr;
    const unsigned o_addr = tmem_base + S::O_COL + x * D + lane_addr;
    const int j_lo = x ? j_b0 : 0, j_hi = x ? n_tiles : n_a;
    float ref = -INFINITY;            // the exponent's reference, already times log2(e) / sqrt(d)
    float l_run = 0.f;                // sum of the row's exponentials, relative to ref
    bool ok = j_hi > j_lo;
    for (int j = j_lo; j < j_hi && ok; ++j) {
      const int c = j - j_lo;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_sfull + 8 * x, c & 1, abort_flag, status, 36));
      if (!ok) break;
      tc_fence_after();
      float sc[8][16];
#pragma unroll
      for (int g = 0; g < 8; ++g) tc_ld16_issue(s_addr + g * 16, sc[g]);
      tc_ld_wait();
#pragma unroll
      for (int g = 0; g < 8; ++g) tc_ld_ready(sc[g]);
      if constexpr (S::SEP_P) {                               // the score buffer may be written again
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_sfree + 8 * x);
      }
      const int k0 = (first_tile + j) * FW_BN;
      if (k0 + FW_BN - 1 > pos_lo || (window > 0 && k0 <= pos_lo + 31 - window)) {
#pragma unroll
        for (int g = 0; g < 8; ++g)
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int key = k0 + g * 16 + i;
            if (!(key <= pos && (window <= 0 || key > pos - window))) sc[g][i] = -INFINITY;
          }
      }
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int g = 0; g < 8; ++g)
#pragma unroll
        for (int i = 0; i < 16; i += 2) m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], sc[g][i], sc[g][i + 1]);
      const float mxs = fmaxf(max3(m4[0], m4[1], m4[2]), m4[3]) * scale_log2;
      if (__any_sync(0xffffffffu, mxs > ref + 8.f)) {          // a warp decides as one: the loads below are its own
        const float new_ref = fmaxf(ref, mxs);
        const float alpha = new_ref == -INFINITY ? 1.f : fast_exp2(ref - new_ref);
        if (c > 0) {
          // the output row may be touched when the tensor core has finished the previous tile's product
          ok = __all_sync(0xffffffffu, mbar_wait(bar_ofull + 8 * x, (c - 1) & 1, abort_flag, status, 37));
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < D; c0 += 32) {
            float t[2][16];
            tc_ld16_issue(o_addr + c0, t[0]);
            tc_ld16_issue(o_addr + c0 + 16, t[1]);
            tc_ld_wait();
            tc_ld_ready(t[0]);
            tc_ld_ready(t[1]);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll
              for (int i = 0; i < 16; ++i) t[u][i] *= alpha;
              tc_st16(o_addr + c0 + u * 16, t[u]);
            }
          }
        }
        l_run *= alpha;
        ref = new_ref;
      }
      const float moff = ref == -INFINITY ? 0.f : ref;
      float2 sum4[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      const float2 scale2 = make_float2(scale_log2, scale_log2), off2 = make_float2(-moff, -moff);
      // 32 keys at a time: their probabilities, two to a column.  They go over the scores' first
      // columns at once, or, where they have columns of their own, when the previous tile's output
      // product has read its probabilities there (it has, as a rule, long before).
      unsigned pk[4][16];
#pragma unroll
      for (int g2 = 0; g2 < 4; ++g2) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          float (&v)[16] = sc[g2 * 2 + u];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const float2 t = __ffma2_rn(make_float2(v[i], v[i + 1]), scale2, off2);
            const float e0 = fast_exp2(t.x), e1 = fast_exp2(t.y);
            sum4[(i >> 1) & 3] = __fadd2_rn(sum4[(i >> 1) & 3], make_float2(e0, e1));
            const __nv_bfloat162 b2 = __floats2bfloat162_rn(e0, e1);
            pk[g2][u * 8 + (i >> 1)] = *reinterpret_cast<const unsigned *>(&b2);
          }
        }
        if constexpr (!S::SEP_P) tc_st16(p_addr + g2 * 16, pk[g2]);
      }
      const float2 sum2 = __fadd2_rn(__fadd2_rn(sum4[0], sum4[1]), __fadd2_rn(sum4[2], sum4[3]));
      l_run += sum2.x + sum2.y;
      if constexpr (S::SEP_P) {
        if (c > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar_ofull + 8 * x, (c - 1) & 1, abort_flag, status, 39));
          if (!ok) break;
          tc_fence_after();
        }
#pragma unroll
        for (int g2 = 0; g2 < 4; ++g2) tc_st16(p_addr + g2 * 16, pk[g2]);
      }
      tc_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull + 8 * x);
    }
    if (ok && j_hi > j_lo) ok = __all_sync(0xffffffffu, mbar_wait(bar_ofull + 8 * x, (j_hi - j_lo - 1) & 1, abort_flag, status, 38));
    if (ok && j_hi > j_lo) {
      tc_fence_after();
      const float inv = 1.f / l_run;
      __nv_bfloat16 *dst = out + (size_t)(q0 + r0 + x * 128 + row) * out_stride + (size_t)h * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        float t[2][16];
        tc_ld16_issue(o_addr + c0, t[0]);
        tc_ld16_issue(o_addr + c0 + 16, t[1]);
        tc_ld_wait();
        tc_ld_ready(t[0]);
        tc_ld_ready(t[1]);
        if (x * 128 + row < rows) {
#pragma unroll
          for (int u = 0; u < 2; ++u)
#pragma unroll
            for (int h8 = 0; h8 < 2; ++h8) {
              uint4 v;
              __nv_bfloat162 t0 = __floats2bfloat162_rn(t[u][h8 * 8] * inv, t[u][h8 * 8 + 1] * inv),
                             t1 = __floats2bfloat162_rn(t[u][h8 * 8 + 2] * inv, t[u][h8 * 8 + 3] * inv),
                             t2 = __floats2bfloat162_rn(t[u][h8 * 8 + 4] * inv, t[u][h8 * 8 + 5] * inv),
                             t3 = __floats2bfloat162_rn(t[u][h8 * 8 + 6] * inv, t[u][h8 * 8 + 7] * inv);
              v.x = *reinterpret_cast<unsigned *>(&t0);
              v.y = *reinterpret_cast<unsigned *>(&t1);
              v.z = *reinterpret_cast<unsigned *>(&t2);
              v.w = *reinterpret_cast<unsigned *>(&t3);
              *reinterpret_cast<uint4 *>(dst + c0 + u * 16 + h8 * 8) = v;
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
                      float scale, int form, int *status, cudaStream_t stream) {
  using S = FtShape<D>;
  CUtensorMap map_q, map_k, map_v;
  int rc = get_map(q, n_tokens, (long long)n_heads * D, q_stride, 64, &map_q);
  if (rc != LLM_OK) return rc;
  rc = get_map(kc, n_pages * n_kv * FT_BN, D, D, 64, &map_k);
  if (rc != LLM_OK) return rc;
  rc = get_map(vc, n_pages * n_kv * FT_BN, D, D, 64, &map_v);
  if (rc != LLM_OK) return rc;
  // Measured: at head size 128 the wide form is ahead from 256 rows on (4 prompts of 2,048: 200 against
  // 206 us, one of 8,192: 539 against 607); at head size 64 only for long prompts (one of 8,192: 430
  // against 468 us, 8 of 2,048: 278 against 282, 8 of 512: 46 against 44; and inside a whole prompt
  // step of 2,048 tokens it is 6 us a layer behind, alone on its SM with all of tensor memory).
  if (form == 2 || (form == 0 && max_q_len > (D == 64 ? 2048 : FT_BM))) {
    using W = FwShape<D>;
    auto kern = attention_prefill_wide_kernel<D>;
    LLM_CHECK_CUDA(llm_allow_smem(kern, W::SMEM), "attention_prefill_tc attribute");
    dim3 grid(n_heads, n_seqs, (max_q_len + FW_BM - 1) / FW_BM);
    LLM_CHECK_CUDA(llm_launch(kern, grid, dim3(FW_THREADS), W::SMEM, stream, map_q, map_k, map_v, (__nv_bfloat16 *)out,
                              out_stride, seq_start, seq_past, page_table, pt_stride, n_heads, n_kv, window,
                              scale * 1.4426950408889634f, status),
                   "attention_prefill_tc launch");
    return LLM_OK;
  }
  auto kern = attention_prefill_tc_kernel<D>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, S::SMEM), "attention_prefill_tc attribute");
  dim3 grid(n_heads, n_seqs, (max_q_len + FT_BM - 1) / FT_BM);
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
// int, may be null) receives a non-zero code if a wait inside the kernel ran out of time.  `form`: 0 the
// library chooses (the wide form when a sequence brings more than 128 rows), 1 CTAs of 128 rows, 2 of 256.
LLM_EXPORT int llm_attention_prefill_tc(const void *q, long long q_stride, long long n_tokens, void *out,
                                        long long out_stride, const void *kc, const void *vc, long long n_pages,
                                        const int *seq_start, const int *seq_past, const int *page_table,
                                        int pt_stride, int n_seqs, int max_q_len, int n_heads, int n_kv, int d,
                                        int page_size, int window, float scale, int form, int *status,
                                        cudaStream_t stream) {
  if (n_seqs == 0 || max_q_len == 0) return LLM_OK;
  LLM_REQUIRE(form >= 0 && form <= 2, "attention_prefill_tc: form %d is not one of 0, 1, 2", form);
  LLM_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && n_heads > 0 && n_heads <= 65535 && n_kv > 0 && n_heads % n_kv == 0,
              "attention_prefill_tc: bad sizes (%d sequences, %d heads, %d kv heads)", n_seqs, n_heads, n_kv);
  LLM_REQUIRE(max_q_len > 0 && max_q_len <= 65535 * 128, "attention_prefill_tc: %d tokens of one sequence in a step", max_q_len);
  LLM_REQUIRE(llm_attention_prefill_tc_supports(d, page_size),
              "attention_prefill_tc: head size %d with pages of %d tokens is not built (64 or 128, pages of 64)", d, page_size);
  LLM_REQUIRE(q_stride % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)kc % 16 == 0 && (uintptr_t)vc % 16 == 0 &&
                  out_stride % 8 == 0 && (uintptr_t)out % 16 == 0,
              "attention_prefill_tc: rows must be 16-byte aligned");
  LLM_REQUIRE(n_pages * n_kv * FT_BN < (1ll << 31), "attention_prefill_tc: the cache has too many rows for one tensor map");
  if (d == 64)
    return launch_prefill_tc<64>(q, q_stride, n_tokens, out, out_stride, kc, vc, n_pages, seq_start, seq_past, page_table,
                                 pt_stride, n_seqs, max_q_len, n_heads, n_kv, window, scale, form, status, stream);
  return launch_prefill_tc<128>(q, q_stride, n_tokens, out, out_stride, kc, vc, n_pages, seq_start, seq_past, page_table,
                                pt_stride, n_seqs, max_q_len, n_heads, n_kv, window, scale, form, status, stream);
}
