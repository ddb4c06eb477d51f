// Causal grouped-query attention for prompt steps on the 5th-generation tensor cores: the flash
// form (running maximum and sum per query row, scores never stored) with both products as
// tcgen05.mma, their accumulators in tensor memory and all operands brought by TMA.
//
// One CTA takes 128 query rows of one head of one sequence.  Its warps:
//   warp 4    one lane loads the Q tile once and then, page by page, the K and V tiles (a page of
//             the cache is a [64, d] block = one key tile) into a ring of shared-memory stages;
//   warp 5    one lane issues S = Q K^T (operands K-major, 128-byte swizzle) into tensor memory and,
//             when the probabilities are ready, O_j = P V_j (V is the MN-major operand: it lies
//             [key][channel] in the cache and is used as it is) into a second accumulator;
//   warps 0-3 a thread per query row: reads its row of S from tensor memory (no shuffles: the row is
//             one lane), masks, keeps the running maximum and sum in 32-bit, writes the row of P as
//             bfloat16 into shared memory in the swizzled layout the tensor core reads, then adds
//             O_j to its output row scaled by exp(old maximum - new maximum).
// The score product of the next tile is issued as soon as the row threads have taken the current
// scores out of tensor memory, so it runs under their exponentials; a second CTA on the same SM fills
// the rest.  Exponentials are exp2 of scores pre-scaled by log2(e) / sqrt(d).
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

constexpr int FT_THREADS = 256;   // warps 0-3: a thread per query row; 4: loader; 5: tensor-core issue; 6, 7: none
constexpr int FT_BM = 128;          // query rows per CTA
constexpr int FT_BN = 64;           // keys per tile = tokens per page

template <int D>
struct FtShape {
  static constexpr int KB = D / 64;                         // 64-wide blocks of the head size
  static constexpr int Q_BYTES = FT_BM * D * 2;
  static constexpr int KV_BYTES = FT_BN * D * 2;            // one of K or V
  static constexpr int P_BYTES = FT_BM * FT_BN * 2;
  static constexpr int STAGES = D == 64 ? 4 : 2;
  static constexpr int TMEM_COLS = 256;                     // two S buffers (64 columns each) + O_j (D columns)
  static constexpr size_t SMEM = Q_BYTES + P_BYTES + (size_t)STAGES * 2 * KV_BYTES + 256;   // two CTAs per SM
  // Registers move from the second warpgroup (loader, issuer) to the first (the row threads), which
  // keep a row of the output and a row of scores each: 2 CTAs x 256 threads x 128 registers at launch.
  static constexpr int REGS_FEW = 56, REGS_MANY = 256 - REGS_FEW;
};


// MN-major operand descriptor: the tile lies [k][64 channels] in 128-byte swizzled rows, 8 rows of k
// per 1024 bytes (checked on the device: 16 k further = 2048 bytes further).
__device__ __forceinline__ unsigned long long smem_desc_mn(unsigned addr) { return smem_desc(addr); }

__host__ __device__ constexpr unsigned instr_desc_mn(int m, int n) { return instr_desc(m, n) | (1u << 16); }

// exp2 of a number that is never above zero here: one instruction (inputs of -inf give 0)
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
  unsigned char *sQ = smem, *sP = smem + S::Q_BYTES, *sKV = sP + S::P_BYTES;
  unsigned long long *bars = (unsigned long long *)(sKV + (size_t)STAGES * 2 * S::KV_BYTES);
  // full[STAGES], empty[STAGES], q_full, s_full[2] (one per score buffer), p_full, o_full, o_free
  const unsigned bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const unsigned bar_q = smem_u32(bars + 2 * STAGES), bar_sfull = bar_q + 8,
                 bar_pfull = bar_q + 24, bar_ofull = bar_q + 32, bar_ofree = bar_q + 40;
  unsigned *tmem_slot = (unsigned *)(bars + 2 * STAGES + 6);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  grid_dependents_launch();
  if (smem_u32(smem) & 1023u) {                               // swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(status, 0, 21);
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
    mbar_init(bar_pfull, 4);
    mbar_init(bar_ofull, 1);
    mbar_init(bar_ofree, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
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

  if (warp >= 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(S::REGS_FEW));
  if (warp == 4) {
    // ------------------------------------------------------------ loader
    if (lane == 0 && n_tiles > 0) {
      mbar_expect_tx(bar_q, S::Q_BYTES);
      for (int kb = 0; kb < S::KB; ++kb) {
        tma_load_2d(smem_u32(sQ) + kb * (FT_BM * 128), &map_q, h * D + kb * 64, q0 + r0, bar_q);
        tma_load_2d(smem_u32(sQ) + kb * (FT_BM * 128) + 64 * 128, &map_q, h * D + kb * 64, q0 + r0 + 64, bar_q);
      }
      int stage = 0;
      unsigned phase = 0;
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, status, 11);
        if (!ok) break;
        const int row = (pt[first_tile + j] * n_kv + kvh) * FT_BN;
        const unsigned dk = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES), dv = dk + S::KV_BYTES;
        mbar_expect_tx(bar_full + 8 * stage, 2 * S::KV_BYTES);
        for (int kb = 0; kb < S::KB; ++kb) {
          tma_load_2d(dk + kb * (FT_BN * 128), &map_k, kb * 64, row, bar_full + 8 * stage);
          tma_load_2d(dv + kb * (FT_BN * 128), &map_v, kb * 64, row, bar_full + 8 * stage);
        }
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok || *abort_flag) {
        const unsigned long long t0 = globaltimer();
        for (int s = 0; s < STAGES; ++s)
          while (!mbar_try(bar_full + 8 * s, 0) && !mbar_try(bar_full + 8 * s, 1) && globaltimer() - t0 < 2000000ull) {
          }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------ tensor-core issue
    if (lane == 0 && n_tiles > 0) {
      constexpr unsigned IDESC_S = instr_desc(FT_BM, FT_BN);          // S[128 x 64 keys], both operands K-major
      constexpr unsigned IDESC_O = instr_desc_mn(FT_BM, 64);          // O_j[128 x 64 channels], V MN-major
      bool ok = mbar_wait(bar_q, 0, abort_flag, status, 12);
      auto issue_s = [&](int j) {                                      // scores of tile j into buffer j & 1
        const int stage = j % STAGES;
        const unsigned ka = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < S::KB; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma(tmem_s + (j & 1) * FT_BN, smem_desc(smem_u32(sQ) + kb * (FT_BM * 128) + kk * 32),
                   smem_desc(ka + kb * (FT_BN * 128) + kk * 32), IDESC_S, (kb > 0 || kk > 0) ? 1u : 0u);
        tc_commit(bar_sfull + 8 * (j & 1));
      };
      if (ok) ok = mbar_wait(bar_full, 0, abort_flag, status, 13);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          // The next tile's scores go into the other buffer at once: its last reader was tile
          // j - 1, whose probabilities this thread has already waited for.
          const int s1 = (j + 1) % STAGES;
          ok = mbar_wait(bar_full + 8 * s1, ((j + 1) / STAGES) & 1, abort_flag, status, 14);
          if (!ok) break;
          tc_fence_after();
          issue_s(j + 1);
        }
        ok = mbar_wait(bar_pfull, j & 1, abort_flag, status, 16) &&
             mbar_wait(bar_ofree, (j & 1) ^ 1, abort_flag, status, 17);
        if (!ok) break;
        tc_fence_after();
        const int stage = j % STAGES;
        const unsigned va = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES) + S::KV_BYTES;
#pragma unroll
        for (int nb = 0; nb < S::KB; ++nb)           // 64 channels at a time
#pragma unroll
          for (int kk = 0; kk < FT_BN / 16; ++kk)    // 16 keys: 32 bytes along P's rows, 16 rows of V
            tc_mma(tmem_o + nb * 64, smem_desc(smem_u32(sP) + kk * 32),
                   smem_desc_mn(va + nb * (FT_BN * 128) + kk * 2048), IDESC_O, kk > 0 ? 1u : 0u);
        tc_commit(bar_ofull);
        tc_commit(bar_empty + 8 * stage);
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------ a thread per query row
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(S::REGS_MANY));
    const int quarter = warp;
    const int row = quarter * 32 + lane;                       // row of the tile = lane of tensor memory
    const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
    const int pos = past + r0 + row;                           // the row's position in its sequence
    float o[D];
#pragma unroll
    for (int c = 0; c < D; ++c) o[c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;
    bool ok = true;
    // o = o * a + (the tile's product in tensor memory), OB * 16 channels with OB loads in flight
    constexpr int OB = D == 64 ? 4 : 2;
    auto add_output = [&](float a) {
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += OB * 16) {
        float t[OB][16];
#pragma unroll
        for (int c = 0; c < OB; ++c) tc_ld16_issue(tmem_o + lane_addr + c0 + c * 16, t[c]);
        tc_ld_wait();
#pragma unroll
        for (int c = 0; c < OB; ++c) tc_ld_ready(t[c]);
#pragma unroll
        for (int c = 0; c < OB; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i) o[c0 + c * 16 + i] = fmaf(o[c0 + c * 16 + i], a, t[c][i]);
      }
    };
    for (int j = 0; j < n_tiles && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_sfull + 8 * (j & 1), (j >> 1) & 1, abort_flag, status, 18));
      if (!ok) break;
      tc_fence_after();
      const unsigned s_addr = tmem_s + (j & 1) * FT_BN + lane_addr;
      const int k0 = (first_tile + j) * FT_BN;
      const bool edge = (k0 + FT_BN - 1 > past + r0) || (window > 0 && k0 <= past + r0 + FT_BM - 1 - window);
      // The row's scores come into registers NB * 16 at a time, with NB loads in flight and one wait.
      // A head size of 64 leaves room for the whole row (NB = 4), which is then read once; a larger
      // one reads it twice, first for the maximum and then for the exponentials.
      constexpr int NB = D == 64 ? 4 : 2;
      auto load_scores = [&](int c0, float (&v)[NB][16]) {
#pragma unroll
        for (int c = 0; c < NB; ++c) tc_ld16_issue(s_addr + c0 + c * 16, v[c]);
        tc_ld_wait();
#pragma unroll
        for (int c = 0; c < NB; ++c) tc_ld_ready(v[c]);
        if (edge) {
#pragma unroll
          for (int c = 0; c < NB; ++c)
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int key = k0 + c0 + c * 16 + i;
              if (!(key <= pos && (window <= 0 || key > pos - window))) v[c][i] = -INFINITY;
            }
        }
      };
      // exponentials of NB * 16 scores and their pieces of the row of P, 16 bytes (8 keys) at a time,
      // where the tensor core expects it: row r lies at (r / 8) * 1024 + (r % 8) * 128, its 16-byte
      // piece c at piece c ^ (r % 8)
      unsigned char *prow = sP + (row >> 3) * 1024 + (row & 7) * 128;
      float sum = 0.f;
      auto write_p = [&](int c0, float (&v)[NB][16], float moff) {
#pragma unroll
        for (int c = 0; c < NB; ++c) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            v[c][i] = fast_exp2(fmaf(v[c][i], scale_log2, -moff));
            sum += v[c][i];
          }
#pragma unroll
          for (int h8 = 0; h8 < 2; ++h8) {
            uint4 w;
            __nv_bfloat162 t0 = __floats2bfloat162_rn(v[c][h8 * 8], v[c][h8 * 8 + 1]),
                           t1 = __floats2bfloat162_rn(v[c][h8 * 8 + 2], v[c][h8 * 8 + 3]),
                           t2 = __floats2bfloat162_rn(v[c][h8 * 8 + 4], v[c][h8 * 8 + 5]),
                           t3 = __floats2bfloat162_rn(v[c][h8 * 8 + 6], v[c][h8 * 8 + 7]);
            w.x = *reinterpret_cast<unsigned *>(&t0);
            w.y = *reinterpret_cast<unsigned *>(&t1);
            w.z = *reinterpret_cast<unsigned *>(&t2);
            w.w = *reinterpret_cast<unsigned *>(&t3);
            *reinterpret_cast<uint4 *>(prow + ((((c0 >> 3) + c * 2 + h8)) ^ (row & 7)) * 16) = w;
          }
        }
      };
      float sc[NB][16];
      float mx = -INFINITY;
#pragma unroll
      for (int c0 = 0; c0 < FT_BN; c0 += NB * 16) {
        load_scores(c0, sc);
#pragma unroll
        for (int c = 0; c < NB; ++c)
#pragma unroll
          for (int i = 0; i < 16; ++i) mx = fmaxf(mx, sc[c][i]);
      }
      const float m_new = fmaxf(m_run, mx);
      const float moff = m_new == -INFINITY ? 0.f : m_new * scale_log2;
      const float alpha = m_run == -INFINITY ? 0.f : fast_exp2(m_run * scale_log2 - moff);
      m_run = m_new;
      // The buffer of P is free when the tensor core has finished the previous tile's product,
      // which ran while this tile's maximum was being found.
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_ofull, (j - 1) & 1, abort_flag, status, 19));
        if (!ok) break;
      }
      if (NB * 16 == FT_BN) {
        write_p(0, sc, moff);
      } else {
#pragma unroll
        for (int c0 = 0; c0 < FT_BN; c0 += NB * 16) {
          load_scores(c0, sc);
          write_p(c0, sc, moff);
        }
      }
      l_run = l_run * alpha + sum;
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is for the tensor core to read
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull);
      // the previous tile's part of the output, while the tensor core works on this tile's
      if (j > 0) {
        tc_fence_after();
        add_output(alpha_prev);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ofree);
      }
      alpha_prev = alpha;
    }
    if (ok && n_tiles > 0) {                          // the last tile's part
      ok = __all_sync(0xffffffffu, mbar_wait(bar_ofull, (n_tiles - 1) & 1, abort_flag, status, 20));
      if (ok) {
        tc_fence_after();
        add_output(alpha_prev);
        tc_fence_before();
      }
    }
    if (ok && row < rows) {
      const float inv = 1.f / l_run;
      __nv_bfloat16 *dst = out + (size_t)(q0 + r0 + row) * out_stride + (size_t)h * D;
#pragma unroll
      for (int c8 = 0; c8 < D / 8; ++c8) {
        uint4 v;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(o[c8 * 8] * inv, o[c8 * 8 + 1] * inv),
                       t1 = __floats2bfloat162_rn(o[c8 * 8 + 2] * inv, o[c8 * 8 + 3] * inv),
                       t2 = __floats2bfloat162_rn(o[c8 * 8 + 4] * inv, o[c8 * 8 + 5] * inv),
                       t3 = __floats2bfloat162_rn(o[c8 * 8 + 6] * inv, o[c8 * 8 + 7] * inv);
        v.x = *reinterpret_cast<unsigned *>(&t0);
        v.y = *reinterpret_cast<unsigned *>(&t1);
        v.z = *reinterpret_cast<unsigned *>(&t2);
        v.w = *reinterpret_cast<unsigned *>(&t3);
        *reinterpret_cast<uint4 *>(dst + c8 * 8) = v;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
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
