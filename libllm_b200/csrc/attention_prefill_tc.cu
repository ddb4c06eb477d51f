// Causal grouped-query attention for prompt steps on the 5th-generation tensor cores: the flash
// form (running maximum and sum per query row, scores never stored) with both products as
// tcgen05.mma, their accumulators in tensor memory and all operands brought by TMA.
//
// One CTA takes 128 query rows of one head of one sequence.  Its warps:
//   warp 0    one lane loads the Q tile once and then, page by page, the K and V tiles (a page of
//             the cache is a [64, d] block = one key tile) into a ring of shared-memory stages;
//   warp 1    one lane issues S = Q K^T (operands K-major, 128-byte swizzle) into tensor memory and,
//             when the probabilities are ready, O_j = P V_j (V is the MN-major operand: it lies
//             [key][channel] in the cache and is used as it is) into a second accumulator;
//   warps 2-5 a thread per query row: reads its row of S from tensor memory (no shuffles: the row is
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

constexpr int FT_THREADS = 192;
constexpr int FT_BM = 128;          // query rows per CTA
constexpr int FT_BN = 64;           // keys per tile = tokens per page

template <int D>
struct FtShape {
  static constexpr int KB = D / 64;                         // 64-wide blocks of the head size
  static constexpr int Q_BYTES = FT_BM * D * 2;
  static constexpr int KV_BYTES = FT_BN * D * 2;            // one of K or V
  static constexpr int P_BYTES = FT_BM * FT_BN * 2;
  static constexpr int STAGES = D == 64 ? 4 : 2;
  static constexpr int TMEM_COLS = D == 64 ? 128 : 256;     // S (64 columns) + O_j (D columns), a power of two
  static constexpr size_t SMEM = 1024 + Q_BYTES + P_BYTES + (size_t)STAGES * 2 * KV_BYTES + 256;
};


// MN-major operand descriptor: the tile lies [k][64 channels] in 128-byte swizzled rows, 8 rows of k
// per 1024 bytes (checked on the device: 16 k further = 2048 bytes further).
__device__ __forceinline__ unsigned long long smem_desc_mn(unsigned addr) { return smem_desc(addr); }

__host__ __device__ constexpr unsigned instr_desc_mn(int m, int n) { return instr_desc(m, n) | (1u << 16); }

template <int D>
__global__ void __launch_bounds__(FT_THREADS, D == 64 ? 2 : 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16 *__restrict__ out,
                            long long out_stride, const int *__restrict__ seq_start, const int *__restrict__ seq_past,
                            const int *__restrict__ page_table, int pt_stride, int n_heads, int n_kv, int window,
                            float scale_log2, int *status) {
  using S = FtShape<D>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char *sQ = smem, *sP = smem + S::Q_BYTES, *sKV = sP + S::P_BYTES;
  unsigned long long *bars = (unsigned long long *)(sKV + (size_t)STAGES * 2 * S::KV_BYTES);
  // full[STAGES], empty[STAGES], q_full, s_full, s_free, p_full, o_full, o_free
  const unsigned bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const unsigned bar_q = smem_u32(bars + 2 * STAGES), bar_sfull = bar_q + 8, bar_sfree = bar_q + 16,
                 bar_pfull = bar_q + 24, bar_ofull = bar_q + 32, bar_ofree = bar_q + 40;
  unsigned *tmem_slot = (unsigned *)(bars + 2 * STAGES + 6);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  grid_dependents_launch();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_q, 1);
    mbar_init(bar_sfull, 1);
    mbar_init(bar_sfree, 4);
    mbar_init(bar_pfull, 4);
    mbar_init(bar_ofull, 1);
    mbar_init(bar_ofree, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((unsigned)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;
  const unsigned tmem_s = tmem_base, tmem_o = tmem_base + FT_BN;

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

  if (warp == 0) {
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
  } else if (warp == 1) {
    // ------------------------------------------------------------ tensor-core issue
    if (lane == 0 && n_tiles > 0) {
      constexpr unsigned IDESC_S = instr_desc(FT_BM, FT_BN);          // S[128 x 64 keys], both operands K-major
      constexpr unsigned IDESC_O = instr_desc_mn(FT_BM, 64);          // O_j[128 x 64 channels], V MN-major
      bool ok = mbar_wait(bar_q, 0, abort_flag, status, 12);
      auto issue_s = [&](int j) {                                      // scores of tile j from its stage
        const int stage = j % STAGES;
        const unsigned ka = smem_u32(sKV + (size_t)stage * 2 * S::KV_BYTES);
#pragma unroll
        for (int kb = 0; kb < S::KB; ++kb)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            tc_mma(tmem_s, smem_desc(smem_u32(sQ) + kb * (FT_BM * 128) + kk * 32),
                   smem_desc(ka + kb * (FT_BN * 128) + kk * 32), IDESC_S, (kb > 0 || kk > 0) ? 1u : 0u);
        tc_commit(bar_sfull);
      };
      if (ok) ok = mbar_wait(bar_full, 0, abort_flag, status, 13);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          // the next tile's scores as soon as the row threads have taken this tile's out of tensor memory
          const int s1 = (j + 1) % STAGES;
          ok = mbar_wait(bar_full + 8 * s1, ((j + 1) / STAGES) & 1, abort_flag, status, 14) &&
               mbar_wait(bar_sfree, j & 1, abort_flag, status, 15);
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
  } else {
    // ------------------------------------------------------------ a thread per query row
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                       // row of the tile = lane of tensor memory
    const unsigned lane_addr = (unsigned)(quarter * 32) << 16;
    const int pos = past + r0 + row;                           // the row's position in its sequence
    float o[D];
#pragma unroll
    for (int c = 0; c < D; ++c) o[c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_sfull, j & 1, abort_flag, status, 18));
      if (!ok) break;
      tc_fence_after();
      float s[FT_BN];
#pragma unroll
      for (int c0 = 0; c0 < FT_BN; c0 += 16) tc_ld16(tmem_s + lane_addr + c0, *reinterpret_cast<float(*)[16]>(&s[c0]));
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sfree);                   // the scores are in registers
      const int k0 = (first_tile + j) * FT_BN;
      const bool edge = (k0 + FT_BN - 1 > past + r0) || (window > 0 && k0 <= past + r0 + FT_BM - 1 - window);
      if (edge) {
#pragma unroll
        for (int c = 0; c < FT_BN; ++c) {
          const int key = k0 + c;
          if (!(key <= pos && (window <= 0 || key > pos - window))) s[c] = -INFINITY;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < FT_BN; ++c) mx = fmaxf(mx, s[c]);
      const float m_new = fmaxf(m_run, mx);
      const float moff = m_new == -INFINITY ? 0.f : m_new * scale_log2;
      const float alpha = m_run == -INFINITY ? 0.f : exp2f(m_run * scale_log2 - moff);
      m_run = m_new;
      float sum = 0.f;
      // the row of P, 16 bytes (8 keys) at a time, where the tensor core expects it: row r lies at
      // (r / 8) * 1024 + (r % 8) * 128, its 16-byte piece c at piece c ^ (r % 8)
      unsigned char *prow = sP + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
      for (int c8 = 0; c8 < FT_BN / 8; ++c8) {
        float p[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          p[i] = exp2f(fmaf(s[c8 * 8 + i], scale_log2, -moff));
          sum += p[i];
        }
        uint4 v;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(p[0], p[1]), t1 = __floats2bfloat162_rn(p[2], p[3]),
                       t2 = __floats2bfloat162_rn(p[4], p[5]), t3 = __floats2bfloat162_rn(p[6], p[7]);
        v.x = *reinterpret_cast<unsigned *>(&t0);
        v.y = *reinterpret_cast<unsigned *>(&t1);
        v.z = *reinterpret_cast<unsigned *>(&t2);
        v.w = *reinterpret_cast<unsigned *>(&t3);
        *reinterpret_cast<uint4 *>(prow + ((c8 ^ (row & 7)) << 4)) = v;
      }
      l_run = l_run * alpha + sum;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is for the tensor core to read
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pfull);
      // this tile's part of the output, when the tensor core has it
      ok = __all_sync(0xffffffffu, mbar_wait(bar_ofull, j & 1, abort_flag, status, 19));
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 16) {
        float v[16];
        tc_ld16(tmem_o + lane_addr + c0, v);
#pragma unroll
        for (int i = 0; i < 16; ++i) o[c0 + i] = fmaf(o[c0 + i], alpha, v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ofree);
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
  if (warp == 1) {
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
