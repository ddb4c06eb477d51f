// Matrix product on the 5th-generation tensor cores: out[M, N] = x[M, K] * W[N, K]^T, bfloat16
// operands, 32-bit accumulation in tensor memory, optional fused SwiGLU and partial products
// over parts of K.  One kernel serves a decoding step of a few tokens, where it streams W once
// from HBM, and a prompt step of thousands.
//
// W's rows are the 128-row operand of tcgen05.mma and the tokens its N operand ("swap AB"): the
// accumulator of a tile is D[128 rows of W][TN tokens] with TN = 16 .. 256, so that a step of 8
// tokens costs no more than one of 16 and the instruction shape is full at any batch.  A CTA is
// persistent (one per SM) and walks over its tiles with three kinds of warps:
//   warp 0   one lane issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of [64 rows x 64 k]
//            boxes of W and a [TN x 64 k] box of x into a ring of shared-memory stages;
//   warp 1   allocates tensor memory; one lane issues tcgen05.mma (four k-steps of 16 per stage)
//            and commits each stage back to the loader and each finished tile to the epilogue;
//   warps 2-5 read the accumulator with tcgen05.ld (each warp its quarter of the 128 lanes),
//            apply the epilogue and store out[token][row], while the next tile's products run
//            into the other accumulator buffer.
// 90 KB (few tokens) to 200 KB (prompts) of loads are in flight per SM, which is what a stream from
// HBM needs.
//
// SwiGLU: W is the stacked gate|up matrix [2I, K].  A tile holds gate rows f..f+63 in its lanes
// 0-63 and up rows I+f..I+f+63 in lanes 64-127; the epilogue warps of the upper half hand their
// values over through shared memory and the lower half stores silu(gate) * up: the stacked
// product never reaches memory (the reference runs a separate launch, src/flint/cuda/swiglu.cu:29-59,
// after cuBLAS, src/flint/cuda/gemm_cublas.cc:160-197).
//
// Rows of W, tokens and K beyond the matrices are zero-filled by TMA and never stored, so every
// size is taken (K a multiple of 8: rows must start on 16 bytes).  Every wait on a barrier has a
// time limit; when it runs out the CTA records a code in `status`, waits for its loads in flight,
// frees its tensor memory and returns.  Weights are loaded before the programmatic dependency on
// the previous kernel is waited for, tokens after it.
#include "common.cuh"
#include "tc_common.cuh"

LLM_DEFINE_LAST_ERROR(llm_gemm_tc_last_error)

namespace {

constexpr int TC_THREADS = 192;
constexpr int TC_ROWS = 128;                   // rows of W per tile (UMMA M)
constexpr int TC_A_BYTES = TC_ROWS * TC_BK * 2;

// SW: 0 plain product; 1 SwiGLU with gate and up rows interleaved in one 128-row tile (64 + 64,
// handed over between epilogue warps: steps of few tokens, where a tile per SM matters); 2 SwiGLU with
// a tile of 128 gate rows and one of 128 up rows per stage and an accumulator for each, so that a
// lane holds both values of a feature (prompt steps).
template <int TN, int SW>
struct TcShape {
  static constexpr int A_TILES = SW == 2 ? 2 : 1;
  static constexpr int A_BYTES = A_TILES * TC_A_BYTES;
  static constexpr int B_BYTES = TN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // Steps of few tokens (TN <= 32) take half of an SM's shared memory, so that the CTA of the next
  // product in the stream can move in beside this one and fill its ring with weights while this
  // one finishes; larger steps take a ring as deep as fits (measured: equal at 1 and 8 tokens,
  // 5 % faster at 64 with the deep ring).
  static constexpr int BUDGET = TN <= 32 ? 100 * 1024 : 200 * 1024;
  static constexpr int STAGES = BUDGET / STAGE_BYTES;
  static constexpr int ACC_COLS = A_TILES * TN;                          // columns of one accumulator buffer
  static constexpr int TMEM_COLS = 2 * ACC_COLS < 32 ? 32 : 2 * ACC_COLS;  // two buffers; a power of two
  static constexpr int XCH_BYTES = 64 * 17 * 4;                        // SwiGLU hand-over: 64 rows x 16 tokens (+1 pad)
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + XCH_BYTES + 256;
  static_assert(TMEM_COLS <= 512, "the accumulators do not fit tensor memory");
};

template <int TN, int SW, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               TO *__restrict__ out, long long ldo, int M, int n_out, int K, int row_tiles, int tok_tiles,
               int k_parts, int kb_per_part, long long part_stride, int *status) {
  using S = TcShape<TN, SW>;
  constexpr bool SWIGLU = SW == 1;                      // the interleaved tile with the hand-over
  constexpr int STAGES = S::STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char *xch_raw = smem + (size_t)STAGES * S::STAGE_BYTES;
  unsigned long long *bars = (unsigned long long *)(xch_raw + S::XCH_BYTES);
  // bars: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], hand-over full and empty;
  // then the TMEM address and the abort flag
  const unsigned bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const unsigned bar_tfull = smem_u32(bars + 2 * STAGES), bar_tempty = smem_u32(bars + 2 * STAGES + 2);
  const unsigned bar_xfull = smem_u32(bars + 2 * STAGES + 4), bar_xempty = smem_u32(bars + 2 * STAGES + 5);
  unsigned *tmem_slot = (unsigned *)(bars + 2 * STAGES + 6);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);

  // The warp's number comes out of a shuffle so that the compiler knows it is the same in all of
  // a warp's lanes: the loader's and the issuer's loops then run in all 32 lanes (address and
  // descriptor arithmetic in the uniform datapath), and only the copy, product and commit
  // instructions themselves are one lane's.  Issued from inside a one-lane branch, a product cost
  // about 115 cycles of that lane, more than it takes the tensor core at 16 to 128 tokens.
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  grid_dependents_launch();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 4);
    }
    mbar_init(bar_xfull, 2);
    mbar_init(bar_xempty, 2);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
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

  const int n_tiles = row_tiles * tok_tiles * k_parts;
  const int n_kblocks_total = (K + TC_BK - 1) / TC_BK;
  constexpr int ROWS_OUT = SW == 1 ? 64 : 128;             // output features per tile

  if (warp == 0) {
    // ------------------------------------------------------------ loader
    const bool leader = elect_one();
    // The walk over this CTA's (tile, k block) pairs, one per stage filled.
    struct Walk {
      int tile, kb, kb1, tok_tile, row_a, row_b;
      bool valid;
    };
    auto start = [&](Walk &w, int tile) {
      w.tile = tile;
      w.valid = tile < n_tiles;
      if (!w.valid) return;
      const int part = tile % k_parts, row_tile = tile / (k_parts * tok_tiles);
      w.tok_tile = (tile / k_parts) % tok_tiles;
      w.kb = part * kb_per_part;
      w.kb1 = min(n_kblocks_total, w.kb + kb_per_part);
      w.row_a = row_tile * ROWS_OUT;
      w.row_b = SW != 0 ? n_out + w.row_a : w.row_a + 64;
    };
    auto next = [&](Walk &w) {
      if (++w.kb >= w.kb1) start(w, w.tile + gridDim.x);
    };
    auto load_w = [&](const Walk &w, int stage) {
      const unsigned dst = smem_u32(smem + (size_t)stage * S::STAGE_BYTES);
      if (leader) {
        mbar_expect_tx(bar_full + 8 * stage, S::STAGE_BYTES);
        if (SW == 2) {                    // 128 gate rows, then 128 up rows: the map's boxes are 128 rows here
          tma_load_2d(dst, &map_w, w.kb * TC_BK, w.row_a, bar_full + 8 * stage);
          tma_load_2d(dst + TC_A_BYTES, &map_w, w.kb * TC_BK, w.row_b, bar_full + 8 * stage);
        } else {
          tma_load_2d(dst, &map_w, w.kb * TC_BK, w.row_a, bar_full + 8 * stage);
          tma_load_2d(dst + TC_A_BYTES / 2, &map_w, w.kb * TC_BK, w.row_b, bar_full + 8 * stage);
        }
      }
    };
    auto load_x = [&](const Walk &w, int stage) {
      if (leader)
        tma_load_2d(smem_u32(smem + (size_t)stage * S::STAGE_BYTES) + S::A_BYTES, &map_x, w.kb * TC_BK,
                    w.tok_tile * TN, bar_full + 8 * stage);
    };
    // Weights first: they do not depend on the kernel before this one, so the whole ring
    // is filled with them while that kernel still runs.  Then the wait, then the tokens of
    // the same stages, then the rest of the walk stage by stage.
    Walk w, w2;
    start(w, blockIdx.x);
    int n_pre = 0;
    for (; w.valid && n_pre < STAGES; next(w), ++n_pre) load_w(w, n_pre);
    start(w2, blockIdx.x);
    grid_dependency_wait();
    for (int s = 0; s < n_pre; ++s, next(w2)) load_x(w2, s);
    int stage = n_pre % STAGES;
    unsigned phase = n_pre == STAGES ? 1u : 0u;
    bool ok = true;
    for (; w.valid; next(w)) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, status, 1));
      if (!ok) break;
      load_w(w, stage);
      load_x(w, stage);
      if (++stage == STAGES) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (leader && (!ok || *abort_flag)) {
      // given up: let the loads that are in flight land before the CTA goes away
      const unsigned long long t0 = globaltimer();
      for (int s = 0; s < STAGES; ++s)
        while (!mbar_try(bar_full + 8 * s, 0) && !mbar_try(bar_full + 8 * s, 1) && globaltimer() - t0 < 2000000ull) {
        }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ tensor-core issue
    const bool leader = elect_one();
    constexpr unsigned IDESC = instr_desc(TC_ROWS, TN);
    int stage = 0;
    unsigned phase = 0;
    int iter = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++iter) {
      const int part = tile % k_parts;
      const int kb0 = part * kb_per_part, kb1 = min(n_kblocks_total, kb0 + kb_per_part);
      const int acc = iter & 1;
      const unsigned acc_phase = (iter >> 1) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, status, 2));
      if (!ok) break;
      tc_fence_after();
      const unsigned d_tmem = tmem_base + acc * S::ACC_COLS;
      for (int kb = kb0; kb < kb1; ++kb) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, 3));
        if (!ok) break;
        tc_fence_after();
        const unsigned a_addr = smem_u32(smem + (size_t)stage * S::STAGE_BYTES);
        const unsigned long long a_desc = smem_desc(a_addr), b_desc = smem_desc(a_addr + S::A_BYTES);
        const unsigned long long a2_desc = smem_desc(a_addr + TC_A_BYTES);
        const unsigned first = kb > kb0 ? 1u : 0u;
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < TC_BK / 16; ++kk) {  // 16 k = 32 bytes further along the swizzled row
            tc_mma(d_tmem, a_desc + (unsigned long long)(kk * 2), b_desc + (unsigned long long)(kk * 2), IDESC,
                   kk > 0 ? 1u : first);
            if (SW == 2)                             // the up rows into the accumulator beside
              tc_mma(d_tmem + TN, a2_desc + (unsigned long long)(kk * 2), b_desc + (unsigned long long)(kk * 2), IDESC,
                     kk > 0 ? 1u : first);
          }
          tc_commit(bar_empty + 8 * stage);          // the stage is free when these products have read it
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && leader) tc_commit(bar_tfull + 8 * acc);      // the tile's accumulator is complete
      __syncwarp();
    }
    grid_dependency_wait();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    grid_dependency_wait();
    const int quarter = warp & 3;                    // the 32 lanes of tensor memory this warp may read
    float *xch = (float *)xch_raw;
    int iter = 0;
    unsigned n_chunk = 0;                            // hand-overs so far (SwiGLU)
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++iter) {
      const int part = tile % k_parts, tok_tile = (tile / k_parts) % tok_tiles, row_tile = tile / (k_parts * tok_tiles);
      const int acc = iter & 1;
      const unsigned acc_phase = (iter >> 1) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, status, 4));
      if (!ok) break;
      tc_fence_after();
      TO *o = out + (size_t)part * part_stride;
      const int row_in_tile = quarter * 32 + lane;
      const int tok0 = tok_tile * TN;
#pragma unroll 1
      for (int c0 = 0; c0 < TN && ok; c0 += 16, ++n_chunk) {
        float v[16];
        tc_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * S::ACC_COLS + c0), v);
        if (SW == 2) {
          float u[16];
          tc_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * S::ACC_COLS + TN + c0), u);
          const int f = row_tile * 128 + row_in_tile;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int tok = tok0 + c0 + i;
            const float g = v[i];
            if (f < n_out && tok < M) o[(size_t)tok * ldo + f] = from_float<TO>(g / (1.f + expf(-g)) * u[i]);
          }
        } else if (SWIGLU) {
          // The upper two warps (up rows) hand their values to the lower two (gate rows of the
          // same features) through shared memory; both directions are barriers with a time limit.
          if (quarter >= 2) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_xempty, (n_chunk & 1) ^ 1, abort_flag, status, 5));
            if (!ok) break;
#pragma unroll
            for (int i = 0; i < 16; ++i) xch[(row_in_tile - 64) * 17 + i] = v[i];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_xfull);
          } else {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_xfull, n_chunk & 1, abort_flag, status, 6));
            if (!ok) break;
            const int f = row_tile * 64 + row_in_tile;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int tok = tok0 + c0 + i;
              const float up = xch[row_in_tile * 17 + i];
              const float g = v[i];
              if (f < n_out && tok < M) o[(size_t)tok * ldo + f] = from_float<TO>(g / (1.f + expf(-g)) * up);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_xempty);
          }
        } else {
          const int f = row_tile * 128 + row_in_tile;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int tok = tok0 + c0 + i;
            if (f < n_out && tok < M) o[(size_t)tok * ldo + f] = from_float<TO>(v[i]);
          }
        }
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)S::TMEM_COLS)
                 : "memory");
  }
}

template <int TN, int SW, typename TO>
int launch_tc(const void *x, long long ldx, const void *W, void *out, long long ldo, int M, int N, int K, int k_parts,
              long long part_stride, int *status, cudaStream_t stream) {
  using S = TcShape<TN, SW>;
  const int n_out = SW != 0 ? N / 2 : N;
  const int rows_out = SW == 1 ? 64 : 128;
  const int row_tiles = (n_out + rows_out - 1) / rows_out;
  const int tok_tiles = (M + TN - 1) / TN;
  const int n_kblocks = (K + TC_BK - 1) / TC_BK;
  const int kb_per_part = (n_kblocks + k_parts - 1) / k_parts;
  LLM_REQUIRE((long long)(k_parts - 1) * kb_per_part < n_kblocks, "gemm_tc: %d parts leave one of them without work (K = %d)", k_parts, K);
  CUtensorMap map_w, map_x;
  int rc = get_map(W, N, K, K, SW == 2 ? 128 : 64, &map_w);
  if (rc != LLM_OK) return rc;
  rc = get_map(x, M, K, ldx, TN, &map_x);
  if (rc != LLM_OK) return rc;
  auto kern = gemm_tc_kernel<TN, SW, TO>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, S::SMEM), "gemm_tc attribute");
  const long long tiles = (long long)row_tiles * tok_tiles * k_parts;
  LLM_REQUIRE(tiles < (1ll << 30), "gemm_tc: too many tiles");
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  LLM_CHECK_CUDA(llm_launch(kern, dim3(grid), dim3(TC_THREADS), S::SMEM, stream, map_w, map_x, (TO *)out, ldo, M, n_out, K,
                            row_tiles, tok_tiles, k_parts, kb_per_part, part_stride, status),
                 "gemm_tc launch");
  return LLM_OK;
}

template <bool SWIGLU, typename TO>
int dispatch_tc(const void *x, long long ldx, const void *W, void *out, long long ldo, int M, int N, int K, int k_parts,
                long long part_stride, int *status, cudaStream_t stream) {
#define TC_GO(TN, SW) return launch_tc<TN, SW, TO>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, status, stream)
  if (SWIGLU) {
    if (M <= 16) TC_GO(16, 1);
    if (M <= 32) TC_GO(32, 1);
    if (M <= 64) TC_GO(64, 1);
    TC_GO(128, 2);
  }
  if (M <= 16) TC_GO(16, 0);
  if (M <= 32) TC_GO(32, 0);
  if (M <= 64) TC_GO(64, 0);
  if (M <= 128) TC_GO(128, 0);
  TC_GO(256, 0);
#undef TC_GO
}

}  // namespace

// How many parts of K a product with this few rows of W should be cut into so that most SMs have a
// tile; 1 when the matrix has tiles enough.  The caller adds the parts (32-bit) in order.
LLM_EXPORT int llm_gemm_tc_suggest_parts(int M, int N, int K) {
  const int tok_tiles = M <= 256 ? 1 : (M + 255) / 256;
  const int tiles = ((N + 127) / 128) * tok_tiles;
  const int kblocks = (K + TC_BK - 1) / TC_BK;
  // the most parts (up to 8) that still leave every SM at most one tile and every part at least
  // four K blocks, none of them empty
  // Above 32 tokens the parts themselves weigh (8 parts of 64 tokens x 2,048 features are 4 MB to
  // write and to read again): four at most (batch 64: 1.735 -> 1.687 ms a step; at 32 tokens eight
  // are still better, 1.297 against 1.350 ms).
  const int cap = M > 32 ? 4 : 8;
  const int most = sm_count() / (tiles > 0 ? tiles : 1) < cap ? sm_count() / (tiles > 0 ? tiles : 1) : cap;
  int parts = 1;
  for (int p = 2; p <= most; ++p) {
    const int per = (kblocks + p - 1) / p;
    if (per >= 4 && (p - 1) * per < kblocks) parts = p;
  }
  return parts;
}

// x [M, K] bfloat16 (row stride ldx elements), W [N, K] bfloat16 contiguous, out [M, N] of out_dtype,
// or [M, N/2] with swiglu (W = stacked gate|up).  With k_parts > 1 (plain product, 32-bit out) part p
// writes its share of K to out + p * part_stride.  `status` (device int, may be null) receives a
// non-zero code if a wait inside the kernel ran out of time.
LLM_EXPORT int llm_gemm_tc(const void *x, long long ldx, const void *W, void *out, long long ldo, int out_dtype,
                           int M, int N, int K, int swiglu, int k_parts, long long part_stride, int *status,
                           cudaStream_t stream) {
  if (M == 0 || N == 0) return LLM_OK;
  LLM_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes %d x %d x %d", M, N, K);
  LLM_REQUIRE(K % 8 == 0 && ldx % 8 == 0, "gemm_tc: K = %d and the row stride %lld must be multiples of 8 (rows start on 16 bytes)", K, ldx);
  LLM_REQUIRE((uintptr_t)x % 16 == 0 && (uintptr_t)W % 16 == 0, "gemm_tc: operands must be 16-byte aligned");
  LLM_REQUIRE(!swiglu || N % 2 == 0, "gemm_tc: a stacked gate|up matrix has an even number of rows");
  LLM_REQUIRE(k_parts >= 1 && k_parts <= 64 && (k_parts == 1 || (!swiglu && out_dtype == LLM_F32)),
              "gemm_tc: parts of K need a plain product with 32-bit output");
  if (swiglu) {
    if (out_dtype == LLM_BF16) return dispatch_tc<true, __nv_bfloat16>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, status, stream);
    if (out_dtype == LLM_F32) return dispatch_tc<true, float>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, status, stream);
  } else {
    if (out_dtype == LLM_BF16) return dispatch_tc<false, __nv_bfloat16>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, status, stream);
    if (out_dtype == LLM_F32) return dispatch_tc<false, float>(x, ldx, W, out, ldo, M, N, K, k_parts, part_stride, status, stream);
  }
  LLM_FAIL("gemm_tc: unknown output dtype %d", out_dtype);
}

// ---------------------------------------------------------------- a wait that runs out, for tests
// One warp waits, through the same bounded wait as the product's warps, on a barrier that nobody
// arrives on: no copy and no tensor memory is in flight.  After `limit_ns` the wait gives up,
// records code 9 in `status` and the kernel returns by itself.  It shows that a wait that runs out
// leaves the device usable and is seen by the host; nothing else launches it.
__global__ void wait_probe_kernel(unsigned long long limit_ns, int *status) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  mbar_wait_limit(smem_u32(&bar), 0, &abort_flag, status, 9, limit_ns);
}

LLM_EXPORT int llm_gemm_tc_wait_probe(long long limit_ns, int *status, cudaStream_t stream) {
  LLM_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ll, "wait_probe: the limit must lie in (0, 100 ms]");
  LLM_REQUIRE(status != nullptr, "wait_probe: no status word");
  wait_probe_kernel<<<1, 32, 0, stream>>>((unsigned long long)limit_ns, status);
  LLM_CHECK_LAUNCH("wait_probe");
  return LLM_OK;
}
