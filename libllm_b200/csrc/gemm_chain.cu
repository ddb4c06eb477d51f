// A chain of products and norms of one decoding step in ONE launch.
//
// A decoding step of a few tokens is a string of small dependent kernels (norm, product, product,
// norm, ...), each of which streams its weights once from HBM and then hands a few kilobytes to
// the next.  Launched one by one, even with programmatic dependent launch, every hand-over costs
// the drain of one grid and the ramp-up of the next.  Here the whole string is a list of jobs that
// one persistent grid (one CTA per SM) works through:
//
//   product   out[M, N] = x[M, K] * W[N, K]^T on the tensor cores, exactly as in gemm_tc.cu (W's
//             rows are the 128-row operand, tokens the N operand, accumulators in tensor memory),
//             32-bit output, optionally in parts of K that the next norm adds up;
//   SwiGLU    the same over a stacked gate|up matrix, storing silu(gate) * up in bfloat16;
//   norm      v = resid + sum of parts (32-bit, parts in index order), resid = v, out = RMSNorm(v)
//             in bfloat16: one row per tile, computed by the CTA's four epilogue warps.
//
// Tiles of all jobs are numbered through and dealt round-robin to the CTAs, so every CTA meets the
// jobs in the same order.  A job whose input another job of the chain writes waits until that
// job's tiles are all done: every epilogue warp adds one to the job's counter in global memory
// after its stores (fence, then atomic), the reader polls the counter with an acquiring load
// before it issues TMA loads of the data.  Seven warps: one loads WEIGHTS, which depend on nothing,
// as far ahead as the ring of stages has room, across tile and job boundaries, also while the job
// they belong to still waits for its input; one follows it through the same stages and loads the
// ACTIVATIONS of a stage once its job may run; one issues the products; four read the accumulators,
// store, and compute the norms' rows.  A stage is two k blocks of 64 (32 KB of weights): what a
// stage costs the loaders and the issuer (a wait on a barrier, a transaction count, a commit) is
// the same for 16 KB and for 32 KB.
//
// Measured (8 tokens, the widths 2,048 / 8,192, cold L2, times from the device's clock inside the
// kernel): output projection done 7-9 us after the start, norm +3.5, gate|up + SwiGLU +12-16,
// down +5.5-7.5, norm +3.5, q|k|v +2-3: 44 us, no less than the same six as launches of their own
// with programmatic dependent launch (39 us inside a step's graph, where the inputs are warm).  A
// hand-over through global memory costs the same either way (the writer's stores become visible,
// its count arrives, the reader's poll and its first dependent load: about 3.5 us), the weights
// that can be fetched ahead are bounded by shared memory either way, and a CTA of this kernel fills
// an SM, so that neither the attention kernel before it nor the one after it overlaps its ends as
// they do with the smaller kernels.  The engine therefore uses it only when asked to
// (LIBLLM_B200_GEMM_CHAIN=1).  Asking L2 for weights further ahead than the ring reaches
// (CH_L2_AHEAD stages, cp.async.bulk.prefetch.tensor) did not shorten any phase and delayed the first.
//
// Every wait has a time limit (barriers: tc_common.cuh; counters: here).  When one runs out the
// CTA records a code in `status`, waits for its loads in flight, frees its tensor memory and
// returns; CTAs that wait for its tiles give up the same way.  The last CTA to finish sets the
// counters back to zero.  Fixed orders of addition: a product's k blocks in order, a norm's parts
// in index order, so a row's result does not depend on what else is in the step.
//
// The reference runs each of these as a launch of its own (src/libllm/llama.cc:81-98, 251-267).
#include "common.cuh"
#include "tc_common.cuh"
#include <string.h>

LLM_DEFINE_LAST_ERROR(llm_gemm_chain_last_error)

// What the host library hands over for one job (plain C; mirrored in csrc/kernels.cc).
struct llm_chain_job {
  int kind;                 // 0 product, 1 SwiGLU product, 2 add + RMSNorm
  int dep0, dep1;           // jobs of this chain that must be complete first; -1: none
  // products
  const void *x;            // [M, K] bfloat16, row stride ldx
  long long ldx;
  const void *w;            // [N, K] bfloat16
  void *out;                // product: 32-bit [parts][M, ldo]; SwiGLU: bfloat16 [M, ldo]; norm: bfloat16 [rows, hidden] or null
  long long ldo;
  int M, N, K, k_parts;
  long long part_stride;    // elements between the parts of a product's output
  // norm
  float *resid;             // [*, hidden] 32-bit
  const float *delta;       // [delta_parts][*, hidden] 32-bit, or null
  int delta_parts;
  long long delta_stride;
  const float *weight;      // [hidden]
  float eps;
  const int *rows;          // source rows (device), or null: row i is row i and resid moves on
  int n_rows, hidden;
};

namespace {

constexpr int CH_THREADS = 224;
constexpr int CH_ROWS = 128;
constexpr int CH_A_BYTES = CH_ROWS * TC_BK * 2;     // one panel: 128 rows of W x 64 k
constexpr int CH_PANELS = 2;                        // panels (k blocks of 64) per stage
constexpr int CH_MAX_JOBS = 8;
#ifndef CH_L2_AHEAD
#define CH_L2_AHEAD 0         // stages beyond the ring whose weights are asked into L2 (32 KB each and CTA); 0: none
#endif
#ifndef CH_RING_KB
#define CH_RING_KB 184
#endif
constexpr int CH_NORM_MAX_H = 8192;
constexpr int CH_XCH_BYTES = 64 * 17 * 4;
enum { JOB_GEMM = 0, JOB_SWIGLU = 1, JOB_NORM = 2 };

struct alignas(64) ChainJob {
  CUtensorMap map_w, map_x;
  void *out;
  long long ldo, part_stride;
  float *resid;
  const float *delta;
  const float *weight;
  const int *rows;
  long long delta_stride;
  int kind, M, n_out, row_tiles, k_parts, kb_per_part, n_kblocks;
  int box_rows;             // rows of W per TMA box: 128 (a plain product's tile), 64 (gate rows, up rows)
  int n_tiles, tile_base, dep0, dep1;
  int delta_parts, hidden;
  float eps;
};
struct ChainParams {
  ChainJob jobs[CH_MAX_JOBS];
  int *counters;            // CH_MAX_JOBS + 1 zeros; left zero
  int *status;
  unsigned long long *trace;   // null, or where times are recorded for measurements (see llm_gemm_chain_trace)
  int n_jobs, total_tiles;
};
static_assert(sizeof(ChainParams) <= 4000, "the chain's parameters must fit a kernel's parameter space");

template <int TN>
struct ChainShape {
  static constexpr int B_BYTES = TN * TC_BK * 2;
  // A stage is two k blocks: the loader's and the issuer's cost per stage (a wait on a barrier, a
  // transaction count, a commit: about 400 cycles together, measured) is the same for 16 KB and
  // for 32 KB of weights, and at 16 KB it alone holds an SM to its share of HBM and no more.
  static constexpr int STAGE_BYTES = CH_PANELS * (CH_A_BYTES + B_BYTES);
  static constexpr int STAGES = (CH_RING_KB * 1024) / STAGE_BYTES;
  static constexpr int TMEM_COLS = 2 * TN < 32 ? 32 : 2 * TN;
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + CH_XCH_BYTES + CH_NORM_MAX_H * 4 + 512;
};

__device__ __forceinline__ int ld_acquire(const int *p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Orders this thread's writes to global memory before reads of them by TMA (the asynchronous proxy).
__device__ __forceinline__ void fence_async_proxy_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// Asks for a box of a tensor to be brought into L2; nothing waits for it.
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ int find_job(const ChainParams &p, int g) {
  int j = 0;
  while (j + 1 < p.n_jobs && g >= p.jobs[j].tile_base + p.jobs[j].n_tiles) ++j;
  return j;
}
// Whether the jobs that `job` reads from are complete (every lane gets lane 0's answer).
__device__ __forceinline__ bool deps_done(const ChainParams &p, const ChainJob &job) {
  bool ok = true;
  if (job.dep0 >= 0) ok = ld_acquire(p.counters + job.dep0) >= 4 * p.jobs[job.dep0].n_tiles;
  if (ok && job.dep1 >= 0) ok = ld_acquire(p.counters + job.dep1) >= 4 * p.jobs[job.dep1].n_tiles;
  return __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
}
// One more tile of `job` is stored: called by every epilogue warp, all lanes.
__device__ __forceinline__ void tile_done(const ChainParams &p, int j, int lane) {
  __syncwarp();
  if (lane == 0) {
    __threadfence();
    fence_async_proxy_global();
    atomicAdd(p.counters + j, 1);
  }
}

template <int TN>
__global__ void __launch_bounds__(CH_THREADS, 1) gemm_chain_kernel(const __grid_constant__ ChainParams p) {
  using S = ChainShape<TN>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char *xch_raw = smem + (size_t)STAGES * S::STAGE_BYTES;
  float *row_buf = (float *)(xch_raw + CH_XCH_BYTES);
  unsigned long long *bars = (unsigned long long *)(row_buf + CH_NORM_MAX_H);
  const unsigned bar_full = smem_u32(bars), bar_empty = smem_u32(bars + STAGES);
  const unsigned bar_tfull = smem_u32(bars + 2 * STAGES), bar_tempty = smem_u32(bars + 2 * STAGES + 2);
  const unsigned bar_xfull = smem_u32(bars + 2 * STAGES + 4), bar_xempty = smem_u32(bars + 2 * STAGES + 5);
  const unsigned bar_norm = smem_u32(bars + 2 * STAGES + 6);
  unsigned *tmem_slot = (unsigned *)(bars + 2 * STAGES + 7);
  volatile int *abort_flag = (volatile int *)(tmem_slot + 1);
  float *red = (float *)(tmem_slot + 2);          // the four warps' sums of a norm's row, two rows in turn

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
    mbar_init(bar_norm, 4);
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

  // The walk over this CTA's (tile, two k blocks) stages, the same for both loaders.
  struct Walk {
    int g, j, kb, kb1, row_a, row_b;
    bool valid;
  };
  // the next product tile of this CTA at or after g (norm tiles are the epilogue's alone)
  auto start = [&](Walk &w, int g) {
    for (;; g += gridDim.x) {
      w.g = g;
      w.valid = g < p.total_tiles;
      if (!w.valid) return;
      w.j = find_job(p, g);
      const ChainJob &job = p.jobs[w.j];
      if (job.kind == JOB_NORM) continue;
      const int t = g - job.tile_base;
      const int part = t % job.k_parts, row_tile = t / job.k_parts;
      w.kb = part * job.kb_per_part;
      w.kb1 = min(job.n_kblocks, w.kb + job.kb_per_part);
      if (job.kind == JOB_SWIGLU) {
        w.row_a = row_tile * 64;
        w.row_b = job.n_out + w.row_a;
      } else {
        w.row_a = row_tile * 128;
        w.row_b = w.row_a + 64;
      }
      return;
    }
  };
  auto next = [&](Walk &w) {
    if ((w.kb += CH_PANELS) >= w.kb1) start(w, w.g + gridDim.x);
  };
  unsigned long long *trace_cta = p.trace ? p.trace + p.total_tiles + (size_t)blockIdx.x * (CH_MAX_JOBS + 2) : nullptr;
  unsigned long long *trace_stage = p.trace && blockIdx.x == 0 ? p.trace + p.total_tiles + (size_t)gridDim.x * (CH_MAX_JOBS + 2) : nullptr;

  if (warp == 0) {
    // ------------------------------------------------------------ loader of weights
    // Weights depend on nothing: this warp fills the ring with them as far ahead as it has room,
    // across tile and job boundaries, also while the job they belong to still waits for its input.
    const bool leader = elect_one();
    if (trace_cta && lane == 0) trace_cta[CH_MAX_JOBS] = globaltimer();
    if (leader)
      for (int j = 0; j < p.n_jobs; ++j)
        if (p.jobs[j].kind != JOB_NORM) tma_prefetch_map(&p.jobs[j].map_w);
    Walk a;
    start(a, blockIdx.x);
    int stage = 0;
    unsigned phase = 1;                          // parity of the stage's release before this use
    unsigned n_a = 0;
    bool ok = true;
#if CH_L2_AHEAD > 0
    Walk c = a;                                  // further ahead than the ring reaches, weights are asked into L2
    unsigned n_c = 0;
#endif
    while (a.valid) {
      if (n_a >= (unsigned)STAGES) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase, abort_flag, p.status, 1));
        if (!ok) break;
      }
      if (leader) {
        const unsigned dst = smem_u32(smem + (size_t)stage * S::STAGE_BYTES);
        const CUtensorMap *map = &p.jobs[a.j].map_w;
        const bool one_box = p.jobs[a.j].box_rows == 128;
        const unsigned bar = bar_full + 8 * stage;
        if (a.kb + 1 < a.kb1) {
          mbar_expect_tx(bar, 2 * (CH_A_BYTES + S::B_BYTES));
          tma_load_2d(dst, map, a.kb * TC_BK, a.row_a, bar);
          tma_load_2d(dst + CH_A_BYTES, map, (a.kb + 1) * TC_BK, a.row_a, bar);
          if (!one_box) {
            tma_load_2d(dst + CH_A_BYTES / 2, map, a.kb * TC_BK, a.row_b, bar);
            tma_load_2d(dst + CH_A_BYTES + CH_A_BYTES / 2, map, (a.kb + 1) * TC_BK, a.row_b, bar);
          }
        } else {
          mbar_expect_tx(bar, CH_A_BYTES + S::B_BYTES);
          tma_load_2d(dst, map, a.kb * TC_BK, a.row_a, bar);
          if (!one_box) tma_load_2d(dst + CH_A_BYTES / 2, map, a.kb * TC_BK, a.row_b, bar);
        }
        if (trace_stage && n_a < 64) trace_stage[n_a * 4] = globaltimer();
      }
      next(a);
      ++n_a;
      if (++stage == STAGES) {
        stage = 0;
        phase ^= 1;
      }
#if CH_L2_AHEAD > 0
      if (n_c < n_a) {
        c = a;
        n_c = n_a;
      }
      while (n_a >= (unsigned)STAGES && c.valid && n_c < n_a + CH_L2_AHEAD) {   // the ring's first filling goes first
        if (leader) {
          const CUtensorMap *map = &p.jobs[c.j].map_w;
          const int np = min(CH_PANELS, c.kb1 - c.kb);
          const bool one_box = p.jobs[c.j].box_rows == 128;
          for (int pn = 0; pn < np; ++pn) {
            tma_prefetch_2d(map, (c.kb + pn) * TC_BK, c.row_a);
            if (!one_box) tma_prefetch_2d(map, (c.kb + pn) * TC_BK, c.row_b);
          }
        }
        next(c);
        ++n_c;
      }
#endif
    }
    grid_dependency_wait();
    if (leader && (!ok || *abort_flag)) {
      // given up: let what is in flight land before the CTA goes away
      const unsigned long long t1 = globaltimer();
      while (globaltimer() - t1 < 2000000ull) {
      }
    }
  } else if (warp == 6) {
    // ------------------------------------------------------------ loader of activations
    // Follows the weights' loader through the same stages: a stage's tokens are loaded when the
    // stage is free and the job that writes them is complete.  Nothing an earlier kernel wrote,
    // and no counter, is looked at before the wait for that kernel.
    const bool leader = elect_one();
    if (leader)
      for (int j = 0; j < p.n_jobs; ++j)
        if (p.jobs[j].kind != JOB_NORM) tma_prefetch_map(&p.jobs[j].map_x);
    grid_dependency_wait();
    if (trace_cta && lane == 0) trace_cta[CH_MAX_JOBS + 1] = globaltimer();
    Walk b;
    start(b, blockIdx.x);
    int stage = 0;
    unsigned phase = 1;
    unsigned n_b = 0;
    int cleared_job = -1;
    bool ok = true;
    while (b.valid && ok) {
      if (b.j != cleared_job) {
        const unsigned long long t0 = globaltimer();
        while (!deps_done(p, p.jobs[b.j])) {
          if (*abort_flag || globaltimer() - t0 > TC_WAIT_NS) {
            if (!*abort_flag) {
              *abort_flag = 1;
              if (p.status && lane == 0) atomicCAS(p.status, 0, 7);
            }
            ok = false;
            break;
          }
          __nanosleep(32);
        }
        if (!ok) break;
        cleared_job = b.j;
        if (trace_cta && lane == 0) trace_cta[b.j] = globaltimer();
      }
      if (n_b >= (unsigned)STAGES) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * stage, phase, abort_flag, p.status, 1));
        if (!ok) break;
      }
      if (leader) {
        const unsigned dst = smem_u32(smem + (size_t)stage * S::STAGE_BYTES) + CH_PANELS * CH_A_BYTES;
        const CUtensorMap *map = &p.jobs[b.j].map_x;
        const unsigned bar = bar_full + 8 * stage;
        tma_load_2d(dst, map, b.kb * TC_BK, 0, bar);
        if (b.kb + 1 < b.kb1) tma_load_2d(dst + S::B_BYTES, map, (b.kb + 1) * TC_BK, 0, bar);
        if (trace_stage && n_b < 64) trace_stage[n_b * 4 + 1] = globaltimer();
      }
      next(b);
      ++n_b;
      if (++stage == STAGES) {
        stage = 0;
        phase ^= 1;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ tensor-core issue
    const bool leader = elect_one();
    constexpr unsigned IDESC = instr_desc(CH_ROWS, TN);
    int stage = 0;
    unsigned phase = 0;
    int iter = 0;
    unsigned n_s = 0;
    bool ok = true;
    for (int g = blockIdx.x; g < p.total_tiles && ok; g += gridDim.x) {
      const ChainJob &job = p.jobs[find_job(p, g)];
      if (job.kind == JOB_NORM) continue;
      const int part = (g - job.tile_base) % job.k_parts;
      const int kb0 = part * job.kb_per_part, kb1 = min(job.n_kblocks, kb0 + job.kb_per_part);
      const int acc = iter & 1;
      const unsigned acc_phase = (iter >> 1) & 1;
      ++iter;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.status, 2));
      if (!ok) break;
      tc_fence_after();
      const unsigned d_tmem = tmem_base + acc * TN;
      for (int kb = kb0; kb < kb1; kb += CH_PANELS) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, 3));
        if (!ok) break;
        tc_fence_after();
        if (leader && trace_stage && n_s < 64) trace_stage[n_s * 4 + 2] = globaltimer();
        ++n_s;
        const unsigned a_addr = smem_u32(smem + (size_t)stage * S::STAGE_BYTES);
        const unsigned long long a_desc = smem_desc(a_addr), b_desc = smem_desc(a_addr + CH_PANELS * CH_A_BYTES);
        const unsigned first = kb > kb0 ? 1u : 0u;
        const bool two = kb + 1 < kb1;
        if (leader) {
#pragma unroll
          for (int kk = 0; kk < TC_BK / 16; ++kk)
            tc_mma(d_tmem, a_desc + (unsigned long long)(kk * 2), b_desc + (unsigned long long)(kk * 2), IDESC,
                   kk > 0 ? 1u : first);
          if (two) {
            // the second panel: descriptors further by a panel (addresses in units of 16 bytes)
#pragma unroll
            for (int kk = 0; kk < TC_BK / 16; ++kk)
              tc_mma(d_tmem, a_desc + (unsigned long long)(CH_A_BYTES / 16 + kk * 2),
                     b_desc + (unsigned long long)(S::B_BYTES / 16 + kk * 2), IDESC, 1u);
          }
          tc_commit(bar_empty + 8 * stage);
        }
        __syncwarp();
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok && leader) tc_commit(bar_tfull + 8 * acc);
      __syncwarp();
    }
    grid_dependency_wait();
  } else {
    // ------------------------------------------------------------ epilogue and norms (warps 2..5)
    grid_dependency_wait();
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;                 // 0 .. 127 among the epilogue threads
    float *xch = (float *)xch_raw;
    int iter = 0;
    unsigned n_hand = 0;                             // SwiGLU hand-overs so far
    unsigned n_norm = 0;                             // norm rows so far
    bool ok = true;
    for (int g = blockIdx.x; g < p.total_tiles && ok; g += gridDim.x) {
      const int j = find_job(p, g);
      const ChainJob &job = p.jobs[j];
      if (job.kind == JOB_NORM) {
        // ---- one row: v = resid + parts, resid = v, out = v * w * rsqrt(mean(v^2) + eps)
        // the norm's weight depends on nothing: on its way before the wait (rows of up to 2,048)
        const int H = job.hidden, n4 = H >> 2;
        float4 wv[4];
        const bool w_early = job.out && n4 <= 4 * 128;
        if (w_early) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (et + k * 128 < n4) wv[k] = *(reinterpret_cast<const float4 *>(job.weight) + et + k * 128);
        }
        {
          const unsigned long long t0 = globaltimer();
          while (!deps_done(p, job)) {
            if (*abort_flag || globaltimer() - t0 > TC_WAIT_NS) {
              if (!*abort_flag) {
                *abort_flag = 1;
                if (p.status && lane == 0) atomicCAS(p.status, 0, 8);
              }
              ok = false;
              break;
            }
            __nanosleep(40);
          }
          if (!ok) break;
        }
        const int i = g - job.tile_base;
        const int r = job.rows ? job.rows[i] : i;
        float *x = job.resid + (size_t)r * H;
        const float *d = job.delta ? job.delta + (size_t)r * H : nullptr;
        const bool moves = job.rows == nullptr && job.delta_parts > 0;
        float ss = 0.f;
        for (int c0 = 0; c0 < n4; c0 += 4 * 128) {
          float4 v[4], dv[4][8];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int c4 = c0 + et + k * 128;
            if (c4 < n4) {
              v[k] = __ldcg(reinterpret_cast<const float4 *>(x) + c4);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                if (q < job.delta_parts) dv[k][q] = __ldcg(reinterpret_cast<const float4 *>(d + (size_t)q * job.delta_stride) + c4);
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int c4 = c0 + et + k * 128;
            if (c4 < n4) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                if (q < job.delta_parts) {
                  v[k].x += dv[k][q].x;
                  v[k].y += dv[k][q].y;
                  v[k].z += dv[k][q].z;
                  v[k].w += dv[k][q].w;
                }
              if (moves) __stcg(reinterpret_cast<float4 *>(x) + c4, v[k]);
              reinterpret_cast<float4 *>(row_buf)[c4] = v[k];
              ss += v[k].x * v[k].x;
              ss += v[k].y * v[k].y;
              ss += v[k].z * v[k].z;
              ss += v[k].w * v[k].w;
            }
          }
        }
        if (job.out) {
          // The four warps' sums meet through shared memory and a barrier with a time limit; two
          // sets of sums in turn, so that a warp that is a row ahead overwrites nothing still read.
          ss = warp_sum(ss);
          float *sums = red + 4 * (n_norm & 1);
          if (lane == 0) {
            sums[quarter] = ss;
            mbar_arrive(bar_norm);
          }
          ok = __all_sync(0xffffffffu, mbar_wait(bar_norm, n_norm & 1, abort_flag, p.status, 8));
          if (!ok) break;
          ++n_norm;
          const float total = ((sums[0] + sums[1]) + sums[2]) + sums[3];
          const float inv = rsqrtf(total / (float)H + job.eps);
          __nv_bfloat16 *o = (__nv_bfloat16 *)job.out + (size_t)i * H;
          if (w_early) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const int c4 = et + k * 128;
              if (c4 < n4) {
                const float4 v = reinterpret_cast<const float4 *>(row_buf)[c4];
                st4(o + 4 * c4, make_float4(v.x * wv[k].x * inv, v.y * wv[k].y * inv, v.z * wv[k].z * inv, v.w * wv[k].w * inv));
              }
            }
          } else {
            for (int c4 = et; c4 < n4; c4 += 128) {
              const float4 v = reinterpret_cast<const float4 *>(row_buf)[c4];
              const float4 w = *(reinterpret_cast<const float4 *>(job.weight) + c4);
              st4(o + 4 * c4, make_float4(v.x * w.x * inv, v.y * w.y * inv, v.z * w.z * inv, v.w * w.w * inv));
            }
          }
        }
        tile_done(p, j, lane);
        if (p.trace && quarter == 0 && lane == 0) p.trace[g] = globaltimer();
        continue;
      }
      // ---- a product's tile
      const int t = g - job.tile_base;
      const int part = t % job.k_parts, row_tile = t / job.k_parts;
      const int acc = iter & 1;
      const unsigned acc_phase = (iter >> 1) & 1;
      ++iter;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, 4));
      if (!ok) break;
      tc_fence_after();
      const int row_in_tile = quarter * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < TN && ok; c0 += 16) {
        if (c0 >= job.M) break;                        // columns of tokens that are not there
        float v[16];
        tc_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * TN + c0), v);
        if (job.kind == JOB_SWIGLU) {
          if (quarter >= 2) {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_xempty, (n_hand & 1) ^ 1, abort_flag, p.status, 5));
            if (!ok) break;
#pragma unroll
            for (int i = 0; i < 16; ++i) xch[(row_in_tile - 64) * 17 + i] = v[i];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_xfull);
          } else {
            ok = __all_sync(0xffffffffu, mbar_wait(bar_xfull, n_hand & 1, abort_flag, p.status, 6));
            if (!ok) break;
            const int f = row_tile * 64 + row_in_tile;
            __nv_bfloat16 *o = (__nv_bfloat16 *)job.out;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int tok = c0 + i;
              const float up = xch[row_in_tile * 17 + i];
              const float gate = v[i];
              if (f < job.n_out && tok < job.M) o[(size_t)tok * job.ldo + f] = __float2bfloat16_rn(gate / (1.f + expf(-gate)) * up);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_xempty);
          }
          ++n_hand;
        } else {
          const int f = row_tile * 128 + row_in_tile;
          float *o = (float *)job.out + (size_t)part * job.part_stride;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int tok = c0 + i;
            if (f < job.n_out && tok < job.M) __stcg(o + (size_t)tok * job.ldo + f, v[i]);
          }
        }
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
      tile_done(p, j, lane);
      if (p.trace && quarter == 0 && lane == 0) p.trace[g] = globaltimer();
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
  if (threadIdx.x == 0) {
    // the last CTA to leave puts the counters back to zero for the next chain
    __threadfence();
    if (atomicAdd(p.counters + CH_MAX_JOBS, 1) == (int)gridDim.x - 1) {
      for (int j = 0; j <= CH_MAX_JOBS; ++j) p.counters[j] = 0;
      __threadfence();
    }
  }
}

template <int TN>
int launch_chain(const ChainParams &p, cudaStream_t stream) {
  using S = ChainShape<TN>;
  auto kern = gemm_chain_kernel<TN>;
  LLM_CHECK_CUDA(llm_allow_smem(kern, S::SMEM), "gemm_chain attribute");
  const int grid = p.total_tiles < sm_count() ? p.total_tiles : sm_count();
  LLM_CHECK_CUDA(llm_launch(kern, dim3(grid), dim3(CH_THREADS), S::SMEM, stream, p), "gemm_chain launch");
  return LLM_OK;
}

}  // namespace

namespace {
unsigned long long *g_trace = nullptr;
}
// For measurements: while `buf` is not null, every chain launched from this thread's library
// records times (the device's nanosecond clock) there: [tile] when the tile's results were stored,
// then per CTA ten words: when the loader saw each job's inputs ready, when the CTA started and when
// the kernel before it was complete.  `buf` holds tiles + 10 * CTAs words of 64 bits.
LLM_EXPORT int llm_gemm_chain_trace(unsigned long long *buf) {
  g_trace = buf;
  return LLM_OK;
}
LLM_EXPORT int llm_gemm_chain_max_jobs() { return CH_MAX_JOBS; }
LLM_EXPORT int llm_gemm_chain_max_tokens() { return 64; }
LLM_EXPORT int llm_gemm_chain_max_hidden() { return CH_NORM_MAX_H; }
LLM_EXPORT int llm_gemm_chain_counters() { return CH_MAX_JOBS + 1; }

// Runs the jobs in order as one launch.  `counters` are llm_gemm_chain_counters() device ints that
// are zero and are left zero; `status` (device int, may be null) receives a non-zero code if a wait
// inside the kernel ran out of time.  A job's dep0/dep1 name the jobs of this chain whose output
// it reads; what earlier launches wrote needs no entry.
LLM_EXPORT int llm_gemm_chain(const llm_chain_job *jobs, int n_jobs, int *counters, int *status, cudaStream_t stream) {
  if (n_jobs == 0) return LLM_OK;
  LLM_REQUIRE(n_jobs > 0 && n_jobs <= CH_MAX_JOBS, "gemm_chain: %d jobs, at most %d fit one launch", n_jobs, CH_MAX_JOBS);
  LLM_REQUIRE(counters != nullptr, "gemm_chain: no counters");
  ChainParams p;
  memset(&p, 0, sizeof(p));
  int max_m = 1;
  for (int j = 0; j < n_jobs; ++j)
    if (jobs[j].kind != JOB_NORM) max_m = jobs[j].M > max_m ? jobs[j].M : max_m;
  LLM_REQUIRE(max_m <= 64, "gemm_chain: %d tokens, at most 64", max_m);
  const int TN = max_m <= 16 ? 16 : max_m <= 32 ? 32 : 64;
  long long base = 0;
  for (int j = 0; j < n_jobs; ++j) {
    const llm_chain_job &in = jobs[j];
    ChainJob &job = p.jobs[j];
    LLM_REQUIRE(in.dep0 < j && in.dep1 < j && in.dep0 >= -1 && in.dep1 >= -1, "gemm_chain: job %d depends on a job that is not before it", j);
    job.kind = in.kind;
    job.dep0 = in.dep0;
    job.dep1 = in.dep1;
    if (in.kind == JOB_NORM) {
      LLM_REQUIRE(in.n_rows > 0 && in.hidden > 0 && in.hidden % 4 == 0 && in.hidden <= CH_NORM_MAX_H,
                  "gemm_chain: a norm over %d rows of width %d (a multiple of 4, at most %d)", in.n_rows, in.hidden, CH_NORM_MAX_H);
      LLM_REQUIRE(in.delta_parts >= 0 && in.delta_parts <= 8 && (in.delta_parts == 0 || in.delta != nullptr), "gemm_chain: a norm adds at most 8 parts");
      LLM_REQUIRE(in.resid != nullptr && (in.out == nullptr || in.weight != nullptr), "gemm_chain: a norm needs its stream and its weight");
      LLM_REQUIRE((uintptr_t)in.resid % 16 == 0 && (uintptr_t)in.delta % 16 == 0 && (uintptr_t)in.weight % 16 == 0 &&
                      (uintptr_t)in.out % 8 == 0 && in.delta_stride % 4 == 0, "gemm_chain: a norm's rows must start on 16 bytes");
      job.out = in.out;
      job.resid = in.resid;
      job.delta = in.delta;
      job.delta_parts = in.delta_parts;
      job.delta_stride = in.delta_stride;
      job.weight = in.weight;
      job.eps = in.eps;
      job.rows = in.rows;
      job.hidden = in.hidden;
      job.k_parts = 1;
      job.n_tiles = in.n_rows;
    } else {
      LLM_REQUIRE(in.kind == JOB_GEMM || in.kind == JOB_SWIGLU, "gemm_chain: unknown kind %d of job %d", in.kind, j);
      LLM_REQUIRE(in.M > 0 && in.N > 0 && in.K > 0, "gemm_chain: bad sizes %d x %d x %d", in.M, in.N, in.K);
      LLM_REQUIRE(in.K % 8 == 0 && in.ldx % 8 == 0, "gemm_chain: K = %d and the row stride %lld must be multiples of 8", in.K, in.ldx);
      LLM_REQUIRE((uintptr_t)in.x % 16 == 0 && (uintptr_t)in.w % 16 == 0, "gemm_chain: operands must be 16-byte aligned");
      const bool sw = in.kind == JOB_SWIGLU;
      LLM_REQUIRE(!sw || (in.N % 2 == 0 && in.k_parts == 1), "gemm_chain: a stacked gate|up product has an even number of rows and one part");
      const int n_out = sw ? in.N / 2 : in.N;
      const int box_rows = sw ? 64 : 128;
      job.box_rows = box_rows;
      const int rows_out = sw ? 64 : 128;
      job.n_out = n_out;
      job.M = in.M;
      job.row_tiles = (n_out + rows_out - 1) / rows_out;
      job.n_kblocks = (in.K + TC_BK - 1) / TC_BK;
      job.k_parts = in.k_parts;
      LLM_REQUIRE(in.k_parts >= 1 && in.k_parts <= 64, "gemm_chain: %d parts", in.k_parts);
      job.kb_per_part = (job.n_kblocks + in.k_parts - 1) / in.k_parts;
      LLM_REQUIRE((long long)(in.k_parts - 1) * job.kb_per_part < job.n_kblocks, "gemm_chain: %d parts leave one of them without work (K = %d)", in.k_parts, in.K);
      job.out = in.out;
      job.ldo = in.ldo;
      job.part_stride = in.part_stride;
      int rc = get_map(in.w, in.N, in.K, in.K, box_rows, &job.map_w);
      if (rc != LLM_OK) return rc;
      rc = get_map(in.x, in.M, in.K, in.ldx, TN, &job.map_x);
      if (rc != LLM_OK) return rc;
      const long long tiles = (long long)job.row_tiles * in.k_parts;
      LLM_REQUIRE(tiles < (1ll << 28), "gemm_chain: too many tiles");
      job.n_tiles = (int)tiles;
    }
    job.tile_base = (int)base;
    base += job.n_tiles;
    LLM_REQUIRE(base < (1ll << 29), "gemm_chain: too many tiles");
  }
  p.counters = counters;
  p.status = status;
  p.trace = g_trace;
  p.n_jobs = n_jobs;
  p.total_tiles = (int)base;
  if (TN == 16) return launch_chain<16>(p, stream);
  if (TN == 32) return launch_chain<32>(p, stream);
  return launch_chain<64>(p, stream);
}
