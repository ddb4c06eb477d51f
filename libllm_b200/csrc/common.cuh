// Shared helpers of the sm_100a kernels: element types, status codes and the error
// string each library keeps for its last failed call.
//
// Every exported function is `extern "C"`, takes raw device pointers plus the CUDA
// stream to launch on, allocates nothing and returns 0 or a non-zero status; the Python
// side (libllm_b200/csrc/ops.py) turns a status into an exception with this message.
// The reference reports errors the same way at its C boundary: a code and a message
// (src/libllm/llm.h:42-47).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define LLM_OK 0
#define LLM_ERR_INVALID 0x0100
#define LLM_ERR_CUDA 0x0102

enum LlmDtype { LLM_F32 = 0, LLM_BF16 = 1 };

static thread_local char g_llm_error[512] = "";

#define LLM_EXPORT extern "C" __attribute__((visibility("default")))

#define LLM_FAIL(...)                                   \
  do {                                                  \
    snprintf(g_llm_error, sizeof(g_llm_error), __VA_ARGS__); \
    return LLM_ERR_INVALID;                             \
  } while (0)

#define LLM_REQUIRE(cond, ...) \
  do {                         \
    if (!(cond)) LLM_FAIL(__VA_ARGS__); \
  } while (0)

#define LLM_CHECK_LAUNCH(name)                                                        \
  do {                                                                                \
    cudaError_t e_ = cudaGetLastError();                                              \
    if (e_ != cudaSuccess) {                                                          \
      snprintf(g_llm_error, sizeof(g_llm_error), "%s: %s", name, cudaGetErrorString(e_)); \
      return LLM_ERR_CUDA;                                                            \
    }                                                                                 \
  } while (0)

#define LLM_CHECK_CUDA(expr, name)                                                    \
  do {                                                                                \
    cudaError_t e_ = (expr);                                                          \
    if (e_ != cudaSuccess) {                                                          \
      snprintf(g_llm_error, sizeof(g_llm_error), "%s: %s", name, cudaGetErrorString(e_)); \
      return LLM_ERR_CUDA;                                                            \
    }                                                                                 \
  } while (0)

#define LLM_DEFINE_LAST_ERROR(fn) \
  LLM_EXPORT const char *fn() { return g_llm_error; }

// Programmatic dependent launch.  A kernel launched with `llm_launch` may start while the
// kernel before it in the stream is still running: its CTAs are scheduled as soon as every
// CTA of the predecessor has called `grid_dependents_launch` (or has exited).  Before it
// reads anything an earlier kernel wrote, and before it writes anything an earlier kernel
// may still read, it calls `grid_dependency_wait`, which returns when the predecessor has
// finished and its writes are visible.  What a kernel does before the wait (index
// arithmetic, loads of weights) overlaps the predecessor's tail.  Every thread of every
// kernel launched this way calls the wait, so completion stays transitive along the stream.
// Without the launch attribute both calls do nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependents_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
static inline bool llm_pdl_enabled() {
  static const bool on = getenv("LIBLLM_B200_NO_PDL") == nullptr;
  return on;
}

// Dynamic shared memory above 48 KB has to be allowed per kernel; the attribute is set when a
// kernel first needs more than it has been allowed so far (a launch outside any stream capture: a
// step runs once before it is captured), never on every launch.
template <typename... KArgs>
static inline cudaError_t llm_allow_smem(void (*kernel)(KArgs...), size_t smem) {
  static thread_local const void *seen[64];
  static thread_local size_t allowed[64];
  static thread_local int n_seen = 0;
  if (smem <= 48 * 1024) return cudaSuccess;
  int i = 0;
  for (; i < n_seen; ++i)
    if (seen[i] == (const void *)kernel) break;
  if (i < n_seen && allowed[i] >= smem) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  if (i == n_seen && n_seen < 64) {
    seen[n_seen] = (const void *)kernel;
    ++n_seen;
  }
  if (i < 64) allowed[i] = smem;
  return cudaSuccess;
}

template <typename... KArgs, typename... Args>
static inline cudaError_t llm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = llm_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same without the attribute: the kernel starts when everything before it in the stream is
// complete.  For a kernel that must not overlap its predecessor.
template <typename... KArgs, typename... Args>
static inline cudaError_t llm_launch_after(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                           cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cfg.attrs = nullptr;
  cfg.numAttrs = 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Streaming multiprocessors of the current device (asked once per process).
static inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Four consecutive values as 32-bit floats, from or to either element type.
__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16 *p) {
  const uint2 raw = *reinterpret_cast<const uint2 *>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float *p, float4 v) { *reinterpret_cast<float4 *>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16 *p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned *>(&a);
  raw.y = *reinterpret_cast<unsigned *>(&b);
  *reinterpret_cast<uint2 *>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block with a fixed order of additions: warps first, then the warp totals
// in warp order.  The result does not depend on how many rows the launch has.
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float *scratch /* THREADS/32 + 1 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < THREADS / 32 ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[THREADS / 32] = t;
  }
  __syncthreads();
  return scratch[THREADS / 32];
}
