#include "parts/linear.h"

#include <cublas_v2.h>
#include <dlfcn.h>

#include <cstdlib>
#include <map>
#include <mutex>

#include "csrc/kernels.h"
#include "parts/chain.h"
#include "util/log.h"

namespace llm {

const FastSwitches &fast_switches() {
  static const FastSwitches s = [] {
    FastSwitches f;
    auto off = [](const char *name) { return getenv(name) != nullptr; };
    auto num = [](const char *name, int fallback) {
      const char *v = getenv(name);
      return v && *v ? atoi(v) : fallback;
    };
    f.gemv = !off("LIBLLM_B200_NO_GEMV");
    f.decode_attention = !off("LIBLLM_B200_NO_DECODE_ATTENTION");
    f.prefill_attention = !off("LIBLLM_B200_NO_PREFILL_ATTENTION");
    f.gemm_tc = !off("LIBLLM_B200_NO_GEMM_TC");
    f.prefill_attention_tc = !off("LIBLLM_B200_NO_PREFILL_ATTENTION_TC");
    f.decode_attention_tc = !off("LIBLLM_B200_NO_DECODE_ATTENTION_TC");
    f.library_gemm = !off("LIBLLM_B200_NO_LIBRARY_GEMM");
    f.gemm_chain = off("LIBLLM_B200_GEMM_CHAIN");      // set: on (measured no faster than the launches it replaces)
    f.add_in_product = !off("LIBLLM_B200_NO_ADD_IN_PRODUCT");
    f.tc_tokens = num("LIBLLM_B200_TC_TOKENS", 256);
    f.fused_gate_up_tokens = num("LIBLLM_B200_FUSED_GATE_UP_TOKENS", 1024);
    f.gemv_tokens = num("LIBLLM_B200_GEMV_TOKENS", 0);
    return f;
  }();
  return s;
}

std::vector<std::string> product_families(DType dtype) {
  std::vector<std::string> fams = {"gemm_plain"};   // the 32-bit path; with bfloat16, products with a bias
  if (dtype == DType::BF16) {
    const FastSwitches &f = fast_switches();
    if (f.gemm_tc) fams.push_back("gemm_tc");
    if (f.gemm_tc && f.gemm_chain) fams.push_back("gemm_chain");
    if (f.gemv && f.gemv_tokens > 0) fams.push_back("gemv");
  }
  return fams;
}

// ---------------------------------------------------------------- the library product
namespace {
struct Cublas {
  void *lib = nullptr;
  decltype(&cublasCreate_v2) create = nullptr;
  decltype(&cublasSetStream_v2) set_stream = nullptr;
  decltype(&cublasSetWorkspace_v2) set_workspace = nullptr;
  using GemmExFn = cublasStatus_t (*)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void *, const void *,
                                      cudaDataType, int, const void *, cudaDataType, int, const void *, void *, cudaDataType, int,
                                      cublasComputeType_t, cublasGemmAlgo_t);
  GemmExFn gemm_ex = nullptr;
  bool tried = false;
  std::map<int, cublasHandle_t> handles;          // per device
  std::map<int, DeviceBuffer> workspaces;
  std::mutex mu;
};
Cublas &cublas() {
  static Cublas c;
  return c;
}

bool open_cublas(Cublas &c) {
  if (c.tried) return c.lib != nullptr;
  c.tried = true;
  const char *names[] = {"libcublas.so.12", "/usr/local/cuda/lib64/libcublas.so.12", "libcublas.so"};
  for (const char *n : names) {
    c.lib = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    if (c.lib) break;
  }
  if (!c.lib) return false;
  c.create = (decltype(c.create))dlsym(c.lib, "cublasCreate_v2");
  c.set_stream = (decltype(c.set_stream))dlsym(c.lib, "cublasSetStream_v2");
  c.set_workspace = (decltype(c.set_workspace))dlsym(c.lib, "cublasSetWorkspace_v2");
  c.gemm_ex = (decltype(c.gemm_ex))dlsym(c.lib, "cublasGemmEx");
  if (!c.create || !c.set_stream || !c.set_workspace || !c.gemm_ex) {
    c.lib = nullptr;
    return false;
  }
  return true;
}
}  // namespace

bool library_gemm_available() {
  Cublas &c = cublas();
  std::lock_guard<std::mutex> g(c.mu);
  return fast_switches().library_gemm && open_cublas(c);
}

bool library_gemm(cudaStream_t stream, const Act &x, const Weight &w, const Act &out, bool accumulate) {
  Cublas &c = cublas();
  std::lock_guard<std::mutex> g(c.mu);
  if (!fast_switches().library_gemm || !open_cublas(c)) return false;
  int dev = 0;
  LLM_CUDA(cudaGetDevice(&dev));
  auto it = c.handles.find(dev);
  if (it == c.handles.end()) {
    cublasHandle_t h = nullptr;
    if (c.create(&h) != CUBLAS_STATUS_SUCCESS) LLM_THROW(Extension, "cublasCreate failed");
    // a workspace of the library's own size would be allocated inside a call; one given to it
    // keeps a captured step free of allocations
    c.workspaces[dev].allocate((size_t)64 << 20);
    it = c.handles.emplace(dev, h).first;
  }
  cublasHandle_t h = it->second;
  if (c.set_stream(h, stream) != CUBLAS_STATUS_SUCCESS) LLM_THROW(Extension, "cublasSetStream failed");
  if (c.set_workspace(h, c.workspaces[dev].get(), c.workspaces[dev].bytes()) != CUBLAS_STATUS_SUCCESS)
    LLM_THROW(Extension, "cublasSetWorkspace failed");
  const float alpha = 1.f, beta = accumulate ? 1.f : 0.f;
  // Row-major out[T, N] = x[T, K] w[N, K]^T is, column-major, out^T[N, T] = w^T(op T)[N, K] x^T[K, T].
  const cublasStatus_t st =
      c.gemm_ex(h, CUBLAS_OP_T, CUBLAS_OP_N, (int)w.rows, (int)x.rows, (int)x.cols, &alpha, w.data(), CUDA_R_16BF, (int)w.cols,
                x.data, CUDA_R_16BF, (int)x.ld, &beta, out.data, out.dtype == DType::BF16 ? CUDA_R_16BF : CUDA_R_32F, (int)out.ld,
                CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  if (st != CUBLAS_STATUS_SUCCESS) LLM_THROW(Extension, "cublasGemmEx failed (status %d) for a %lld x %lld x %lld product", (int)st,
                                             (long long)x.rows, (long long)w.rows, (long long)x.cols);
  return true;
}

// ---------------------------------------------------------------- choice of the product
Act small_batch_linear(StepContext &ctx, const Act &x, const Weight &w, DType out_dtype, bool swiglu, bool parts_ok) {
  const FastSwitches &f = fast_switches();
  const int T = (int)x.rows, K = (int)x.cols;
  const int n = (int)(swiglu ? w.rows / 2 : w.rows);
  Act none;
  const bool use_gemv = f.gemv && T <= f.gemv_tokens && kernels::gemv_supported(x, w);
  if (f.gemm_tc && T <= f.tc_tokens && !use_gemv && kernels::gemm_tc_supported(x, w)) {
    int parts = 1;
    if (parts_ok && !swiglu && out_dtype == DType::F32) parts = kernels::gemm_tc_suggest_parts(T, n, K);
    Act out = ctx.arena->act(out_dtype, T, n, parts > 1 ? parts : 1);
    if (ctx.chain && ctx.chain->add_product(x, w, out, swiglu, ctx.stream)) return out;
    flush_chain(ctx);
    kernels::gemm_tc(x, w, out, swiglu, ctx.tc_status, ctx.stream);
    return out;
  }
  flush_chain(ctx);
  if (!use_gemv) return none;
  int parts = 1;
  if (parts_ok && !swiglu && out_dtype == DType::F32) parts = kernels::gemv_suggest_parts(T, n, K);
  Act out = ctx.arena->act(out_dtype, T, n, parts > 1 ? parts : 1);
  kernels::gemv_bf16(x, w, out, swiglu, ctx.stream);
  return out;
}

Act linear(StepContext &ctx, const Act &x, const Weight &w, const float *bias, DType out_dtype, bool parts_ok) {
  if (x.cols != w.cols)
    LLM_THROW(InvalidArg, "linear: activations of width %lld meet a matrix of width %lld", (long long)x.cols, (long long)w.cols);
  const int T = (int)x.rows;
  if (x.dtype == DType::F32 || bias != nullptr) {
    flush_chain(ctx);
    // the true 32-bit path; and, in bfloat16, a product with a bias (CUDA cores: such a model pays
    // for it, which load() says once)
    Act out = ctx.arena->act(out_dtype, T, w.rows);
    kernels::gemm_plain(x, w, bias, out, ctx.stream);
    return out;
  }
  Act y = small_batch_linear(ctx, x, w, out_dtype, false, parts_ok);
  if (y.data) return y;
  const bool lib_ok = x.cols % 8 == 0 && (uintptr_t)x.data % 16 == 0;
  if (parts_ok && lib_ok && out_dtype == DType::F32 && ctx.residual_sink && ctx.sink_rows == T && ctx.sink_cols == w.rows &&
      fast_switches().add_in_product) {
    // the residual addition rides on the product's store: one pass over the stream less per norm
    Act sink;
    sink.data = ctx.residual_sink;
    sink.dtype = DType::F32;
    sink.rows = T;
    sink.cols = sink.ld = w.rows;
    sink.part_stride = sink.rows * sink.cols;
    if (library_gemm(ctx.stream, x, w, sink, true)) return sink;
  }
  Act out = ctx.arena->act(out_dtype, T, w.rows);
  if (lib_ok && library_gemm(ctx.stream, x, w, out)) return out;
  if (fast_switches().gemm_tc && kernels::gemm_tc_supported(x, w)) {
    kernels::gemm_tc(x, w, out, false, ctx.tc_status, ctx.stream);
    return out;
  }
  static bool said = false;
  if (!said) {
    said = true;
    log_warning("a bfloat16 product of width %lld runs on the CUDA cores: the tensor-core kernels want a width that is a "
                "multiple of 8", (long long)x.cols);
  }
  kernels::gemm_plain(x, w, nullptr, out, ctx.stream);
  return out;
}

}  // namespace llm
