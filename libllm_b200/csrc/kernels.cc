#include "csrc/kernels.h"

#include <dirent.h>
#include <dlfcn.h>

#include <atomic>
#include <cstdlib>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

namespace llm {
namespace kernels {

namespace {
struct Family {
  std::string path;
  void *handle = nullptr;
  const char *(*last_error)() = nullptr;
};
std::map<std::string, Family> &families() {
  static std::map<std::string, Family> f;
  return f;
}
std::mutex &lock() {
  static std::mutex m;
  return m;
}
std::atomic<long long> g_launches{0};
bool g_manifest_read = false;

std::string own_folder() {
  Dl_info info;
  if (dladdr((void *)&own_folder, &info) && info.dli_fname) {
    std::string p = info.dli_fname;
    const size_t slash = p.rfind('/');
    return slash == std::string::npos ? "." : p.substr(0, slash);
  }
  return ".";
}

void read_manifest_locked() {
  if (g_manifest_read) return;
  g_manifest_read = true;
  const char *env = getenv("LIBLLM_B200_KERNEL_DIR");
  const std::string dir = env && *env ? env : own_folder();
  std::ifstream f(dir + "/kernels.manifest");
  std::string line;
  while (std::getline(f, line)) {
    std::istringstream ls(line);
    std::string fam, path;
    if (!(ls >> fam)) continue;
    std::getline(ls, path);
    const size_t b = path.find_first_not_of(" \t");
    if (b == std::string::npos) continue;
    path = path.substr(b);
    if (path[0] != '/') path = dir + "/" + path;
    if (!families().count(fam)) families()[fam].path = path;
  }
}

Family &open_family(const std::string &name) {
  std::lock_guard<std::mutex> g(lock());
  read_manifest_locked();
  auto it = families().find(name);
  if (it == families().end() || it->second.path.empty())
    LLM_THROW(Extension, "the kernel library '%s' is not built (run `python -m libllm_b200.csrc.build %s`); there is no fallback",
              name.c_str(), name.c_str());
  Family &f = it->second;
  if (!f.handle) {
    f.handle = dlopen(f.path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!f.handle) LLM_THROW(Extension, "cannot load %s: %s", f.path.c_str(), dlerror());
    f.last_error = (const char *(*)())dlsym(f.handle, ("llm_" + name + "_last_error").c_str());
  }
  return f;
}

[[noreturn]] void fail(const std::string &family, const char *fn, int status) {
  Family &f = open_family(family);
  const std::string msg = f.last_error ? f.last_error() : "";
  if (status == STATUS_INVALID_ARG) throw Error(ErrorKind::Unsupported, msg);
  LLM_THROW(Extension, "%s failed (status %#x): %s", fn, status, msg.c_str());
}

template <typename Fn>
Fn resolve(const char *family, const char *name) {
  return (Fn)symbol(family, name);
}

#define LLM_KERNEL(family, name, ...)                                           \
  using name##_fn_t = int (*)(__VA_ARGS__);                                     \
  static name##_fn_t name##_fn() {                                              \
    static name##_fn_t f = resolve<name##_fn_t>(family, #name);                 \
    return f;                                                                   \
  }
#define LLM_CALL(family, name, ...)                                             \
  do {                                                                          \
    g_launches.fetch_add(1, std::memory_order_relaxed);                         \
    const int st_ = name##_fn()(__VA_ARGS__);                                   \
    if (st_ != 0) fail(family, #name, st_);                                     \
  } while (0)

inline int code(DType t) { return (int)t; }
}  // namespace

void set_library(const std::string &family, const std::string &path) {
  std::lock_guard<std::mutex> g(lock());
  Family &f = families()[family];
  if (f.handle && f.path != path)
    LLM_THROW(Extension, "the kernel library '%s' is loaded from %s already", family.c_str(), f.path.c_str());
  f.path = path;
}

bool available(const std::string &family) {
  std::lock_guard<std::mutex> g(lock());
  read_manifest_locked();
  auto it = families().find(family);
  return it != families().end() && !it->second.path.empty();
}

void *symbol(const std::string &family, const std::string &name) {
  Family &f = open_family(family);
  void *p = dlsym(f.handle, name.c_str());
  if (!p) LLM_THROW(Extension, "%s does not export %s (a stale build?)", f.path.c_str(), name.c_str());
  return p;
}

std::vector<std::string> loaded_libraries() {
  std::lock_guard<std::mutex> g(lock());
  std::vector<std::string> out;
  for (const auto &kv : families())
    if (kv.second.handle) out.push_back(kv.second.path);
  return out;
}

long long launches() { return g_launches.load(); }

// ---------------------------------------------------------------- elementwise
LLM_KERNEL("elementwise", llm_embedding, int, const void *, const int *, const int *, const int *, float *, int, int, int, cudaStream_t)
LLM_KERNEL("elementwise", llm_copy_words, const int *, int *, int, cudaStream_t)
LLM_KERNEL("elementwise", llm_gather_words, const int *, int, const int *, int, int *, cudaStream_t)
LLM_KERNEL("elementwise", llm_add_rmsnorm, float *, const void *, int, int, long long, const float *, float, void *, int,
           const int *, int, int, cudaStream_t)
LLM_KERNEL("elementwise", llm_gather_rows_add, const float *, const void *, int, int, long long, const int *, int, float *, int, cudaStream_t)
LLM_KERNEL("elementwise", llm_swiglu, int, int, const void *, void *, int, int, cudaStream_t)
LLM_KERNEL("elementwise", llm_scale_rows, float *, long long, float, cudaStream_t)
LLM_KERNEL("elementwise", llm_logit_transform, float *, long long, float, float, cudaStream_t)
LLM_KERNEL("elementwise", llm_random_fill, void *, int, long long, unsigned long long, int, float, float, cudaStream_t)

void embedding(DType dt, const void *table, const int *tokens, const int *fed_tokens, const int *fed_rows, float *out,
               int n, int hidden, int vocab, cudaStream_t s) {
  LLM_CALL("elementwise", llm_embedding, code(dt), table, tokens, fed_rows ? fed_tokens : nullptr, fed_rows, out, n, hidden, vocab, s);
}
void copy_words(const int *src, int *dst, int n, cudaStream_t s) { LLM_CALL("elementwise", llm_copy_words, src, dst, n, s); }
void gather_words(const int *src1, int n1, const int *src2, int n2, int *dst, cudaStream_t s) {
  LLM_CALL("elementwise", llm_gather_words, src1, n1, src2, n2, dst, s);
}
void add_rmsnorm(float *resid, const Act *delta, const float *weight, float eps, void *out, DType out_dtype, const int *rows,
                 int n_rows, int hidden, cudaStream_t s) {
  const bool has = delta && delta->data;
  LLM_CALL("elementwise", llm_add_rmsnorm, resid, has ? delta->data : nullptr, has ? code(delta->dtype) : 0,
           has ? delta->parts : 0, has ? (long long)delta->part_stride : 0, weight, eps, out, code(out_dtype), rows, n_rows,
           hidden, s);
}
void gather_rows_add(const float *resid, const Act *delta, const int *rows, int n_rows, float *out, int hidden, cudaStream_t s) {
  const bool has = delta && delta->data;
  LLM_CALL("elementwise", llm_gather_rows_add, resid, has ? delta->data : nullptr, has ? code(delta->dtype) : 0, has ? delta->parts : 0,
           has ? (long long)delta->part_stride : 0, rows, n_rows, out, hidden, s);
}
void swiglu(const Act &gu, void *out, DType out_dtype, cudaStream_t s) {
  LLM_CALL("elementwise", llm_swiglu, code(gu.dtype), code(out_dtype), gu.data, out, (int)gu.rows, (int)(gu.cols / 2), s);
}
void scale_rows(float *x, long long n, float scale, cudaStream_t s) { LLM_CALL("elementwise", llm_scale_rows, x, n, scale, s); }
void logit_transform(float *logits, long long n, float scale, float softcap, cudaStream_t s) {
  LLM_CALL("elementwise", llm_logit_transform, logits, n, scale, softcap, s);
}
void random_fill(void *out, DType dtype, long long n, unsigned long long seed, int law, float a, float b, cudaStream_t s) {
  LLM_CALL("elementwise", llm_random_fill, out, code(dtype), n, seed, law, a, b, s);
}

// ---------------------------------------------------------------- products
LLM_KERNEL("gemm_plain", llm_gemm_plain, int, int, const void *, long long, const void *, long long, const float *, void *,
           long long, int, int, int, cudaStream_t)
LLM_KERNEL("gemm_tc", llm_gemm_tc, const void *, long long, const void *, void *, long long, int, int, int, int, int, int,
           long long, int *, cudaStream_t)
LLM_KERNEL("gemv", llm_gemv_bf16, const void *, long long, const void *, void *, long long, int, int, int, int, int, int,
           long long, cudaStream_t)

void gemm_plain(const Act &x, const Weight &w, const float *bias, const Act &out, cudaStream_t s) {
  LLM_CALL("gemm_plain", llm_gemm_plain, code(x.dtype), code(out.dtype), x.data, (long long)x.ld, w.data(), (long long)w.cols,
           bias, out.data, (long long)out.ld, (int)x.rows, (int)w.rows, (int)x.cols, s);
}
bool gemm_tc_supported(const Act &x, const Weight &w) {
  return x.dtype == DType::BF16 && w.dtype == DType::BF16 && x.rows > 0 && x.cols % 8 == 0 && (x.rows == 1 || x.ld % 8 == 0) &&
         (uintptr_t)x.data % 16 == 0 && (uintptr_t)w.data() % 16 == 0;
}
int gemm_tc_suggest_parts(int M, int N, int K) {
  static auto f = resolve<int (*)(int, int, int)>("gemm_tc", "llm_gemm_tc_suggest_parts");
  return f(M, N, K);
}
void gemm_tc(const Act &x, const Weight &w, const Act &out, bool swiglu, int *status, cudaStream_t s) {
  LLM_CALL("gemm_tc", llm_gemm_tc, x.data, (long long)(x.rows > 1 ? x.ld : x.cols), w.data(), out.data,
           (long long)(x.rows > 1 ? out.ld : out.cols), code(out.dtype), (int)x.rows, (int)w.rows, (int)x.cols, swiglu ? 1 : 0,
           out.parts, (long long)out.part_stride, status, s);
}
LLM_KERNEL("gemm_tc", llm_gemm_tc_wait_probe, long long, int *, cudaStream_t)
void gemm_tc_wait_probe(long long limit_ns, int *status, cudaStream_t s) { LLM_CALL("gemm_tc", llm_gemm_tc_wait_probe, limit_ns, status, s); }
LLM_KERNEL("gemm_chain", llm_gemm_chain, const ChainJob *, int, int *, int *, cudaStream_t)
static int chain_limit(const char *name) {
  return resolve<int (*)()>("gemm_chain", name)();
}
int gemm_chain_max_jobs() {
  static const int v = chain_limit("llm_gemm_chain_max_jobs");
  return v;
}
int gemm_chain_max_tokens() {
  static const int v = chain_limit("llm_gemm_chain_max_tokens");
  return v;
}
int gemm_chain_max_hidden() {
  static const int v = chain_limit("llm_gemm_chain_max_hidden");
  return v;
}
int gemm_chain_counters() {
  static const int v = chain_limit("llm_gemm_chain_counters");
  return v;
}
void gemm_chain(const ChainJob *jobs, int n_jobs, int *counters, int *status, cudaStream_t s) {
  LLM_CALL("gemm_chain", llm_gemm_chain, jobs, n_jobs, counters, status, s);
}
bool gemv_supported(const Act &x, const Weight &w) {
  return x.dtype == DType::BF16 && w.dtype == DType::BF16 && x.rows > 0 && x.rows <= 64 && x.cols % 8 == 0 && x.ld % 8 == 0 &&
         (uintptr_t)x.data % 16 == 0 && (uintptr_t)w.data() % 16 == 0;
}
int gemv_suggest_parts(int M, int N, int K) {
  static auto f = resolve<int (*)(int, int, int)>("gemv", "llm_gemv_suggest_parts");
  return f(M, N, K);
}
void gemv_bf16(const Act &x, const Weight &w, const Act &out, bool swiglu, cudaStream_t s) {
  LLM_CALL("gemv", llm_gemv_bf16, x.data, (long long)(x.rows > 1 ? x.ld : x.cols), w.data(), out.data,
           (long long)(x.rows > 1 ? out.ld : out.cols), code(out.dtype), (int)x.rows, (int)w.rows, (int)x.cols, swiglu ? 1 : 0,
           out.parts, (long long)out.part_stride, s);
}

// ---------------------------------------------------------------- rotation and cache append
LLM_KERNEL("rope", llm_rope_cache_write, int, int, const void *, long long, void *, long long, int, int, int, int, const float *,
           int, int, const int *, const int *, const int *, int, void *, void *, int, int, cudaStream_t)

void rope_cache_write(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, const float *table, int table_rows,
                      int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride, void *kcache,
                      void *vcache, int page_size, bool write_cache, cudaStream_t s) {
  LLM_CALL("rope", llm_rope_cache_write, code(qkv.dtype), code(q_out.dtype), qkv.data, (long long)qkv.ld, q_out.data,
           (long long)q_out.ld, (int)qkv.rows, n_heads, n_kv, d, table, table_rows, rot_dim, tok_seq, tok_pos, page_table,
           pt_stride, kcache, vcache, page_size, write_cache ? 1 : 0, s);
}

// ---------------------------------------------------------------- attention
LLM_KERNEL("attention_generic", llm_attention_generic, int, const void *, long long, void *, long long, const void *, const void *,
           const int *, const int *, const int *, int, int, int, int, int, int, int, float, cudaStream_t)
LLM_KERNEL("attention_decode", llm_attention_decode, const void *, long long, void *, long long, const void *, const void *,
           const int *, const int *, int, int, int, int, int, int, int, int, int, float, float *, float *, cudaStream_t)
LLM_KERNEL("attention_decode_tc", llm_attention_decode_tc, const float *, long long, int, long long, const float *, int, int,
           const int *, const int *, int, void *, void *, int, int, int, int, int, int, int, int, int, int, float, float *,
           float *, int *, void *, long long, cudaStream_t)
LLM_KERNEL("attention_prefill", llm_attention_prefill, const void *, long long, void *, long long, const void *, const void *,
           const int *, const int *, const int *, int, int, int, int, int, int, int, int, float, cudaStream_t)
LLM_KERNEL("attention_prefill_tc", llm_attention_prefill_tc, const void *, long long, long long, void *, long long, const void *,
           const void *, long long, const int *, const int *, const int *, int, int, int, int, int, int, int, int, float, int,
           int *, cudaStream_t)

void attention_generic(const Act &q, const Act &out, const void *kc, const void *vc, const int *tok_seq, const int *tok_pos,
                       const int *page_table, int pt_stride, int n_heads, int n_kv, int d, int page_size, int window,
                       float scale, cudaStream_t s) {
  LLM_CALL("attention_generic", llm_attention_generic, code(q.dtype), q.data, (long long)q.ld, out.data, (long long)out.ld, kc, vc,
           tok_seq, tok_pos, page_table, pt_stride, (int)q.rows, n_heads, n_kv, d, page_size, window, scale, s);
}
bool attention_decode_supported(int d, int group) {
  static auto f = resolve<int (*)(int, int)>("attention_decode", "llm_attention_decode_supports");
  return f(d, group) != 0;
}
void attention_decode(const Act &q, const Act &out, const void *kc, const void *vc, const int *tok_pos, const int *page_table,
                      int pt_stride, int n_heads, int n_kv, int d, int page_size, int chunk, int n_splits, int window,
                      float scale, float *ws_o, float *ws_ml, cudaStream_t s) {
  const int B = (int)q.rows;
  LLM_CALL("attention_decode", llm_attention_decode, q.data, (long long)(B > 1 ? q.ld : q.cols), out.data,
           (long long)(B > 1 ? out.ld : out.cols), kc, vc, tok_pos, page_table, pt_stride, B, n_heads, n_kv, d, page_size, chunk,
           n_splits, window, scale, ws_o, ws_ml, s);
}
bool attention_decode_tc_supported(int d, int page_size, int group) {
  static auto f = resolve<int (*)(int, int, int)>("attention_decode_tc", "llm_attention_decode_tc_supports");
  return f(d, page_size, group) != 0;
}
int attention_decode_tc_ctas_per_sm(int d) {
  static auto f = resolve<int (*)(int)>("attention_decode_tc", "llm_attention_decode_tc_ctas_per_sm");
  return f(d);
}
void attention_decode_tc(const Act &qkv, const float *table, int table_rows, int rot_dim, const int *tok_pos,
                         const int *page_table, int pt_stride, void *kc, void *vc, bool write_cache, int n_seqs, int n_heads,
                         int n_kv, int d, int page_size, int chunk, int max_len, int n_splits, int window, float scale,
                         float *ws_o, float *ws_ml, int *counters, const Act &out, cudaStream_t s) {
  LLM_CALL("attention_decode_tc", llm_attention_decode_tc, (const float *)qkv.data, (long long)(n_seqs > 1 ? qkv.ld : qkv.cols),
           qkv.parts, (long long)qkv.part_stride, table, table_rows, rot_dim, tok_pos, page_table, pt_stride, kc, vc,
           write_cache ? 1 : 0, n_seqs, n_heads, n_kv, d, page_size, chunk, max_len, n_splits, window, scale, ws_o, ws_ml,
           counters, out.data, (long long)(n_seqs > 1 ? out.ld : out.cols), s);
}
bool attention_prefill_supported(int d, int page_size) {
  static auto f = resolve<int (*)(int, int)>("attention_prefill", "llm_attention_prefill_supports");
  return f(d, page_size) != 0;
}
void attention_prefill(const Act &q, const Act &out, const void *kc, const void *vc, const int *seq_start, const int *seq_past,
                       const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads, int n_kv, int d,
                       int page_size, int window, float scale, cudaStream_t s) {
  LLM_CALL("attention_prefill", llm_attention_prefill, q.data, (long long)q.ld, out.data, (long long)out.ld, kc, vc, seq_start,
           seq_past, page_table, pt_stride, n_seqs, max_q_len, n_heads, n_kv, d, page_size, window, scale, s);
}
bool attention_prefill_tc_supported(int d, int page_size) {
  static auto f = resolve<int (*)(int, int)>("attention_prefill_tc", "llm_attention_prefill_tc_supports");
  return f(d, page_size) != 0;
}
void attention_prefill_tc(const Act &q, const Act &out, const void *kc, const void *vc, long long n_pages, const int *seq_start,
                          const int *seq_past, const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads,
                          int n_kv, int d, int page_size, int window, float scale, int *status, cudaStream_t s) {
  LLM_CALL("attention_prefill_tc", llm_attention_prefill_tc, q.data, (long long)q.ld, (long long)q.rows, out.data,
           (long long)out.ld, kc, vc, n_pages, seq_start, seq_past, page_table, pt_stride, n_seqs, max_q_len, n_heads, n_kv, d,
           page_size, window, scale, 0, status, s);
}

// ---------------------------------------------------------------- sampling
LLM_KERNEL("sampling", llm_argmax, const float *, long long, int, int, int *, cudaStream_t)
LLM_KERNEL("sampling", llm_sample, const float *, long long, int, int, float, int, float, const float *, int *, cudaStream_t)

void argmax(const float *logits, long long stride, int n_rows, int vocab, int *out, cudaStream_t s) {
  LLM_CALL("sampling", llm_argmax, logits, stride, n_rows, vocab, out, s);
}
void sample(const float *logits, long long stride, int n_rows, int vocab, float temperature, int top_k, float top_p,
            const float *uniforms, int *out, cudaStream_t s) {
  LLM_CALL("sampling", llm_sample, logits, stride, n_rows, vocab, temperature, top_k, top_p, uniforms, out, s);
}

}  // namespace kernels
}  // namespace llm
