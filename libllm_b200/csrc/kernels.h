// The host library's view of the kernel libraries: one C++ function per exported kernel.
//
// Each family of kernels (libllm_b200/csrc/*.cu) is a shared library of its own, built by
// libllm_b200/csrc/build.py for sm_100a when something first needs it.  The host library opens a
// family when one of its functions is first called and turns a non-zero status into an llm::Error
// that carries the family's own message.  There is no fallback: a family that is not built, or
// that cannot be loaded, is an error that says so.
#pragma once
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "util/device.h"

namespace llm {
namespace kernels {

// Where a family's library lies.  Set by whoever built them (the Python package after
// csrc/build.py ran); otherwise the file `kernels.manifest` (lines "family path") in the folder
// named by LIBLLM_B200_KERNEL_DIR, or else in the folder of this library itself, is read.
void set_library(const std::string &family, const std::string &path);
bool available(const std::string &family);
void *symbol(const std::string &family, const std::string &name);
std::vector<std::string> loaded_libraries();

// ---- elementwise
void embedding(DType table_dtype, const void *table, const int *tokens, const int *fed_tokens, const int *fed_rows,
               float *out, int n_tokens, int hidden, int vocab, cudaStream_t s);
void copy_words(const int *src, int *dst, int n, cudaStream_t s);
void gather_words(const int *src1, int n1, const int *src2, int n2, int *dst, cudaStream_t s);
void add_rmsnorm(float *resid, const Act *delta, const float *weight, float eps, void *out, DType out_dtype,
                 const int *rows, int n_rows, int hidden, cudaStream_t s);
// out[i] = resid[rows[i]] + delta's parts at that row (32-bit)
void gather_rows_add(const float *resid, const Act *delta, const int *rows, int n_rows, float *out, int hidden, cudaStream_t s);
void swiglu(const Act &gu, void *out, DType out_dtype, cudaStream_t s);
void scale_rows(float *x, long long n, float scale, cudaStream_t s);
void logit_transform(float *logits, long long n, float scale, float softcap, cudaStream_t s);
void random_fill(void *out, DType dtype, long long n, unsigned long long seed, int law, float a, float b, cudaStream_t s);
// ---- products
void gemm_plain(const Act &x, const Weight &w, const float *bias, const Act &out, cudaStream_t s);
bool gemm_tc_supported(const Act &x, const Weight &w);
int gemm_tc_suggest_parts(int M, int N, int K);
void gemm_tc(const Act &x, const Weight &w, const Act &out, bool swiglu, int *status, cudaStream_t s);
void gemm_tc_wait_probe(long long limit_ns, int *status, cudaStream_t s);
// One job of a chain of products and norms run as one launch (csrc/gemm_chain.cu, which has the
// same structure under the name llm_chain_job).
struct ChainJob {
  int kind;                 // 0 product, 1 SwiGLU product, 2 add + RMSNorm
  int dep0, dep1;           // jobs of the chain that must be complete first; -1: none
  const void *x;
  long long ldx;
  const void *w;
  void *out;
  long long ldo;
  int M, N, K, k_parts;
  long long part_stride;
  float *resid;
  const float *delta;
  int delta_parts;
  long long delta_stride;
  const float *weight;
  float eps;
  const int *rows;
  int n_rows, hidden;
};
int gemm_chain_max_jobs();
int gemm_chain_max_tokens();
int gemm_chain_max_hidden();
int gemm_chain_counters();
void gemm_chain(const ChainJob *jobs, int n_jobs, int *counters, int *status, cudaStream_t s);
bool gemv_supported(const Act &x, const Weight &w);
int gemv_suggest_parts(int M, int N, int K);
void gemv_bf16(const Act &x, const Weight &w, const Act &out, bool swiglu, cudaStream_t s);
// ---- rotation and cache append
void rope_cache_write(const Act &qkv, const Act &q_out, int n_heads, int n_kv, int d, const float *table, int table_rows,
                      int rot_dim, const int *tok_seq, const int *tok_pos, const int *page_table, int pt_stride,
                      void *kcache, void *vcache, int page_size, bool write_cache, cudaStream_t s);
// ---- attention
void attention_generic(const Act &q, const Act &out, const void *kc, const void *vc, const int *tok_seq, const int *tok_pos,
                       const int *page_table, int pt_stride, int n_heads, int n_kv, int d, int page_size, int window,
                       float scale, cudaStream_t s);
bool attention_decode_supported(int d, int group);
void attention_decode(const Act &q, const Act &out, const void *kc, const void *vc, const int *tok_pos, const int *page_table,
                      int pt_stride, int n_heads, int n_kv, int d, int page_size, int chunk, int n_splits, int window,
                      float scale, float *ws_o, float *ws_ml, cudaStream_t s);
bool attention_decode_tc_supported(int d, int page_size, int group);
int attention_decode_tc_ctas_per_sm(int d);
void attention_decode_tc(const Act &qkv, const float *table, int table_rows, int rot_dim, const int *tok_pos,
                         const int *page_table, int pt_stride, void *kc, void *vc, bool write_cache, int n_seqs, int n_heads,
                         int n_kv, int d, int page_size, int chunk, int max_len, int n_splits, int window, float scale,
                         float *ws_o, float *ws_ml, int *counters, const Act &out, cudaStream_t s);
bool attention_prefill_supported(int d, int page_size);
void attention_prefill(const Act &q, const Act &out, const void *kc, const void *vc, const int *seq_start, const int *seq_past,
                       const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads, int n_kv, int d,
                       int page_size, int window, float scale, cudaStream_t s);
bool attention_prefill_tc_supported(int d, int page_size);
void attention_prefill_tc(const Act &q, const Act &out, const void *kc, const void *vc, long long n_pages, const int *seq_start,
                          const int *seq_past, const int *page_table, int pt_stride, int n_seqs, int max_q_len, int n_heads,
                          int n_kv, int d, int page_size, int window, float scale, int *status, cudaStream_t s);
// ---- sampling
void argmax(const float *logits, long long stride, int n_rows, int vocab, int *out, cudaStream_t s);
void sample(const float *logits, long long stride, int n_rows, int vocab, float temperature, int top_k, float top_p,
            const float *uniforms, int *out, cudaStream_t s);

// Kernel launches issued through this file since the process started (graph replays not counted).
long long launches();

}  // namespace kernels
}  // namespace llm
