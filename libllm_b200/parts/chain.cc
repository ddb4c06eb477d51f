#include "parts/chain.h"

namespace llm {

int Chain::writer_of(const void *p) const {
  const char *c = (const char *)p;
  for (int j = (int)jobs_.size() - 1; j >= 0; --j) {
    if (c >= written_[(size_t)j].begin && c < written_[(size_t)j].end) return j;
    if (c >= also_written_[(size_t)j].begin && c < also_written_[(size_t)j].end) return j;
  }
  return -1;
}

void Chain::push(const kernels::ChainJob &job, Span written, Span also_written, cudaStream_t stream) {
  if ((int)jobs_.size() >= kernels::gemm_chain_max_jobs()) flush(stream);
  jobs_.push_back(job);
  written_.push_back(written);
  also_written_.push_back(also_written);
}

bool Chain::add_product(const Act &x, const Weight &w, const Act &out, bool swiglu, cudaStream_t stream) {
  if (x.rows > kernels::gemm_chain_max_tokens() || !kernels::gemm_tc_supported(x, w)) return false;
  if (swiglu ? (out.dtype != DType::BF16 || out.parts != 1) : out.dtype != DType::F32) return false;
  if ((int)jobs_.size() >= kernels::gemm_chain_max_jobs()) flush(stream);      // before the writers are looked up
  kernels::ChainJob job = {};
  job.kind = swiglu ? 1 : 0;
  job.dep0 = writer_of(x.data);
  job.dep1 = -1;
  job.x = x.data;
  job.ldx = x.rows > 1 ? x.ld : x.cols;
  job.w = w.data();
  job.out = out.data;
  job.ldo = x.rows > 1 ? out.ld : out.cols;
  job.M = (int)x.rows;
  job.N = (int)w.rows;
  job.K = (int)x.cols;
  job.k_parts = out.parts;
  job.part_stride = out.part_stride;
  const size_t bytes = out.parts > 1 ? (size_t)out.parts * (size_t)out.part_stride * dtype_size(out.dtype)
                                     : (size_t)out.rows * (size_t)out.ld * dtype_size(out.dtype);
  push(job, Span{(const char *)out.data, (const char *)out.data + bytes}, Span{nullptr, nullptr}, stream);
  return true;
}

bool Chain::add_norm(float *resid, const Act *delta, const float *weight, float eps, void *out, const int *rows, int n_rows,
                     int hidden, cudaStream_t stream) {
  const bool has = delta && delta->data;
  if (hidden % 4 != 0 || hidden > kernels::gemm_chain_max_hidden() || n_rows <= 0 || !out) return false;
  if (has && (delta->dtype != DType::F32 || delta->parts > 8 || delta->part_stride % 4 != 0)) return false;
  if ((int)jobs_.size() >= kernels::gemm_chain_max_jobs()) flush(stream);
  kernels::ChainJob job = {};
  job.kind = 2;
  job.dep0 = has ? writer_of(delta->data) : -1;
  job.dep1 = writer_of(resid);
  if (job.dep1 == job.dep0) job.dep1 = -1;
  job.out = out;
  job.resid = resid;
  job.delta = has ? (const float *)delta->data : nullptr;
  job.delta_parts = has ? delta->parts : 0;
  job.delta_stride = has ? delta->part_stride : 0;
  job.weight = weight;
  job.eps = eps;
  job.rows = rows;
  job.n_rows = n_rows;
  job.hidden = hidden;
  // The norm of all rows moves the residual stream on; the rows it may touch are not known here
  // when `rows` picks them, and then it does not write the stream at all.
  Span stream_rows{nullptr, nullptr};
  if (!rows && has) stream_rows = Span{(const char *)resid, (const char *)(resid + (size_t)n_rows * (size_t)hidden)};
  push(job, Span{(const char *)out, (const char *)out + (size_t)n_rows * (size_t)hidden * 2}, stream_rows, stream);
  return true;
}

void Chain::flush(cudaStream_t stream) {
  if (jobs_.empty()) return;
  std::vector<kernels::ChainJob> jobs;
  jobs.swap(jobs_);
  written_.clear();
  also_written_.clear();
  ++launches_;
  kernels::gemm_chain(jobs.data(), (int)jobs.size(), counters_, status_, stream);
}

}  // namespace llm
