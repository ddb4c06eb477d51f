// Products and norms of a decoding step, queued and launched together.
//
// A step of one token per sequence is a string of small dependent launches.  While a Chain is
// attached to the step (StepContext::chain), linear() and the RMSNorm do not launch: they append
// a job and hand back the buffer the job will fill.  flush() turns the queue into one launch of
// the chained kernel (libllm_b200/csrc/gemm_chain.cu), which runs the jobs in order and lets each
// wait, inside the kernel, for the job whose output it reads.  Whoever is about to launch
// anything else on the step's stream, or to hand a buffer to code outside the library, calls
// flush_chain() first: the attention, parts that come through the plug-in interface, the end of
// the model's forward pass.  A job that the kernel does not take (another type, too many tokens,
// a width it has no room for) is refused by add_*(), and the caller flushes and launches as it
// would without a chain.
#pragma once
#include <vector>

#include "csrc/kernels.h"
#include "parts/part.h"

namespace llm {

class Chain {
 public:
  Chain(int *counters, int *status) : counters_(counters), status_(status) {}
  // out = x w^T (32-bit, out.parts parts of K), or silu(gate) * up of the stacked product (bfloat16).
  bool add_product(const Act &x, const Weight &w, const Act &out, bool swiglu, cudaStream_t stream);
  // v = resid + delta's parts; resid = v unless `rows`; out = RMSNorm(v) in bfloat16.
  bool add_norm(float *resid, const Act *delta, const float *weight, float eps, void *out, const int *rows, int n_rows,
                int hidden, cudaStream_t stream);
  void flush(cudaStream_t stream);
  bool empty() const { return jobs_.empty(); }
  long long launches() const { return launches_; }

 private:
  struct Span {
    const char *begin, *end;
  };
  int writer_of(const void *p) const;            // the last job that writes the buffer p lies in; -1: none
  void push(const kernels::ChainJob &job, Span written, Span also_written, cudaStream_t stream);
  std::vector<kernels::ChainJob> jobs_;
  std::vector<Span> written_, also_written_;
  int *counters_, *status_;
  long long launches_ = 0;
};

inline void flush_chain(StepContext &ctx) {
  if (ctx.chain) ctx.chain->flush(ctx.stream);
}

}  // namespace llm
