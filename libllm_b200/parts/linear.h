// y = x @ W^T (+ b) for the parts: picks the matrix product for the engine's type.
//
// float32: the plain CUDA-core product with 32-bit accumulation (no tensor cores, no
// reduced-precision mode).  bfloat16: the hand-written tcgen05 product when the step has few
// tokens, the library product (cuBLAS) otherwise, as the reference calls cuBLAS for its products
// (src/flint/cuda/gemm_cublas.cc:160-197) and a kernel of its own when one row is multiplied
// (src/flint/cuda/matvec.cu:61-87).
#pragma once
#include "parts/part.h"

namespace llm {

// Switches read once from the environment, so that a kernel can be compared with the general one.
struct FastSwitches {
  bool gemm_tc = true, gemv = true, decode_attention = true, prefill_attention = true, prefill_attention_tc = true,
       decode_attention_tc = true, library_gemm = true;
  bool add_in_product = true;          // prompt steps: the library product adds its result to the residual stream itself
  bool gemm_chain = false;             // queue a decoding step's products and norms into single launches (parts/chain.h)
  int tc_tokens = 256;                 // steps of up to this many tokens take the tcgen05 product
  int fused_gate_up_tokens = 1024;     // prompt steps from this many tokens fuse SwiGLU into the product ...
  int fused_gate_up_max_k = 3072;      // ... when the width is at most this
  int gemv_tokens = 0;                 // steps of up to this many tokens take the mma.sync weight streamer
};
const FastSwitches &fast_switches();

// Kernel families that the products of an engine of this type launch.
std::vector<std::string> product_families(DType dtype);

// x [T, K] in the engine's type, w [N, K]; returns [T, N] in out_dtype.  With parts_ok (for
// results that go into the residual addition, which adds parts in order) the result may be
// [parts, T, N] partial products to be summed, or, when the block has named the residual
// stream's rows (StepContext::residual_sink) and the library product runs, the stream itself with
// the result already added to it.
Act linear(StepContext &ctx, const Act &x, const Weight &w, const float *bias, DType out_dtype, bool parts_ok = false);

// The product for steps of few tokens; data == nullptr when it does not take the case.  With
// `swiglu`, w is the stacked gate|up matrix [2I, K] and the result is silu(gate) * up, [T, I].
Act small_batch_linear(StepContext &ctx, const Act &x, const Weight &w, DType out_dtype, bool swiglu, bool parts_ok);

// out[T, N] = x[T, K] @ w[N, K]^T by cuBLAS (bfloat16 operands, 32-bit accumulation); false when
// the library is not to be had.
// With `accumulate` the product is added to what `out` holds (32-bit out).
bool library_gemm(cudaStream_t stream, const Act &x, const Weight &w, const Act &out, bool accumulate = false);
bool library_gemm_available();

}  // namespace llm
