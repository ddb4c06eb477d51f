// The generation loop above the step function.
//
// The reference's loop serves one sequence: stop if the current token is a stop token, prefill or
// decode, pick the next token, stop if that is a stop token; the stop token is never handed out
// (src/libllm/generator.cc:140-156).  This loop does the same for many requests: it forms batches
// of unequal prompts, runs each batch's prompts in one step and then one token per live sequence
// per step, drops sequences as they end (their slots and pages go back at once) and starts the
// next batch when a batch is done.
#pragma once
#include <functional>
#include <set>
#include <vector>

#include "engine/step.h"

namespace llm {

// Splits requests, in order, into batches that fit the cache when every sequence grows to its
// full length (prompt + new tokens, rounded up to whole pages).  A request that cannot fit alone
// is an error.
std::vector<std::vector<int>> plan_batches(const std::vector<int> &prompt_lengths, const std::vector<int> &max_new_tokens,
                                           int64_t capacity_tokens, int max_batch, int page_size = 64, int64_t max_seq_len = 0);

// (ends, emit): a stop token ends the sequence and is not emitted; reaching the limit ends it
// after emitting.
struct StopDecision {
  bool ends, emit;
};
StopDecision should_stop(int token, int n_generated, int max_new_tokens, const std::set<int> &stop_tokens);

struct GenerateOptions {
  SamplingParams sampling;
  uint64_t seed = 0;
  bool use_model_stop_tokens = true;       // false: `stop_tokens` instead of the model's own
  std::vector<int> stop_tokens;
  int max_batch = 64;
  std::function<void(int request, int token)> on_token;
};

// Generated tokens per prompt.  `max_new_tokens` holds one number, or one per prompt.
std::vector<std::vector<int>> generate(Engine &engine, const std::vector<std::vector<int>> &prompts,
                                       const std::vector<int> &max_new_tokens, const GenerateOptions &options);

// One prompt completed token by token, in the manner of the reference's completion handle
// (src/libllm/llm.cc:266-308): next() hands out one token per call until the sequence ends.
class Completion {
 public:
  Completion(Engine &engine, std::vector<int> prompt, int max_new_tokens, const SamplingParams &sampling, uint64_t seed,
             const std::set<int> &stop_tokens);
  ~Completion();
  // False when the sequence has ended (a stop token, the limit, or the longest sequence).
  bool next(int *token);

 private:
  void finish();
  Engine &engine_;
  std::vector<int> prompt_;
  int limit_;
  SamplingParams sampling_;
  uint64_t seed_;
  std::set<int> stops_;
  int slot_ = -1;
  int produced_ = 0;
  bool started_ = false, ended_ = false;
  PendingTokens running_;
};

}  // namespace llm
