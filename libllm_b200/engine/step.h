// The step function: a batch of sequences, each bringing its next tokens (a whole prompt, a piece
// of one, or a single token), run as one batch from the cache.
//
// The reference has two entry points for one sequence, `prefill` and `decode`
// (src/libllm/model_for_generation.h:62-69, src/libllm/llama.cc:349-368), and a rectangular batch
// inside the model.  Here one function takes ragged batches: the tokens of all sequences lie one
// after another, per-token arrays say which sequence and position each belongs to, and the
// kernels index the paged cache with them.  Only the tokens given are computed; padding does not
// exist.
//
// Steps in which every sequence brings one token are captured once per batch shape as a CUDA
// graph and replayed; the graph's first kernel brings the step's descriptor (tokens, positions,
// page tables) from pinned host memory into the graph's fixed buffer, its last one takes the
// sampled tokens and the tensor-core kernels' status word out.  Prompt steps are launched one
// kernel after another: their kernels are long enough for the host to stay ahead.
#pragma once
#include <map>
#include <memory>
#include <vector>

#include "engine/model.h"

namespace llm {

// One sequence's share of a step: its slot, its next tokens, and the places among these tokens
// whose logits are wanted.
struct StepItem {
  int slot = 0;
  std::vector<int> tokens;
  std::vector<int> want;
  int fed_row = -1;          // >= 0: its one token is the one the previous step sampled for this row
};

// temperature 0 is greedy; top_k 0 draws from the whole vocabulary.  The defaults are the
// reference's (src/libllm/llm.cc:125-132).
struct SamplingParams {
  float temperature = 1.0f;
  int top_k = 50;
  float top_p = 0.8f;
  void validate() const;
  bool greedy() const { return temperature == 0.f; }
  bool operator<(const SamplingParams &o) const {
    if (temperature != o.temperature) return temperature < o.temperature;
    if (top_k != o.top_k) return top_k < o.top_k;
    return top_p < o.top_p;
  }
};

class Engine;

// What a step leaves on the device.  The memory is the engine's: the next step (for a step of
// single tokens, the step after next of the same shape) writes it again.
struct StepResult {
  const float *logits = nullptr;     // [n_rows, vocab], 32-bit, in the order of the items and of their `want`
  int n_rows = 0;
  const int *tokens = nullptr;       // [n_rows] when the step sampled
};

// Tokens of a step on their way from the device to the host.
class PendingTokens {
 public:
  PendingTokens() = default;
  bool valid() const { return engine_ != nullptr; }
  int size() const { return n_; }
  // Waits for the copy; throws Error(Extension) if a tensor-core kernel of the step gave up
  // waiting on a barrier (its results are then not valid).
  std::vector<int> result();

 private:
  friend class Engine;
  Engine *engine_ = nullptr;
  int n_ = 0;
  const int *host_ = nullptr;        // n tokens, then the status word
  cudaEvent_t done_ = nullptr;
};

class Engine {
 public:
  struct Options {
    int64_t max_tokens = 65536;      // tokens all live sequences may hold together (each rounded up to a page): sizes the cache
    int64_t max_seq_len = 0;         // 0: the model's own
    int max_slots = 0;               // 0: one per page
    int max_step_tokens = 8192;      // a step with more tokens is cut into pieces of this many
    int page_size = 64;
    bool use_graphs = true;
    int device = 0;
  };
  Engine(std::unique_ptr<Model> model, const Options &options);
  ~Engine();
  Engine(const Engine &) = delete;
  Engine &operator=(const Engine &) = delete;

  Model &model() { return *model_; }
  KVCache &cache() { return *cache_; }
  const Options &options() const { return opt_; }
  int64_t max_seq_len() const { return max_seq_len_; }
  int64_t vocab() const { return model_->spec().vocab_size; }
  cudaStream_t stream() const { return stream_; }
  int device() const { return opt_.device; }
  void make_current() const;

  int open_sequence();
  void close_sequence(int slot);
  int sequence_length(int slot) const { return cache_->length(slot); }

  // Runs the items' tokens.  Without `sampling` the result holds the logits at the wanted places.
  // With it, a token is drawn at each wanted place; `uniforms` then holds one number in [0, 1) per
  // wanted place (null: zeros).  Returns when the work is queued on the engine's stream.
  StepResult step(const std::vector<StepItem> &items, const SamplingParams *sampling = nullptr, const float *uniforms = nullptr);
  // Copies a step's logits to host memory, waits, and checks the status word.
  void read_logits(const StepResult &r, float *host);
  void read_tokens(const StepResult &r, int *host);

  // Runs a step that samples one token per item (each wants exactly one place) and returns at
  // once: the tokens stay on the device (row i = item i), where the next step's items may take
  // them from (StepItem::fed_row), and are on their way to pinned host memory.
  PendingTokens step_tokens(const std::vector<StepItem> &items, const SamplingParams &sampling, const float *uniforms);

  void synchronize();
  // Reads the status word (waits for the device); throws if a kernel gave up waiting since the last check.
  void check_status();
  int *status_word() const { return status_.as<int>(); }

  long long steps_run() const { return steps_run_; }
  long long graphs_captured() const { return graphs_captured_; }
  long long graph_replays() const { return graph_replays_; }
  long long chain_launches() const;   // launches of queued products and norms (outside graph replays)
  int last_tokens_capacity() const { return last_capacity_; }
  // Bytes the last step brought from pinned host memory to the device (its descriptor) and from
  // the device to the host by itself (a single-token step's sampled tokens and status word).
  long long last_step_h2d_bytes() const { return last_h2d_; }
  long long last_step_d2h_bytes() const { return last_d2h_; }

 private:
  friend class PendingTokens;
  struct Piece {
    int index, slot, start, count, past;
  };
  class Descriptor;
  struct DecodeGraph;
  struct GraphKey {
    int batch, width;
    bool sampled;
    SamplingParams sampling;
    bool operator<(const GraphKey &o) const;
  };

  void validate(const std::vector<StepItem> &items) const;
  void fill(Descriptor &d, const std::vector<Piece> &pieces, const std::vector<StepItem> &items, const std::vector<int> &want_rows,
            const float *uniforms, int n_uniforms);
  StepContext context(Descriptor &d, const std::vector<Piece> &pieces, int n_want, bool decode_only, int max_kv_len, Arena *arena,
                      std::vector<const int *> *tables);
  void sample(const Act &logits, const SamplingParams &s, const float *uniforms_dev, int *out);
  StepResult run_eager(const std::vector<StepItem> &items, const SamplingParams *sampling, const float *uniforms);
  StepResult run_decode_graph(const std::vector<StepItem> &items, const SamplingParams *sampling, const float *uniforms);
  Act graph_body(DecodeGraph &g);
  void raise_status(int code);

  std::unique_ptr<Model> model_;
  Options opt_;
  int64_t max_seq_len_ = 0;
  std::unique_ptr<KVCache> cache_;
  cudaStream_t stream_ = nullptr;
  int sm_count_ = 148;
  Arena scratch_, results_, layer_scratch_[2];
  DeviceBuffer status_, counters_, last_tokens_;
  std::unique_ptr<Chain> chain_;     // the queue of the step being launched (parts/chain.h)
  int last_capacity_ = 0;
  std::vector<std::unique_ptr<Descriptor>> eager_desc_;
  size_t eager_turn_ = 0;
  struct HostTokens {
    PinnedBuffer buf;
    cudaEvent_t done = nullptr;
  };
  std::vector<HostTokens> token_ring_;
  size_t token_turn_ = 0;
  PinnedBuffer status_host_;
  std::map<GraphKey, std::unique_ptr<DecodeGraph>> graphs_[2];
  std::map<GraphKey, int> graph_turn_;
  DecodeGraph *last_graph_ = nullptr;
  long long chain_launches_ = 0;
  long long steps_run_ = 0, graphs_captured_ = 0, graph_replays_ = 0, last_h2d_ = 0, last_d2h_ = 0;
};

}  // namespace llm
