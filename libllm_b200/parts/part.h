// Interfaces of the parts a layer is put together from, what a step hands them, and the
// registry of part classes.
//
//   Norm              residual stream (+ pending addition) -> normalised activations
//   PositionEncoding  places tokens for a mixer: rotates q and k and appends k, v to the cache
//   Mixer             mixes along the sequence; may keep keys/values in the cache (cache_need)
//                     and fixed-size state per sequence (state_need)
//   FeedForward       acts on each token alone
//   Block             joins a mixer and a feed-forward to the residual stream
//
// Every part takes its sizes and constants from its description (a JSON object, see
// libllm_b200/parts/spec.h), states the tensors it needs by name (tensor_needs) and receives
// them through load().  No part knows which model it is in.  Activations are [tokens, width]
// with the step's tokens of all sequences one after another; which token belongs to which
// sequence and position is in StepContext.  A constructor touches no device: a model can be
// built on a machine without one to ask what tensors it needs.
//
// The reference has one class per part of its one architecture (src/libllm/llama.cc:81-267,
// src/libllm/layers.cc:36-112) and no registry.
#pragma once
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "parts/spec.h"
#include "util/device.h"
#include "util/json.h"
#include "weights/state_map.h"

namespace llm {

class Arena;
class Chain;

// What a part may know about the engine it is built for.
struct BuildEnv {
  DType dtype = DType::BF16;         // the engine's type: float32 or bfloat16
  int64_t max_positions = 0;         // longest sequence the engine will hold
  int page_size = 64;
  // Tables that several parts with the same description share (one rotary table per model, not
  // one per layer): key -> weight.  Filled by the parts themselves at load().
  std::map<std::string, std::shared_ptr<Weight>> *shared = nullptr;
};

// Keys and values a mixer wants kept per sequence.  kind "full" keeps every position, "window"
// only the last `window` (older pages are given back).  Keys and values have widths of their
// own; v_dim 0 keeps one vector per position (a latent) in the key storage alone.
struct CacheNeed {
  std::string kind = "full";
  int n_kv_heads = 0;
  int k_dim = 0;
  int v_dim = 0;
  int window = 0;                    // 0: none
  bool operator==(const CacheNeed &o) const {
    return kind == o.kind && n_kv_heads == o.n_kv_heads && k_dim == o.k_dim && v_dim == o.v_dim && window == o.window;
  }
};

// One fixed-size tensor per sequence, zero when a sequence starts.
struct StateNeed {
  std::string name;
  std::vector<int64_t> shape;
  DType dtype = DType::F32;
};

// The view of the cache one run of a layer gets.
struct LayerCache {
  void *k = nullptr;                 // [pages, kv_heads, page_size, k_dim]
  void *v = nullptr;                 // [pages, kv_heads, page_size, v_dim]; null when v_dim is 0
  int64_t n_pages = 0;
  const int *page_table = nullptr;   // device, int32 [sequences, table_width]
  int table_width = 0;
  int page_size = 64;
  bool writes = true;                // false: reads another run's keys and values
  int group = 0;
  DType dtype = DType::BF16;
  CacheNeed need;
};

// The fixed-size state of one run: name -> [slots, *shape] on the device.
struct StateTensor {
  std::string name;
  void *data = nullptr;
  std::vector<int64_t> shape;        // per sequence
  DType dtype = DType::F32;
  int64_t n_slots = 0;
};
using StateView = std::vector<StateTensor>;

// One step: T tokens of B sequences, each sequence's tokens contiguous.  The pointers are device
// memory.  The host copies are the step's own only when `captured` is false: a step that is
// being captured into a graph is replayed with other sequences, so a part that reads them must
// say that it cannot be captured (Part::capturable).
struct StepContext {
  DType dtype = DType::BF16;
  cudaStream_t stream = nullptr;
  int n_tokens = 0, n_seqs = 0, n_want = 0;
  const int *tokens = nullptr;       // [T]
  const int *tok_seq = nullptr;      // [T] index of the token's sequence in the step
  const int *tok_pos = nullptr;      // [T] absolute position of the token
  const int *seq_start = nullptr;    // [B+1] offsets of each sequence's tokens
  const int *seq_past = nullptr;     // [B] tokens already cached before this step
  const int *seq_slot = nullptr;     // [B] slot of each sequence
  const int *want_rows = nullptr;    // [W] token rows whose logits are asked for
  std::vector<int> q_lens, past_lens, slots;
  int max_q_len = 0, max_kv_len = 0;
  bool decode_only = false;          // every sequence brings exactly one token
  bool captured = false;
  Arena *arena = nullptr;            // device memory that lives until the step's results are read
  // When set, the model gives every layer one of these two in turn, emptied first: what a layer
  // allocates has to outlive the layer after it (the pending residual addition) and no more.  A
  // prompt step of thousands of tokens then holds two layers' activations, not all layers'.
  Arena *layer_arenas[2] = {nullptr, nullptr};
  int *tc_status = nullptr;          // the word in which tensor-core kernels record a wait that ran out
  int *zero_counters = nullptr;      // int32 zeros that kernels may count in if they leave them zero
  int n_zero_counters = 0;
  int sm_count = 148;                // streaming multiprocessors of the device
  // When set, products and norms are queued and launched together (parts/chain.h).  Whoever
  // launches anything else on `stream`, or hands a buffer to code outside, calls flush_chain() first.
  Chain *chain = nullptr;
  // Set by a block around its mixer and its feed-forward: the rows of the 32-bit residual stream that
  // the part's result will be added to.  A part whose last product can add to them as it stores
  // (the library product of a prompt step, with its beta) does so and returns an Act whose data IS
  // this pointer; the block then has nothing left to add.  Parts that ignore it lose nothing.
  float *residual_sink = nullptr;
  int64_t sink_rows = 0, sink_cols = 0;
  // Set by the model for the last layer of a step that wants the logits of fewer rows than it has
  // tokens (a prompt whose last token alone is wanted): after that layer's mixer nothing but these
  // rows of the residual stream is read.  A block may then go on with those rows alone
  // (ResidualStream::picked); one that ignores it computes all rows as before.
  const int *rows_read_after = nullptr;
  int n_rows_read_after = 0;
  bool nothing_read_after = false;   // the same with no row wanted at all (a piece of a long prompt): the mixer's cache writes are all that counts
};

// Device memory for a step's activations: handed out front to back, taken back all at once.
class Arena {
 public:
  explicit Arena(size_t chunk_bytes = (size_t)64 << 20) : chunk_bytes_(chunk_bytes) {}
  void *alloc(size_t bytes, size_t align = 256);
  template <typename T>
  T *alloc_n(size_t n) { return reinterpret_cast<T *>(alloc(n * sizeof(T))); }
  Act act(DType dtype, int64_t rows, int64_t cols, int parts = 1);
  void reset() { chunk_ = 0; used_ = 0; asked_ = 0; }
  // Call between steps, with nothing of the arena in use: several chunks (the arena grew while a
  // step ran) become one that holds the most a step has asked for.  May wait for the device.
  void compact();
  size_t reserved() const;
  // While set, the arena may not grow (a graph is being captured: no allocation may happen).
  void set_frozen(bool f) { frozen_ = f; }

 private:
  size_t chunk_bytes_;
  std::vector<DeviceBuffer> chunks_;
  size_t chunk_ = 0, used_ = 0, asked_ = 0, peak_ = 0;
  bool frozen_ = false;
};

// The 32-bit residual stream and an addition that has not been applied yet.  The addition is
// folded into the next norm's pass over the row.
struct ResidualStream {
  float *resid = nullptr;
  int64_t rows = 0, hidden = 0;
  Act pending;                       // data == nullptr: nothing pending
  bool picked = false;               // the rows are StepContext::rows_read_after, in that order, and no others
};

// What load() fetches tensors through: the files of a model folder, tensors in host memory, or
// random numbers drawn on the device.
class Loader {
 public:
  explicit Loader(DType engine) : engine(engine) {}
  virtual ~Loader() = default;
  // Converts the tensor of `need` to `target` and puts it at `dst` on the device.
  virtual void fetch_into(const TensorNeed &need, DType target, void *dst) const = 0;
  virtual bool has(const std::string &name) const = 0;
  // The same into a new buffer, in the type the need's role calls for.
  Weight fetch(const TensorNeed &need) const;
  const DType engine;
};

class Part {
 public:
  Part(const Json &spec, const BuildEnv &env) : spec_(spec), env_(env) {}
  virtual ~Part() = default;
  virtual std::vector<TensorNeed> tensor_needs() const { return {}; }
  virtual void load(const Loader &) {}
  // Kernel families (libllm_b200/csrc/build.py) this part launches.
  virtual std::vector<std::string> kernel_families() const { return {}; }
  // Whether a step of single tokens through this part may be captured in a CUDA graph.
  virtual bool capturable() const { return true; }
  const Json &spec() const { return spec_; }
  const BuildEnv &env() const { return env_; }

 protected:
  Json spec_;
  BuildEnv env_;
};

class Norm : public Part {
 public:
  using Part::Part;
  // Applies stream.pending (in 32-bit) first.  With `rows` only those rows are normalised and the
  // residual stream is left as it is.
  virtual Act forward(StepContext &ctx, ResidualStream &stream, const int *rows = nullptr, int n_rows = 0) = 0;
};

// What an attention-like mixer tells its position part about the stacked q|k|v rows.
struct QkvLayout {
  int n_heads = 0, n_kv_heads = 0, head_dim = 0;
};

class PositionEncoding : public Part {
 public:
  using Part::Part;
  // Places the step's tokens: writes the (rotated) queries of the stacked rows `qkv` to `q_out`
  // and, when the cache is the run's own, appends the (rotated) keys and the values to it.
  virtual void rotate_and_store(StepContext &ctx, const Act &qkv, const Act &q_out, const QkvLayout &layout,
                                LayerCache &cache) = 0;
  // A table [positions, rotary_dim] (cosines, then sines) of a rotation that pairs channel i with
  // i + rotary_dim/2, if that is what this part does: kernels that fuse the rotation read it.
  // Null: no such table, and only rotate_and_store() is used.
  virtual const float *half_split_table(int *rows, int *rotary_dim) const {
    (void)rows;
    (void)rotary_dim;
    return nullptr;
  }
};

class Mixer : public Part {
 public:
  using Part::Part;
  virtual bool wants_cache() const { return false; }
  virtual CacheNeed cache_need() const { return CacheNeed(); }
  virtual std::vector<StateNeed> state_need() const { return {}; }
  // x [T, hidden] in the engine's type -> [T, hidden] or [parts, T, hidden], 32-bit.
  virtual Act forward(StepContext &ctx, const Act &x, LayerCache *cache, StateView *state) = 0;
};

class FeedForward : public Part {
 public:
  using Part::Part;
  virtual Act forward(StepContext &ctx, const Act &x) = 0;
};

class Block : public Part {
 public:
  using Part::Part;
  virtual Mixer *mixer_part() = 0;
  virtual void forward(StepContext &ctx, ResidualStream &stream, LayerCache *cache, StateView *state) = 0;
};

// ---------------------------------------------------------------- registry
// Categories are "norm", "position", "mixer", "feed_forward" and "block".  A new part registers
// a factory under (category, kind) and is then chosen by any description that carries its kind;
// no file of the library has to change for that.
using PartFactory = std::function<std::unique_ptr<Part>(const Json &spec, const BuildEnv &env)>;
void register_part(const std::string &category, const std::string &kind, PartFactory factory, bool replace = false);
std::unique_ptr<Part> build_part(const std::string &category, const Json &spec, const BuildEnv &env);
template <typename T>
std::unique_ptr<T> build_as(const std::string &category, const Json &spec, const BuildEnv &env) {
  std::unique_ptr<Part> p = build_part(category, spec, env);
  T *t = dynamic_cast<T *>(p.get());
  if (!t) LLM_THROW(Config, "the %s of kind '%s' does not have the interface of its category", category.c_str(),
                    spec.get("kind").is_string() ? spec.get("kind").as_string().c_str() : "?");
  p.release();
  return std::unique_ptr<T>(t);
}
std::vector<std::string> known_parts(const std::string &category);

// f_i = theta^(-2i/d) for i < d/2, rescaled by `scaling` (null, or the "llama3" parameters).
std::vector<double> rotary_frequencies(int64_t rotary_dim, double theta, const Json &scaling);

}  // namespace llm
