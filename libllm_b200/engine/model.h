// The generic model: a token table, the layers of a ModelSpec in the order of its schedule, a last
// norm and the output matrix.  It knows parts and their interfaces, not architectures; the
// architecture's name is used once, to look up the function that describes it
// (libllm_b200/config/config.h).
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "cache/kv_cache.h"
#include "parts/part.h"
#include "parts/spec.h"

namespace llm {

DType parse_dtype(const std::string &name);     // "bfloat16" or "float32"

// Random weights: matrices N(0, std), norm weights 1 + U(-0.1, 0.1), biases N(0, std).
struct RandomLaw {
  int law;        // 0 normal(a, b), 1 uniform [a, b)
  float a, b;
};
RandomLaw random_law(const TensorNeed &need, float std = 0.02f);

class Model {
 public:
  // Builds the parts; touches no device.  `config` is the architecture's configuration in normal form.
  Model(ModelSpec spec, Json config, DType dtype, int64_t max_positions = 0, int page_size = 64);

  const ModelSpec &spec() const { return spec_; }
  const Json &config() const { return config_; }
  DType dtype() const { return dtype_; }
  int64_t max_positions() const { return max_positions_; }
  int page_size() const { return env_.page_size; }

  std::vector<TensorNeed> tensor_needs() const;
  std::vector<std::string> kernel_families() const;
  // Whether steps of single tokens may be captured as CUDA graphs (every part says so).
  bool capturable() const;

  // Checks the tensors against the needs (one error for everything that does not fit) and brings
  // them to the device.  Returns the report (ignored and, when not strict, unexpected tensors).
  WeightsReport load(const StateMap &state, bool strict = true);
  // The random-weights mode without files: tensors are drawn on the device from (seed, name).
  void load_random(uint64_t seed);
  bool loaded() const { return loaded_; }

  // What the cache must hold, per schedule entry.
  void cache_needs(std::vector<CacheNeed> *needs, std::vector<char> *has) const;
  std::vector<std::vector<StateNeed>> state_needs() const;

  // Runs the tokens of `ctx` through every scheduled layer and returns 32-bit logits for
  // ctx.want_rows, [W, vocab] (the reference computes logits of the last position only,
  // src/libllm/llama.cc:353-354; its tests of all positions, src/libllm/llama_test.cc:92-97).
  // A token either comes with the step or is row fed_rows[t] of fed_tokens on the device.
  Act forward(StepContext &ctx, KVCache &cache, const std::vector<const int *> &tables, int table_width,
              const int *fed_tokens, const int *fed_rows);

 private:
  void load_with(const Loader &loader);
  ModelSpec spec_;
  Json config_;
  DType dtype_;
  int64_t max_positions_;
  BuildEnv env_;
  std::map<std::string, std::shared_ptr<Weight>> shared_;
  std::vector<std::unique_ptr<Block>> layers_;
  std::unique_ptr<Norm> final_norm_;
  Weight embedding_, head_own_;
  const Weight *head_ = nullptr;
  bool loaded_ = false;
};

// A model from a folder's config.json alone (no weights yet).
std::unique_ptr<Model> model_from_config(const Json &config_json, DType dtype, int64_t max_positions = 0);

// The random-weights mode that writes a model folder: config.json as given and model.safetensors
// with random tensors under the names and shapes the architecture asks for, drawn on the host.
void create_random_model(const std::string &folder, const Json &config_json, uint64_t seed, const std::string &dtype = "bfloat16");
// The same tensors in host memory (for tests): name -> 32-bit values.
void random_tensor_host(const TensorNeed &need, uint64_t seed, std::vector<float> *out);

}  // namespace llm
