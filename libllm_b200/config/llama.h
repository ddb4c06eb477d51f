// LlamaConfig: the typed configuration of the Llama dense decoder.
//
// Fields are those the reference's loader reads (src/libllm/llama.cc:53-75) under the names its
// exporter takes them from in config.json (tools/llama_exporter.py:90-100), plus what the exporter
// resolves offline and this library resolves itself: the rotary base and its "llama3" rescaling
// (the reference stores a finished table, tools/llama_exporter.py:54-62), the head size, tied
// embeddings and the stop tokens.
#pragma once
#include <string>
#include <vector>

#include "parts/spec.h"
#include "util/json.h"

namespace llm {

struct RopeScaling {
  bool present = false;          // false: plain frequencies
  std::string rope_type;         // "llama3"
  double factor = 1, low_freq_factor = 1, high_freq_factor = 4;
  int64_t original_max_position_embeddings = 0;
};

struct LlamaConfig {
  std::string model_type;
  int64_t hidden_size = 0, num_hidden_layers = 0, num_attention_heads = 0, num_key_value_heads = 0;
  int64_t head_dim = 0, intermediate_size = 0, vocab_size = 0, max_position_embeddings = 0;
  double rms_norm_eps = 0, rope_theta = 10000.0;
  RopeScaling rope_scaling;
  bool tie_word_embeddings = false, attention_bias = false;
  std::vector<int> eos_token_ids;
  int64_t bos_token_id = -1;     // -1: none

  Json to_json() const;          // the normal form: config.json's own keys, every one present
};

// Checks follow the reference where it has them: hidden_size must divide by the number of heads
// when no head size is given ("invalid hidden_size and num_heads", src/libllm/llama.cc:117-118);
// the activation must be silu and pretraining_tp 1 (tools/llama_exporter.py:87-88).
LlamaConfig parse_llama_config(const Json &config_json);
ModelSpec describe_llama(const LlamaConfig &c);

}  // namespace llm
