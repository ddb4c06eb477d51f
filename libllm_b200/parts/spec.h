// The description of a model as data: which parts each layer is made of, with every size and
// constant as a field, the order in which layers run, and the names of their tensors.
//
// An architecture (libllm_b200/config/llama.cc) turns its configuration into one ModelSpec; the
// generic model (libllm_b200/engine/model.cc) builds the part that each description names through
// the part registry (libllm_b200/parts/part.h).  A part's description is a JSON object whose
// "kind" selects the class; the other keys are that class's own and are read, with checks, by
// its constructor.  A description knows nothing about the model it is used in.  The reference
// builds its one architecture in code (src/libllm/llama.cc:111-141, 231-249, 273-292); the keys
// here are the arguments of those build functions.
//
//   norm "rmsnorm":        size, eps, weight (tensor name)
//   position "rope":       head_dim, rotary_dim, theta, scaling (null or the llama3 parameters)
//   mixer "attention":     hidden, n_heads, n_kv_heads, head_dim, v_head_dim (default head_dim),
//                          position (a position description or null), window (null: all keys),
//                          scale (null: 1/sqrt(head_dim)), bias, q, k, v, o (tensor names)
//   feed_forward "swiglu": hidden, intermediate, gate, up, down (tensor names)
//   block "prenorm":       mixer_norm, mixer, ff_norm, ff (descriptions)
#pragma once
#include <string>
#include <vector>

#include "util/json.h"

namespace llm {

// One run of a layer.  `layer` indexes ModelSpec::layers; the same layer may be named by several
// entries (its weights are then used twice, each run with a cache of its own).  `cache_from`
// names an earlier entry whose cache this run reads instead of keeping one: it appends nothing.
struct ScheduleEntry {
  int layer = 0;
  int cache_from = -1;
};

struct ModelSpec {
  std::string name;
  int64_t vocab_size = 0;
  int64_t hidden = 0;
  std::string embedding;                  // tensor name of the token table
  std::vector<Json> layers;               // block descriptions
  std::vector<ScheduleEntry> schedule;
  Json final_norm;
  std::string head;                       // output matrix; empty: the token table
  int64_t max_positions = 0;
  std::vector<int> stop_tokens;
  double embedding_scale = 1.0;           // token rows are multiplied by this before the first layer
  double logit_scale = 1.0;               // logits are multiplied by this ...
  double logit_softcap = 0.0;             // ... and, if positive, bounded: cap * tanh(logit / cap)
  // Tensors that may lie in the files without any part asking for them ('*' matches any run of
  // characters).  Other unexpected tensors are reported as a warning, not an error.
  std::vector<std::string> ignore_tensors;

  Json to_json() const;
  static ModelSpec from_json(const Json &j);
};

}  // namespace llm
