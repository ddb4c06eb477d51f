#include "config/llama.h"

#include "config/config.h"

namespace llm {

static RopeScaling parse_rope_scaling(const Json &raw, const std::string &where) {
  RopeScaling s;
  if (raw.is_null()) return s;
  if (!raw.is_object()) LLM_THROW(Config, "%s: 'rope_scaling' must be an object or null", where.c_str());
  const Json &kind = raw.has("rope_type") ? raw.get("rope_type") : raw.get("type");
  if (kind.is_null() || (kind.is_string() && kind.as_string() == "default")) return s;
  if (!kind.is_string() || kind.as_string() != "llama3")
    LLM_THROW(Config, "%s: rope_scaling type %s is not supported (only 'llama3')", where.c_str(), kind.dump().c_str());
  ConfigReader r(raw, where + ": rope_scaling");
  s.present = true;
  s.rope_type = "llama3";
  s.factor = r.number("factor");
  s.low_freq_factor = r.number("low_freq_factor");
  s.high_freq_factor = r.number("high_freq_factor");
  s.original_max_position_embeddings = r.integer("original_max_position_embeddings");
  if (s.high_freq_factor <= s.low_freq_factor)
    LLM_THROW(Config, "%s: rope_scaling needs high_freq_factor > low_freq_factor", where.c_str());
  return s;
}

LlamaConfig parse_llama_config(const Json &data) {
  const std::string where = "config.json";
  ConfigReader r(data, where);
  LlamaConfig c;
  c.hidden_size = r.integer("hidden_size");
  c.num_attention_heads = r.integer("num_attention_heads");
  c.num_key_value_heads = r.integer_or("num_key_value_heads", c.num_attention_heads);
  if (r.present("head_dim")) {
    c.head_dim = r.integer("head_dim");
  } else {
    if (c.hidden_size % c.num_attention_heads != 0)
      LLM_THROW(Config, "%s: invalid hidden_size and num_attention_heads (%lld is not a multiple of %lld) and no head_dim given",
                where.c_str(), (long long)c.hidden_size, (long long)c.num_attention_heads);
    c.head_dim = c.hidden_size / c.num_attention_heads;
  }
  if (c.num_attention_heads % c.num_key_value_heads != 0)
    LLM_THROW(Config, "%s: num_attention_heads (%lld) must be a multiple of num_key_value_heads (%lld)", where.c_str(),
              (long long)c.num_attention_heads, (long long)c.num_key_value_heads);
  if (c.head_dim % 2 != 0)
    LLM_THROW(Config, "%s: head_dim (%lld) must be even for rotary pairs", where.c_str(), (long long)c.head_dim);
  const std::string act = r.string_or("hidden_act", "silu");
  if (act != "silu") LLM_THROW(Config, "%s: hidden_act '%s' is not supported (only 'silu')", where.c_str(), act.c_str());
  if (r.integer_or("pretraining_tp", 1) != 1) LLM_THROW(Config, "%s: pretraining_tp must be 1", where.c_str());
  if (r.boolean_or("mlp_bias", false)) LLM_THROW(Config, "%s: mlp_bias is not supported", where.c_str());
  c.vocab_size = r.integer("vocab_size");
  const Json &eos = r.raw("eos_token_id");
  if (eos.is_int()) {
    c.eos_token_ids.push_back((int)eos.as_int());
  } else if (eos.is_array()) {
    for (const auto &e : eos.items()) {
      if (!e.is_int()) LLM_THROW(Config, "%s: 'eos_token_id' must be an integer or a list of integers", where.c_str());
      c.eos_token_ids.push_back((int)e.as_int());
    }
  } else if (!eos.is_null()) {
    LLM_THROW(Config, "%s: 'eos_token_id' must be an integer or a list of integers", where.c_str());
  }
  for (int e : c.eos_token_ids)
    if (e < 0 || e >= c.vocab_size)
      LLM_THROW(Config, "%s: eos_token_id %d lies outside the vocabulary (%lld)", where.c_str(), e, (long long)c.vocab_size);
  c.model_type = r.string("model_type");
  c.num_hidden_layers = r.integer("num_hidden_layers");
  c.intermediate_size = r.integer("intermediate_size");
  c.max_position_embeddings = r.integer("max_position_embeddings");
  c.rms_norm_eps = r.number("rms_norm_eps");
  c.rope_theta = r.number_or("rope_theta", 10000.0);
  c.rope_scaling = parse_rope_scaling(r.raw("rope_scaling"), where);
  c.tie_word_embeddings = r.boolean_or("tie_word_embeddings", false);
  c.attention_bias = r.boolean_or("attention_bias", false);
  c.bos_token_id = r.integer_or("bos_token_id", -1, 0);
  return c;
}

static Json rope_scaling_json(const RopeScaling &s) {
  if (!s.present) return Json();
  Json o = Json::object();
  o.set("rope_type", s.rope_type);
  o.set("factor", s.factor);
  o.set("low_freq_factor", s.low_freq_factor);
  o.set("high_freq_factor", s.high_freq_factor);
  o.set("original_max_position_embeddings", s.original_max_position_embeddings);
  return o;
}

Json LlamaConfig::to_json() const {
  Json j = Json::object();
  j.set("model_type", model_type);
  j.set("hidden_size", hidden_size);
  j.set("num_hidden_layers", num_hidden_layers);
  j.set("num_attention_heads", num_attention_heads);
  j.set("num_key_value_heads", num_key_value_heads);
  j.set("head_dim", head_dim);
  j.set("intermediate_size", intermediate_size);
  j.set("vocab_size", vocab_size);
  j.set("max_position_embeddings", max_position_embeddings);
  j.set("rms_norm_eps", rms_norm_eps);
  j.set("rope_theta", rope_theta);
  j.set("rope_scaling", rope_scaling_json(rope_scaling));
  j.set("tie_word_embeddings", tie_word_embeddings);
  j.set("attention_bias", attention_bias);
  j.set("eos_token_id", eos_token_ids.empty() ? Json()
                        : eos_token_ids.size() == 1 ? Json(eos_token_ids[0]) : Json::list(eos_token_ids));
  j.set("bos_token_id", bos_token_id < 0 ? Json() : Json(bos_token_id));
  j.set("hidden_act", "silu");
  return j;
}

// Layer structure and sizes follow the reference's build functions (src/libllm/llama.cc:111-141,
// 231-249, 273-292); tensor names are the checkpoint's own, the ones the reference's exporter
// reads them from (tools/llama_exporter.py:35-78).
ModelSpec describe_llama(const LlamaConfig &c) {
  auto norm = [&](const std::string &weight) {
    Json n = Json::object();
    n.set("kind", "rmsnorm");
    n.set("size", c.hidden_size);
    n.set("eps", c.rms_norm_eps);
    n.set("weight", weight);
    return n;
  };
  Json rope = Json::object();
  rope.set("kind", "rope");
  rope.set("head_dim", c.head_dim);
  rope.set("rotary_dim", c.head_dim);
  rope.set("theta", c.rope_theta);
  rope.set("scaling", rope_scaling_json(c.rope_scaling));

  ModelSpec s;
  s.name = "llama";
  s.vocab_size = c.vocab_size;
  s.hidden = c.hidden_size;
  s.embedding = "model.embed_tokens.weight";
  for (int64_t i = 0; i < c.num_hidden_layers; ++i) {
    const std::string p = "model.layers." + std::to_string(i) + ".";
    Json attn = Json::object();
    attn.set("kind", "attention");
    attn.set("hidden", c.hidden_size);
    attn.set("n_heads", c.num_attention_heads);
    attn.set("n_kv_heads", c.num_key_value_heads);
    attn.set("head_dim", c.head_dim);
    attn.set("position", rope);
    attn.set("window", Json());
    attn.set("scale", Json());
    attn.set("bias", c.attention_bias);
    attn.set("q", p + "self_attn.q_proj.weight");
    attn.set("k", p + "self_attn.k_proj.weight");
    attn.set("v", p + "self_attn.v_proj.weight");
    attn.set("o", p + "self_attn.o_proj.weight");
    Json ff = Json::object();
    ff.set("kind", "swiglu");
    ff.set("hidden", c.hidden_size);
    ff.set("intermediate", c.intermediate_size);
    ff.set("gate", p + "mlp.gate_proj.weight");
    ff.set("up", p + "mlp.up_proj.weight");
    ff.set("down", p + "mlp.down_proj.weight");
    Json block = Json::object();
    block.set("kind", "prenorm");
    block.set("mixer_norm", norm(p + "input_layernorm.weight"));
    block.set("mixer", attn);
    block.set("ff_norm", norm(p + "post_attention_layernorm.weight"));
    block.set("ff", ff);
    s.layers.push_back(block);
    s.schedule.push_back({(int)i, -1});
  }
  s.final_norm = norm("model.norm.weight");
  s.head = c.tie_word_embeddings ? "" : "lm_head.weight";
  s.max_positions = c.max_position_embeddings;
  s.stop_tokens = c.eos_token_ids;
  // A tied checkpoint may still carry a copy of the output matrix, and older exports carry each
  // layer's rotary frequencies: neither is used.
  if (c.tie_word_embeddings) s.ignore_tensors.push_back("lm_head.weight");
  s.ignore_tensors.push_back("model.layers.*.self_attn.rotary_emb.inv_freq");
  return s;
}

void register_builtin_architectures() {
  Architecture a;
  a.name = "llama";
  a.parse = [](const Json &j) { return parse_llama_config(j).to_json(); };
  a.describe = [](const Json &normal) { return describe_llama(parse_llama_config(normal)); };
  // straight into the table: register_architecture() would wait for this very call to finish
  extern void register_architecture_unlocked(Architecture);
  register_architecture_unlocked(std::move(a));
}

}  // namespace llm
