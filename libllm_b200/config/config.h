// Typed reads of a configuration and the one registry from an architecture's name to its model.
//
// The reference keeps one typed struct per architecture, filled key by key from the model's own
// configuration section, and picks the model class by the `type` string
// (src/libllm/llama.cc:53-75, src/libllm/model_for_generation.cc:33-52).  Here the keys are those
// of the checkpoint's config.json, and the `if (type == ...)` chain is a table that an
// architecture adds itself to: a name, a function that checks config.json and returns it in
// normal form (defaults filled in), and a function that describes the model as data (ModelSpec).
// Nothing else in the library knows an architecture's name.
#pragma once
#include <functional>
#include <string>
#include <vector>

#include "parts/spec.h"
#include "util/json.h"

namespace llm {

// Reads keys of one JSON object with type checks; errors name the file and the key.
class ConfigReader {
 public:
  ConfigReader(const Json &data, std::string where, ErrorKind kind = ErrorKind::Config)
      : data_(data), where_(std::move(where)), kind_(kind) {}

  bool present(const std::string &key) const { return data_.has(key) && !data_.get(key).is_null(); }
  int64_t integer(const std::string &key, int64_t minimum = 1) const;                     // required
  int64_t integer_or(const std::string &key, int64_t fallback, int64_t minimum = 1) const;
  double number(const std::string &key, bool positive = true) const;
  double number_or(const std::string &key, double fallback, bool positive = true) const;
  bool boolean_or(const std::string &key, bool fallback) const;
  std::string string(const std::string &key) const;
  std::string string_or(const std::string &key, const std::string &fallback) const;
  const Json &raw(const std::string &key) const { return data_.get(key); }
  const Json &object(const std::string &key) const;                                       // required
  const std::string &where() const { return where_; }
  [[noreturn]] void fail(const std::string &msg) const;

 private:
  const Json &need(const std::string &key) const;
  const Json &data_;
  std::string where_;
  ErrorKind kind_;
};

struct Architecture {
  std::string name;
  // config.json as read -> the architecture's configuration in normal form (every key present,
  // defaults filled in, values checked).  Throws Error(Config).
  std::function<Json(const Json &)> parse;
  // the normal form -> the model as data
  std::function<ModelSpec(const Json &)> describe;
};

void register_architecture(Architecture arch, bool replace = false);
std::vector<std::string> known_architectures();
// An unknown name is an error that lists the known ones (the reference: "unexpected model type",
// src/libllm/model_for_generation.cc:47-49).
const Architecture &architecture_for(const std::string &model_type);

Json read_config_json(const std::string &folder);
// config.json of `folder` in its architecture's normal form.
Json load_config(const std::string &folder);
// The same for a config.json already in memory.
Json parse_config(const Json &config_json);

}  // namespace llm
