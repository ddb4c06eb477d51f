#include "config/config.h"

#include <algorithm>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

namespace llm {

void ConfigReader::fail(const std::string &msg) const { throw Error(kind_, where_ + ": " + msg); }

const Json &ConfigReader::need(const std::string &key) const {
  if (!present(key)) fail("required key '" + key + "' is missing");
  return data_.get(key);
}

static std::string shown(const Json &v) { return v.dump(); }

int64_t ConfigReader::integer(const std::string &key, int64_t minimum) const {
  const Json &v = need(key);
  if (!v.is_int()) fail("'" + key + "' must be an integer, found " + shown(v));
  if (v.as_int() < minimum) fail(format("'%s' must be at least %lld, found %lld", key.c_str(), (long long)minimum, (long long)v.as_int()));
  return v.as_int();
}

int64_t ConfigReader::integer_or(const std::string &key, int64_t fallback, int64_t minimum) const {
  return present(key) ? integer(key, minimum) : fallback;
}

double ConfigReader::number(const std::string &key, bool positive) const {
  const Json &v = need(key);
  if (!v.is_number()) fail("'" + key + "' must be a number, found " + shown(v));
  if (positive && !(v.as_number() > 0)) fail("'" + key + "' must be positive, found " + shown(v));
  return v.as_number();
}

double ConfigReader::number_or(const std::string &key, double fallback, bool positive) const {
  return present(key) ? number(key, positive) : fallback;
}

bool ConfigReader::boolean_or(const std::string &key, bool fallback) const {
  if (!present(key)) return fallback;
  const Json &v = data_.get(key);
  if (!v.is_bool()) fail("'" + key + "' must be true or false, found " + shown(v));
  return v.as_bool();
}

std::string ConfigReader::string(const std::string &key) const {
  const Json &v = need(key);
  if (!v.is_string()) fail("'" + key + "' must be a string, found " + shown(v));
  return v.as_string();
}

std::string ConfigReader::string_or(const std::string &key, const std::string &fallback) const {
  return present(key) ? string(key) : fallback;
}

const Json &ConfigReader::object(const std::string &key) const {
  const Json &v = need(key);
  if (!v.is_object()) fail("'" + key + "' must be an object, found " + shown(v));
  return v;
}

// ---------------------------------------------------------------- registry
namespace {
std::map<std::string, Architecture> &table() {
  static std::map<std::string, Architecture> t;
  return t;
}
std::mutex &table_lock() {
  static std::mutex m;
  return m;
}
}  // namespace

void register_builtin_architectures();   // config/llama.cc
void register_architecture_unlocked(Architecture arch) { table()[arch.name] = std::move(arch); }

static void ensure_builtin() {
  static std::once_flag once;
  std::call_once(once, register_builtin_architectures);
}

void register_architecture(Architecture arch, bool replace) {
  ensure_builtin();
  std::lock_guard<std::mutex> lock(table_lock());
  if (table().count(arch.name) && !replace)
    LLM_THROW(Config, "architecture '%s' is registered already", arch.name.c_str());
  table()[arch.name] = std::move(arch);
}

std::vector<std::string> known_architectures() {
  ensure_builtin();
  std::lock_guard<std::mutex> lock(table_lock());
  std::vector<std::string> out;
  for (const auto &kv : table()) out.push_back(kv.first);
  return out;
}

const Architecture &architecture_for(const std::string &model_type) {
  ensure_builtin();
  std::lock_guard<std::mutex> lock(table_lock());
  auto it = table().find(model_type);
  if (it == table().end()) {
    std::string known;
    for (const auto &kv : table()) known += (known.empty() ? "" : ", ") + kv.first;
    LLM_THROW(Config, "unexpected model type '%s'; registered: %s", model_type.c_str(), known.c_str());
  }
  return it->second;
}

Json read_config_json(const std::string &folder) {
  const std::string path = folder + "/config.json";
  std::ifstream f(path, std::ios::binary);
  if (!f) LLM_THROW(Config, "%s: no such file", path.c_str());
  std::stringstream ss;
  ss << f.rdbuf();
  Json data;
  try {
    data = Json::parse(ss.str(), path);
  } catch (const Error &e) {
    throw Error(ErrorKind::Config, e.what());
  }
  if (!data.is_object()) LLM_THROW(Config, "%s: the top level must be an object", path.c_str());
  return data;
}

Json parse_config(const Json &config_json) {
  if (!config_json.is_object() || !config_json.get("model_type").is_string())
    LLM_THROW(Config, "config.json: required key 'model_type' is missing");
  return architecture_for(config_json.get("model_type").as_string()).parse(config_json);
}

Json load_config(const std::string &folder) {
  const Json data = read_config_json(folder);
  if (!data.get("model_type").is_string())
    LLM_THROW(Config, "%s/config.json: required key 'model_type' is missing", folder.c_str());
  return architecture_for(data.get("model_type").as_string()).parse(data);
}

}  // namespace llm
