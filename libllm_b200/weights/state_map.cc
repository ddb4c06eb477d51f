#include "weights/state_map.h"

#include <sys/stat.h>

#include <algorithm>
#include <cstring>
#include <fstream>
#include <set>
#include <sstream>
#include <thread>

namespace llm {

static bool is_file(const std::string &p) {
  struct stat st;
  return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

bool name_matches(const std::string &pattern, const std::string &name) {
  // iterative glob with '*' only
  size_t p = 0, n = 0, star = std::string::npos, mark = 0;
  while (n < name.size()) {
    if (p < pattern.size() && pattern[p] != '*' && pattern[p] == name[n]) {
      ++p;
      ++n;
    } else if (p < pattern.size() && pattern[p] == '*') {
      star = p++;
      mark = n;
    } else if (star != std::string::npos) {
      p = star + 1;
      n = ++mark;
    } else {
      return false;
    }
  }
  while (p < pattern.size() && pattern[p] == '*') ++p;
  return p == pattern.size();
}

std::string shape_text(const std::vector<int64_t> &shape) {
  std::string s = "(";
  for (size_t i = 0; i < shape.size(); ++i) s += (i ? ", " : "") + std::to_string(shape[i]);
  if (shape.size() == 1) s += ",";
  return s + ")";
}

std::unique_ptr<StateMap> StateMap::from_folder(const std::string &folder) {
  const std::string index = folder + "/model.safetensors.index.json", single = folder + "/model.safetensors";
  std::unique_ptr<StateMap> sm(new StateMap(folder));
  std::vector<std::string> files;
  if (is_file(index)) {
    std::ifstream f(index, std::ios::binary);
    std::stringstream ss;
    ss << f.rdbuf();
    Json j;
    try {
      j = Json::parse(ss.str(), index);
    } catch (const Error &e) {
      throw Error(ErrorKind::Weights, e.what());
    }
    std::set<std::string> shard_names;
    const Json &wm = j.get("weight_map");
    if (wm.is_object())
      for (const auto &m : wm.members())
        if (m.second.is_string()) shard_names.insert(m.second.as_string());
    std::string missing;
    for (const auto &n : shard_names)
      if (!is_file(folder + "/" + n)) missing += (missing.empty() ? "" : ", ") + n;
    if (!missing.empty())
      LLM_THROW(Weights, "%s: shard files named by model.safetensors.index.json are missing: %s", folder.c_str(), missing.c_str());
    for (const auto &n : shard_names) files.push_back(folder + "/" + n);
  } else if (is_file(single)) {
    files.push_back(single);
  } else {
    LLM_THROW(Weights, "%s: neither model.safetensors nor model.safetensors.index.json found", folder.c_str());
  }
  for (const auto &path : files) {
    sm->files_.emplace_back(new SafetensorsFile(path));
    const SafetensorsFile &f = *sm->files_.back();
    for (const auto &n : f.names()) {
      if (sm->tensors_.count(n))
        LLM_THROW(Weights, "%s: tensor '%s' is stored twice (%s and %s)", folder.c_str(), n.c_str(), sm->origin_[n].c_str(), path.c_str());
      sm->tensors_[n] = f.tensor(n);
      sm->origin_[n] = path;
      sm->names_.push_back(n);
    }
  }
  return sm;
}

void StateMap::add(const std::string &name, const StoredTensor &t) {
  if (tensors_.count(name)) LLM_THROW(Weights, "%s: tensor '%s' is given twice", where_.c_str(), name.c_str());
  if ((int64_t)t.nbytes != t.numel() * (int64_t)stored_type_size(t.dtype))
    LLM_THROW(Weights, "%s: tensor '%s' has %zu bytes, its shape needs %lld", where_.c_str(), name.c_str(), t.nbytes,
              (long long)(t.numel() * (int64_t)stored_type_size(t.dtype)));
  tensors_[name] = t;
  names_.push_back(name);
}

const StoredTensor &StateMap::stored(const std::string &name) const {
  auto it = tensors_.find(name);
  if (it == tensors_.end()) {
    WeightsReport r;
    r.missing.push_back(name);
    throw WeightsError("tensor \"" + name + "\" not found in model.", r);
  }
  return it->second;
}

WeightsReport StateMap::check(const std::vector<TensorNeed> &needs, const std::vector<std::string> &ignore, bool strict) const {
  WeightsReport r;
  std::set<std::string> wanted;
  for (const auto &n : needs) {
    wanted.insert(n.name);
    if (!has(n.name)) {
      if (!n.optional) r.missing.push_back(n.name);
      continue;
    }
    const auto &found = tensors_.at(n.name).shape;
    if (found != n.shape) r.wrong_shape.push_back({n.name, n.shape, found});
  }
  for (const auto &n : names_) {
    if (wanted.count(n)) continue;
    bool ign = false;
    for (const auto &p : ignore) ign = ign || name_matches(p, n);
    (ign ? r.ignored : r.unexpected).push_back(n);
  }
  std::sort(r.unexpected.begin(), r.unexpected.end());
  const bool bad = !r.missing.empty() || !r.wrong_shape.empty() || (strict && !r.unexpected.empty());
  if (!bad) return r;
  std::string msg = format("%s: the weights do not fit the model (%zu missing, %zu unexpected, %zu with a wrong shape)",
                           where_.c_str(), r.missing.size(), r.unexpected.size(), r.wrong_shape.size());
  for (const auto &m : r.missing) msg += "\n  missing: tensor \"" + m + "\" not found in model.";
  for (const auto &u : r.unexpected)
    msg += "\n  unexpected: tensor \"" + u + "\" is in the files but no part of the model asks for it.";
  for (const auto &w : r.wrong_shape)
    msg += "\n  wrong shape: " + w.name + ": invalid shape: " + shape_text(w.expected) + " expected, but " + shape_text(w.found) + " found.";
  throw WeightsError(msg, r);
}

DType StateMap::device_dtype(const TensorNeed &need, DType engine) {
  if (need.role == TensorRole::Table) return DType::I32;
  if (need.role == TensorRole::Vector) return DType::F32;
  return engine;
}

namespace {
template <typename F>
void parallel_for(int64_t n, F fn) {
  const int64_t grain = 1 << 20;
  int workers = (int)std::min<int64_t>(std::max(1u, std::thread::hardware_concurrency()), (n + grain - 1) / grain);
  if (workers <= 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> pool;
  const int64_t per = (n + workers - 1) / workers;
  for (int w = 0; w < workers; ++w) {
    const int64_t a = w * per, b = std::min(n, a + per);
    if (a < b) pool.emplace_back([=] { fn(a, b); });
  }
  for (auto &t : pool) t.join();
}

float read_float(const uint8_t *p, StoredType t, int64_t i) {
  switch (t) {
    case StoredType::F32: { float v; memcpy(&v, p + 4 * i, 4); return v; }
    case StoredType::F64: { double v; memcpy(&v, p + 8 * i, 8); return (float)v; }
    case StoredType::F16: { uint16_t v; memcpy(&v, p + 2 * i, 2); return half_to_float(v); }
    case StoredType::BF16: { uint16_t v; memcpy(&v, p + 2 * i, 2); return bf16_to_float(v); }
    default: return 0.f;
  }
}
int64_t read_int(const uint8_t *p, StoredType t, int64_t i) {
  switch (t) {
    case StoredType::I64: { int64_t v; memcpy(&v, p + 8 * i, 8); return v; }
    case StoredType::I32: { int32_t v; memcpy(&v, p + 4 * i, 4); return v; }
    case StoredType::I16: { int16_t v; memcpy(&v, p + 2 * i, 2); return v; }
    case StoredType::I8: return (int8_t)p[i];
    case StoredType::U8:
    case StoredType::BOOL: return p[i];
    default: return 0;
  }
}
}  // namespace

void StateMap::fetch_into(const TensorNeed &need, DType target, void *dst) const {
  const StoredTensor &t = stored(need.name);
  if (t.shape != need.shape) {
    WeightsReport r;
    r.wrong_shape.push_back({need.name, need.shape, t.shape});
    throw WeightsError(need.name + ": invalid shape: " + shape_text(need.shape) + " expected, but " + shape_text(t.shape) + " found.", r);
  }
  const int64_t n = t.numel();
  if (n == 0) return;
  const bool is_float = stored_type_is_float(t.dtype);
  if (need.role == TensorRole::Table) {
    if (is_float) LLM_THROW(Weights, "%s: an integer table is stored as %s", need.name.c_str(), stored_type_name(t.dtype));
  } else if (!is_float) {
    LLM_THROW(Weights, "%s: stored as %s, a floating-point tensor is needed", need.name.c_str(), stored_type_name(t.dtype));
  }
  // the stored form is the device's form: one copy
  if ((target == DType::BF16 && t.dtype == StoredType::BF16) || (target == DType::F32 && t.dtype == StoredType::F32) ||
      (target == DType::I32 && t.dtype == StoredType::I32)) {
    LLM_CUDA(cudaMemcpy(dst, t.data, t.nbytes, cudaMemcpyHostToDevice));
    return;
  }
  std::vector<uint8_t> staging((size_t)n * dtype_size(target));
  const uint8_t *src = t.data;
  const StoredType st = t.dtype;
  if (target == DType::I32) {
    int32_t *out = (int32_t *)staging.data();
    parallel_for(n, [=](int64_t a, int64_t b) { for (int64_t i = a; i < b; ++i) out[i] = (int32_t)read_int(src, st, i); });
  } else if (target == DType::F32) {
    float *out = (float *)staging.data();
    parallel_for(n, [=](int64_t a, int64_t b) { for (int64_t i = a; i < b; ++i) out[i] = read_float(src, st, i); });
  } else {
    uint16_t *out = (uint16_t *)staging.data();
    parallel_for(n, [=](int64_t a, int64_t b) { for (int64_t i = a; i < b; ++i) out[i] = float_to_bf16(read_float(src, st, i)); });
  }
  LLM_CUDA(cudaMemcpy(dst, staging.data(), staging.size(), cudaMemcpyHostToDevice));
}

}  // namespace llm
