#include "parts/part.h"

#include <algorithm>
#include <mutex>

namespace llm {

// ---------------------------------------------------------------- arena
void *Arena::alloc(size_t bytes, size_t align) {
  if (bytes == 0) bytes = align;
  asked_ += (bytes + align - 1) / align * align + align;
  peak_ = std::max(peak_, asked_);
  for (;;) {
    if (chunk_ < chunks_.size()) {
      const size_t start = (used_ + align - 1) / align * align;
      if (start + bytes <= chunks_[chunk_].bytes()) {
        used_ = start + bytes;
        return (char *)chunks_[chunk_].get() + start;
      }
      ++chunk_;
      used_ = 0;
      continue;
    }
    if (frozen_)
      LLM_THROW(Extension, "a captured step asked for more device memory (%zu bytes) than its first run", bytes);
    // at least as much again as is held: a step that needs gigabytes asks the driver a few times, not hundreds
    chunks_.emplace_back(std::max({chunk_bytes_, bytes + align, std::min(reserved() / 2, (size_t)1 << 30)}));
  }
}

void Arena::compact() {
  if (frozen_ || chunks_.size() <= 1) return;
  // kernels of earlier steps may still be reading the chunks
  cudaDeviceSynchronize();
  chunks_.clear();
  chunks_.emplace_back(std::max(chunk_bytes_, peak_ + peak_ / 4));
  reset();
}

Act Arena::act(DType dtype, int64_t rows, int64_t cols, int parts) {
  Act a;
  a.dtype = dtype;
  a.rows = rows;
  a.cols = cols;
  a.ld = cols;
  a.parts = parts;
  a.part_stride = rows * cols;
  a.data = alloc((size_t)parts * (size_t)rows * (size_t)cols * dtype_size(dtype));
  return a;
}

size_t Arena::reserved() const {
  size_t n = 0;
  for (const auto &c : chunks_) n += c.bytes();
  return n;
}

// ---------------------------------------------------------------- registry
namespace {
const char *CATEGORIES[] = {"norm", "position", "mixer", "feed_forward", "block"};
std::map<std::pair<std::string, std::string>, PartFactory> &table() {
  static std::map<std::pair<std::string, std::string>, PartFactory> t;
  return t;
}
std::mutex &table_lock() {
  static std::mutex m;
  return m;
}
void ensure_builtin();
}  // namespace

void register_builtin_parts();   // parts/builtin.cc

namespace {
void ensure_builtin() {
  static std::once_flag once;
  std::call_once(once, register_builtin_parts);
}
}  // namespace

void register_part_raw(const std::string &category, const std::string &kind, PartFactory factory) {
  std::lock_guard<std::mutex> g(table_lock());
  table()[std::make_pair(category, kind)] = std::move(factory);
}

Weight Loader::fetch(const TensorNeed &need) const {
  Weight w;
  w.dtype = StateMap::device_dtype(need, engine);
  int64_t n = 1;
  for (auto s : need.shape) n *= s;
  w.rows = need.shape.size() >= 2 ? need.shape[0] : 1;
  w.cols = w.rows > 0 ? n / w.rows : 0;
  w.buf.allocate((size_t)n * dtype_size(w.dtype));
  fetch_into(need, w.dtype, w.buf.get());
  return w;
}

void register_part(const std::string &category, const std::string &kind, PartFactory factory, bool replace) {
  ensure_builtin();
  bool known = false;
  for (const char *c : CATEGORIES) known = known || category == c;
  if (!known)
    LLM_THROW(Config, "unknown part category '%s' (one of norm, position, mixer, feed_forward, block)", category.c_str());
  std::lock_guard<std::mutex> g(table_lock());
  const auto key = std::make_pair(category, kind);
  if (table().count(key) && !replace) LLM_THROW(Config, "%s '%s' is registered already", category.c_str(), kind.c_str());
  table()[key] = std::move(factory);
}

std::unique_ptr<Part> build_part(const std::string &category, const Json &spec, const BuildEnv &env) {
  ensure_builtin();
  if (!spec.is_object() || !spec.get("kind").is_string())
    LLM_THROW(Config, "a %s description must be an object with a 'kind'", category.c_str());
  const std::string kind = spec.get("kind").as_string();
  PartFactory factory;
  {
    std::lock_guard<std::mutex> g(table_lock());
    auto it = table().find({category, kind});
    if (it != table().end()) factory = it->second;
  }
  if (!factory) {
    std::string known;
    for (const auto &k : known_parts(category)) known += (known.empty() ? "" : ", ") + k;
    LLM_THROW(Config, "no %s of kind '%s' is registered (known: %s)", category.c_str(), kind.c_str(), known.c_str());
  }
  return factory(spec, env);
}

std::vector<std::string> known_parts(const std::string &category) {
  ensure_builtin();
  std::lock_guard<std::mutex> g(table_lock());
  std::vector<std::string> out;
  for (const auto &kv : table())
    if (kv.first.first == category) out.push_back(kv.first.second);
  return out;
}

}  // namespace llm
