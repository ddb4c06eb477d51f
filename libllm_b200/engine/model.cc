#include "engine/model.h"

#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <fstream>
#include <set>
#include <thread>

#include "config/config.h"
#include "csrc/kernels.h"
#include "parts/chain.h"
#include "parts/linear.h"
#include "sampling/rng.h"
#include "util/log.h"

namespace llm {

DType parse_dtype(const std::string &name) {
  if (name == "bfloat16" || name == "bf16") return DType::BF16;
  if (name == "float32" || name == "fp32" || name == "f32") return DType::F32;
  LLM_THROW(InvalidArg, "dtype '%s' is not supported (bfloat16 or float32)", name.c_str());
}

RandomLaw random_law(const TensorNeed &need, float std) {
  const bool is_bias = need.name.size() >= 4 && need.name.compare(need.name.size() - 4, 4, "bias") == 0;
  if (need.role == TensorRole::Vector && !is_bias) return {1, 0.9f, 1.1f};
  return {0, 0.f, std};
}

namespace {

class StateMapLoader : public Loader {
 public:
  StateMapLoader(const StateMap &s, DType engine) : Loader(engine), state_(s) {}
  void fetch_into(const TensorNeed &need, DType target, void *dst) const override { state_.fetch_into(need, target, dst); }
  bool has(const std::string &name) const override { return state_.has(name); }

 private:
  const StateMap &state_;
};

class RandomLoader : public Loader {
 public:
  RandomLoader(uint64_t seed, DType engine) : Loader(engine), seed_(seed) {}
  void fetch_into(const TensorNeed &need, DType target, void *dst) const override {
    if (need.role == TensorRole::Table) LLM_THROW(Weights, "%s: integer tables have no random form", need.name.c_str());
    int64_t n = 1;
    for (auto s : need.shape) n *= s;
    const RandomLaw law = random_law(need);
    // Values are drawn in 32-bit and rounded to bfloat16 once, as a stored checkpoint's are.
    kernels::random_fill(dst, target, n, tensor_seed(seed_, need.name), law.law, law.a, law.b, nullptr);
  }
  bool has(const std::string &) const override { return true; }

 private:
  uint64_t seed_;
};

}  // namespace

Model::Model(ModelSpec spec, Json config, DType dtype, int64_t max_positions, int page_size)
    : spec_(std::move(spec)), config_(std::move(config)), dtype_(dtype) {
  if (dtype != DType::F32 && dtype != DType::BF16) LLM_THROW(InvalidArg, "an engine computes in bfloat16 or float32");
  max_positions_ = max_positions > 0 ? std::min(max_positions, spec_.max_positions) : spec_.max_positions;
  env_.dtype = dtype;
  env_.max_positions = max_positions_;
  env_.page_size = page_size;
  env_.shared = &shared_;
  for (const auto &l : spec_.layers) layers_.push_back(build_as<Block>("block", l, env_));
  final_norm_ = build_as<Norm>("norm", spec_.final_norm, env_);
  for (size_t i = 0; i < spec_.schedule.size(); ++i) {
    const ScheduleEntry &e = spec_.schedule[i];
    if (e.layer < 0 || e.layer >= (int)layers_.size())
      LLM_THROW(Config, "schedule entry %zu names layer %d, the model has %zu", i, e.layer, layers_.size());
    if (e.cache_from >= (int)i)
      LLM_THROW(Config, "schedule entry %zu reads the cache of entry %d, which does not run before it", i, e.cache_from);
  }
}

std::vector<TensorNeed> Model::tensor_needs() const {
  std::vector<TensorNeed> needs;
  needs.push_back({spec_.embedding, {spec_.vocab_size, spec_.hidden}});
  for (const auto &l : layers_)
    for (auto &n : l->tensor_needs()) needs.push_back(n);
  for (auto &n : final_norm_->tensor_needs()) needs.push_back(n);
  if (!spec_.head.empty()) needs.push_back({spec_.head, {spec_.vocab_size, spec_.hidden}});
  return needs;
}

std::vector<std::string> Model::kernel_families() const {
  std::set<std::string> fams = {"elementwise", "sampling"};
  for (auto &f : product_families(dtype_)) fams.insert(f);
  for (const auto &l : layers_)
    for (auto &f : l->kernel_families()) fams.insert(f);
  for (auto &f : final_norm_->kernel_families()) fams.insert(f);
  return std::vector<std::string>(fams.begin(), fams.end());
}

bool Model::capturable() const {
  for (const auto &l : layers_)
    if (!l->capturable()) return false;
  return final_norm_->capturable();
}

void Model::load_with(const Loader &loader) {
  const std::vector<TensorNeed> needs = tensor_needs();
  embedding_ = loader.fetch(needs.front());
  for (auto &l : layers_) l->load(loader);
  final_norm_->load(loader);
  if (spec_.head.empty()) {
    head_ = &embedding_;
  } else {
    head_own_ = loader.fetch(needs.back());
    head_ = &head_own_;
  }
  LLM_CUDA(cudaDeviceSynchronize());
  loaded_ = true;
}

WeightsReport Model::load(const StateMap &state, bool strict) {
  WeightsReport report = state.check(tensor_needs(), spec_.ignore_tensors, strict);
  if (!report.unexpected.empty()) {
    std::string names;
    for (size_t i = 0; i < report.unexpected.size() && i < 8; ++i) names += (i ? ", " : "") + report.unexpected[i];
    log_warning("%s: %zu tensors are in the files but no part of the model asks for them (%s%s)", state.where().c_str(),
                report.unexpected.size(), names.c_str(), report.unexpected.size() > 8 ? ", ..." : "");
  }
  load_with(StateMapLoader(state, dtype_));
  return report;
}

void Model::load_random(uint64_t seed) { load_with(RandomLoader(seed, dtype_)); }

void Model::cache_needs(std::vector<CacheNeed> *needs, std::vector<char> *has) const {
  needs->clear();
  has->clear();
  for (const auto &e : spec_.schedule) {
    Mixer *m = layers_[(size_t)e.layer]->mixer_part();
    const bool own = m && e.cache_from < 0 && m->wants_cache();
    needs->push_back(own ? m->cache_need() : CacheNeed());
    has->push_back(own ? 1 : 0);
  }
}

std::vector<std::vector<StateNeed>> Model::state_needs() const {
  std::vector<std::vector<StateNeed>> out;
  for (const auto &e : spec_.schedule) {
    Mixer *m = layers_[(size_t)e.layer]->mixer_part();
    out.push_back(m ? m->state_need() : std::vector<StateNeed>());
  }
  return out;
}

Act Model::forward(StepContext &ctx, KVCache &cache, const std::vector<const int *> &tables, int table_width,
                   const int *fed_tokens, const int *fed_rows) {
  if (!loaded_) LLM_THROW(InvalidArg, "the model has no weights yet");
  const int64_t T = ctx.n_tokens, H = spec_.hidden;
  float *resid = ctx.arena->alloc_n<float>((size_t)(T * H));
  kernels::embedding(embedding_.dtype, embedding_.data(), ctx.tokens, fed_tokens, fed_rows, resid, (int)T, (int)H,
                     (int)spec_.vocab_size, ctx.stream);
  if (spec_.embedding_scale != 1.0) kernels::scale_rows(resid, T * H, (float)spec_.embedding_scale, ctx.stream);
  ResidualStream stream;
  stream.resid = resid;
  stream.rows = T;
  stream.hidden = H;
  Arena *const step_arena = ctx.arena;
  for (size_t i = 0; i < spec_.schedule.size(); ++i) {
    const ScheduleEntry &e = spec_.schedule[i];
    if (ctx.layer_arenas[0] && ctx.layer_arenas[1]) {
      ctx.arena = ctx.layer_arenas[i & 1];
      ctx.arena->reset();
    }
    const bool last = i + 1 == spec_.schedule.size();
    ctx.rows_read_after = last && ctx.n_want > 0 && ctx.n_want < ctx.n_tokens ? ctx.want_rows : nullptr;
    ctx.n_rows_read_after = ctx.rows_read_after ? ctx.n_want : 0;
    ctx.nothing_read_after = last && ctx.n_want == 0;
    LayerCache lc;
    const bool has_cache = cache.layer_cache((int)i, e.cache_from, tables, table_width, &lc);
    StateView sv = cache.state_view((int)i);
    layers_[(size_t)e.layer]->forward(ctx, stream, has_cache ? &lc : nullptr, sv.empty() ? nullptr : &sv);
  }
  ctx.arena = step_arena;
  ctx.nothing_read_after = false;
  if (ctx.n_want == 0) {
    flush_chain(ctx);
    return Act();
  }
  ctx.rows_read_after = nullptr;
  ctx.nothing_read_after = false;
  Act h = stream.picked ? final_norm_->forward(ctx, stream) : final_norm_->forward(ctx, stream, ctx.want_rows, ctx.n_want);
  Act logits = linear(ctx, h, *head_, nullptr, DType::F32);
  flush_chain(ctx);
  if (spec_.logit_scale != 1.0 || spec_.logit_softcap > 0.0)
    kernels::logit_transform((float *)logits.data, logits.rows * logits.cols, (float)spec_.logit_scale, (float)spec_.logit_softcap,
                             ctx.stream);
  return logits;
}

std::unique_ptr<Model> model_from_config(const Json &config_json, DType dtype, int64_t max_positions) {
  if (!config_json.is_object() || !config_json.get("model_type").is_string())
    LLM_THROW(Config, "config.json: required key 'model_type' is missing");
  const Architecture &arch = architecture_for(config_json.get("model_type").as_string());
  Json normal = arch.parse(config_json);
  ModelSpec spec = arch.describe(normal);
  return std::unique_ptr<Model>(new Model(std::move(spec), std::move(normal), dtype, max_positions));
}

// ---------------------------------------------------------------- random weights on the host
void random_tensor_host(const TensorNeed &need, uint64_t seed, std::vector<float> *out) {
  if (need.role == TensorRole::Table) LLM_THROW(Weights, "%s: integer tables have no random form", need.name.c_str());
  int64_t n = 1;
  for (auto s : need.shape) n *= s;
  out->resize((size_t)n);
  const RandomLaw law = random_law(need);
  const uint64_t ts = tensor_seed(seed, need.name);
  float *dst = out->data();
  auto work = [=](int64_t a, int64_t b) {
    for (int64_t i = a; i < b; ++i) {
      const uint64_t h1 = splitmix64(ts ^ splitmix64((uint64_t)i)), h2 = splitmix64(h1);
      const double u1 = ((double)(h1 >> 40) + 1.0) / 16777216.0, u2 = (double)(h2 >> 40) / 16777216.0;
      dst[i] = law.law == 0 ? (float)(law.a + law.b * std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2))
                            : (float)(law.a + (law.b - law.a) * u2);
    }
  };
  const int workers = (int)std::min<int64_t>(std::max(1u, std::thread::hardware_concurrency()), (n + (1 << 18) - 1) >> 18);
  if (workers <= 1) {
    work(0, n);
  } else {
    std::vector<std::thread> pool;
    const int64_t per = (n + workers - 1) / workers;
    for (int w = 0; w < workers; ++w)
      if (w * per < n) pool.emplace_back(work, w * per, std::min(n, (w + 1) * per));
    for (auto &t : pool) t.join();
  }
}

void create_random_model(const std::string &folder, const Json &config_json, uint64_t seed, const std::string &dtype) {
  const DType dt = parse_dtype(dtype);
  std::unique_ptr<Model> model = model_from_config(config_json, dt);
  ::mkdir(folder.c_str(), 0777);
  {
    std::ofstream f(folder + "/config.json");
    if (!f) LLM_THROW(Weights, "%s: cannot write config.json", folder.c_str());
    f << config_json.dump(1) << "\n";
  }
  std::vector<NamedTensor> tensors;
  std::vector<std::vector<uint8_t>> storage;
  std::vector<float> values;
  for (const auto &need : model->tensor_needs()) {
    if (need.optional) continue;
    random_tensor_host(need, seed, &values);
    NamedTensor nt;
    nt.name = need.name;
    nt.tensor.shape = need.shape;
    if (dt == DType::BF16) {
      storage.emplace_back(values.size() * 2);
      uint16_t *p = (uint16_t *)storage.back().data();
      for (size_t i = 0; i < values.size(); ++i) p[i] = float_to_bf16(values[i]);
      nt.tensor.dtype = StoredType::BF16;
    } else {
      storage.emplace_back(values.size() * 4);
      std::copy(values.begin(), values.end(), (float *)storage.back().data());
      nt.tensor.dtype = StoredType::F32;
    }
    nt.tensor.data = storage.back().data();
    nt.tensor.nbytes = storage.back().size();
    tensors.push_back(nt);
  }
  Json meta = Json::object();
  meta.set("format", "pt");
  write_safetensors(folder + "/model.safetensors", tensors, meta);
}

}  // namespace llm
