// Parts and architectures that come through the C interface of include/llm_plugin.h: adapters
// from the function tables to the classes of parts/part.h.
#include <cstring>

#include "config/config.h"
#include "csrc/kernels.h"
#include "include/llm_plugin.h"
#include "parts/chain.h"
#include "parts/part.h"

namespace llm {
namespace {

std::string plugin_error(const llm_part_vtable_t &vt, const char *what) {
  const char *msg = vt.last_error ? vt.last_error(vt.user) : nullptr;
  return std::string(what) + (msg && *msg ? std::string(": ") + msg : std::string(" failed"));
}

std::string env_json(const BuildEnv &env) {
  Json j = Json::object();
  j.set("dtype", dtype_name(env.dtype));
  j.set("max_positions", env.max_positions);
  j.set("page_size", env.page_size);
  return j.dump();
}

DType dtype_of_name(const std::string &n) {
  if (n == "float32") return DType::F32;
  if (n == "bfloat16") return DType::BF16;
  if (n == "int32") return DType::I32;
  LLM_THROW(Config, "a plug-in names the element type '%s' (float32, bfloat16 or int32)", n.c_str());
}

llm_act_t to_c(const Act &a) {
  llm_act_t c;
  c.data = a.data;
  c.dtype = (int32_t)a.dtype;
  c.rows = a.rows;
  c.cols = a.cols;
  c.ld = a.ld;
  c.parts = a.parts;
  c.part_stride = a.part_stride;
  return c;
}

llm_step_t to_c(const StepContext &ctx) {
  llm_step_t s;
  memset(&s, 0, sizeof(s));
  s.dtype = (int32_t)ctx.dtype;
  s.stream = (void *)ctx.stream;
  s.n_tokens = ctx.n_tokens;
  s.n_seqs = ctx.n_seqs;
  s.n_want = ctx.n_want;
  s.tokens = ctx.tokens;
  s.tok_seq = ctx.tok_seq;
  s.tok_pos = ctx.tok_pos;
  s.seq_start = ctx.seq_start;
  s.seq_past = ctx.seq_past;
  s.seq_slot = ctx.seq_slot;
  s.want_rows = ctx.want_rows;
  s.q_lens = ctx.q_lens.data();
  s.past_lens = ctx.past_lens.data();
  s.slots = ctx.slots.data();
  s.max_q_len = ctx.max_q_len;
  s.max_kv_len = ctx.max_kv_len;
  s.decode_only = ctx.decode_only;
  s.captured = ctx.captured;
  return s;
}

// What every adapter shares: the instance, its tensors and their loading.
class PluginCore {
 public:
  PluginCore(const llm_part_vtable_t &vt, const Json &spec, const BuildEnv &env) : vt_(vt) {
    if (!vt_.create) LLM_THROW(Config, "a plug-in part needs a create function");
    self_ = vt_.create(spec.dump().c_str(), env_json(env).c_str(), vt_.user);
    if (!self_) throw Error(ErrorKind::Config, plugin_error(vt_, "building a plug-in part"));
  }
  ~PluginCore() {
    if (self_ && vt_.destroy) vt_.destroy(self_);
  }
  std::vector<TensorNeed> tensor_needs() const {
    std::vector<TensorNeed> out;
    if (!vt_.tensor_needs) return out;
    const char *text = vt_.tensor_needs(self_);
    if (!text) throw Error(ErrorKind::Config, plugin_error(vt_, "a plug-in's tensor_needs"));
    const Json j = Json::parse(text, "a plug-in's tensor needs");
    if (!j.is_array()) LLM_THROW(Config, "a plug-in's tensor needs must be a list");
    for (const auto &e : j.items()) {
      ConfigReader r(e, "a plug-in's tensor need");
      TensorNeed n;
      n.name = r.string("name");
      if (!e.get("shape").is_array()) r.fail("'shape' must be a list");
      for (const auto &d : e.get("shape").items()) n.shape.push_back(d.as_int());
      const std::string role = r.string_or("role", "matrix");
      n.role = role == "vector" ? TensorRole::Vector : role == "table" ? TensorRole::Table : TensorRole::Matrix;
      n.optional = r.boolean_or("optional", false);
      out.push_back(n);
    }
    return out;
  }
  void load(const Loader &l) {
    for (const auto &need : tensor_needs()) {
      if (need.optional && !l.has(need.name)) continue;
      weights_.push_back(l.fetch(need));
      const Weight &w = weights_.back();
      if (vt_.load_tensor &&
          vt_.load_tensor(self_, need.name.c_str(), w.data(), (int32_t)w.dtype, need.shape.data(), (int32_t)need.shape.size()) != 0)
        throw Error(ErrorKind::Weights, plugin_error(vt_, ("a plug-in's load_tensor for " + need.name).c_str()));
    }
  }
  const llm_part_vtable_t &vt() const { return vt_; }
  void *self() const { return self_; }

 private:
  llm_part_vtable_t vt_;
  void *self_ = nullptr;
  std::vector<Weight> weights_;
};

class PluginMixer : public Mixer {
 public:
  PluginMixer(const llm_part_vtable_t &vt, const Json &spec, const BuildEnv &env) : Mixer(spec, env), core_(vt, spec, env) {
    if (!vt.mixer_forward) LLM_THROW(Config, "a plug-in mixer needs mixer_forward");
    if (vt.needs) {
      const char *text = vt.needs(core_.self());
      if (!text) throw Error(ErrorKind::Config, plugin_error(vt, "a plug-in's needs"));
      const Json j = Json::parse(text, "a plug-in's needs");
      const Json &c = j.get("cache");
      if (c.is_object()) {
        ConfigReader r(c, "a plug-in's cache need");
        has_cache_ = true;
        cache_.kind = r.string_or("kind", "full");
        cache_.n_kv_heads = (int)r.integer("n_kv_heads");
        cache_.k_dim = (int)r.integer("k_dim");
        cache_.v_dim = (int)r.integer_or("v_dim", cache_.k_dim, 0);
        cache_.window = (int)r.integer_or("window", 0, 0);
        if (cache_.kind != "full" && cache_.kind != "window") r.fail("'kind' must be \"full\" or \"window\"");
      }
      const Json &st = j.get("state");
      if (st.is_array())
        for (const auto &e : st.items()) {
          ConfigReader r(e, "a plug-in's state need");
          StateNeed n;
          n.name = r.string("name");
          if (!e.get("shape").is_array() || e.get("shape").size() > 4) r.fail("'shape' must be a list of at most 4 sizes");
          for (const auto &d : e.get("shape").items()) n.shape.push_back(d.as_int());
          n.dtype = dtype_of_name(r.string_or("dtype", "float32"));
          state_.push_back(n);
        }
    }
  }
  std::vector<TensorNeed> tensor_needs() const override { return core_.tensor_needs(); }
  void load(const Loader &l) override { core_.load(l); }
  bool capturable() const override { return core_.vt().capturable != 0; }
  bool wants_cache() const override { return has_cache_; }
  CacheNeed cache_need() const override { return cache_; }
  std::vector<StateNeed> state_need() const override { return state_; }
  Act forward(StepContext &ctx, const Act &x, LayerCache *cache, StateView *state) override {
    flush_chain(ctx);                  // the part launches on the stream itself
    const int64_t width = core_.vt().out_width > 0 ? core_.vt().out_width : x.cols;
    Act out = ctx.arena->act(DType::F32, x.rows, width);
    const llm_step_t step = to_c(ctx);
    const llm_act_t cx = to_c(x);
    llm_act_t cout = to_c(out);
    llm_layer_cache_t lc;
    if (cache) {
      memset(&lc, 0, sizeof(lc));
      lc.k = cache->k;
      lc.v = cache->v;
      lc.n_pages = cache->n_pages;
      lc.page_table = cache->page_table;
      lc.table_width = cache->table_width;
      lc.page_size = cache->page_size;
      lc.writes = cache->writes;
      lc.group = cache->group;
      lc.dtype = (int32_t)cache->dtype;
      lc.n_kv_heads = cache->need.n_kv_heads;
      lc.k_dim = cache->need.k_dim;
      lc.v_dim = cache->need.v_dim;
      lc.window = cache->need.window;
    }
    std::vector<llm_state_tensor_t> st;
    if (state)
      for (const auto &t : *state) {
        llm_state_tensor_t c;
        memset(&c, 0, sizeof(c));
        c.name = t.name.c_str();
        c.data = t.data;
        c.ndim = (int32_t)t.shape.size();
        for (size_t i = 0; i < t.shape.size() && i < 4; ++i) c.shape[i] = t.shape[i];
        c.dtype = (int32_t)t.dtype;
        c.n_slots = t.n_slots;
        st.push_back(c);
      }
    if (core_.vt().mixer_forward(core_.self(), &step, &cx, cache ? &lc : nullptr, st.data(), (int32_t)st.size(), &cout) != 0)
      throw Error(ErrorKind::Extension, plugin_error(core_.vt(), "a plug-in mixer's forward"));
    return out;
  }

 private:
  PluginCore core_;
  bool has_cache_ = false;
  CacheNeed cache_;
  std::vector<StateNeed> state_;
};

class PluginFeedForward : public FeedForward {
 public:
  PluginFeedForward(const llm_part_vtable_t &vt, const Json &spec, const BuildEnv &env) : FeedForward(spec, env), core_(vt, spec, env) {
    if (!vt.ff_forward) LLM_THROW(Config, "a plug-in feed-forward needs ff_forward");
  }
  std::vector<TensorNeed> tensor_needs() const override { return core_.tensor_needs(); }
  void load(const Loader &l) override { core_.load(l); }
  bool capturable() const override { return core_.vt().capturable != 0; }
  Act forward(StepContext &ctx, const Act &x) override {
    flush_chain(ctx);
    const int64_t width = core_.vt().out_width > 0 ? core_.vt().out_width : x.cols;
    Act out = ctx.arena->act(DType::F32, x.rows, width);
    const llm_step_t step = to_c(ctx);
    const llm_act_t cx = to_c(x);
    llm_act_t cout = to_c(out);
    if (core_.vt().ff_forward(core_.self(), &step, &cx, &cout) != 0)
      throw Error(ErrorKind::Extension, plugin_error(core_.vt(), "a plug-in feed-forward's forward"));
    return out;
  }

 private:
  PluginCore core_;
};

// A position encoding that brings a table of its own angles; the rotation itself (channel i with
// i + rotary_dim/2) and the append to the cache are the library's kernels.
class PluginPosition : public PositionEncoding {
 public:
  PluginPosition(const llm_part_vtable_t &vt, const Json &spec, const BuildEnv &env) : PositionEncoding(spec, env), core_(vt, spec, env) {
    if (!vt.position_table) LLM_THROW(Config, "a plug-in position encoding needs position_table");
  }
  std::vector<TensorNeed> tensor_needs() const override { return core_.tensor_needs(); }
  void load(const Loader &l) override { core_.load(l); }
  std::vector<std::string> kernel_families() const override { return {"rope"}; }
  const float *half_split_table(int *rows, int *rotary_dim) const override {
    int32_t r = 0, d = 0;
    const float *t = core_.vt().position_table(core_.self(), &r, &d);
    if (!t) throw Error(ErrorKind::Extension, plugin_error(core_.vt(), "a plug-in position encoding's table"));
    *rows = r;
    *rotary_dim = d;
    return t;
  }
  void rotate_and_store(StepContext &ctx, const Act &qkv, const Act &q_out, const QkvLayout &l, LayerCache &cache) override {
    int rows = 0, rot = 0;
    const float *table = half_split_table(&rows, &rot);
    flush_chain(ctx);
    kernels::rope_cache_write(qkv, q_out, l.n_heads, l.n_kv_heads, l.head_dim, table, rows, rot, ctx.tok_seq, ctx.tok_pos,
                              cache.page_table, cache.table_width, cache.k, cache.v, cache.page_size, cache.writes, ctx.stream);
  }

 private:
  PluginCore core_;
};

}  // namespace
}  // namespace llm

// ---------------------------------------------------------------- the C entry points
namespace llm {
int guard_api(const std::function<void()> &body);     // capi/llm_api.cc: runs body, keeps an error's message, returns its status
}

extern "C" __attribute__((visibility("default"))) int32_t llm_register_part(const char *category, const char *kind,
                                                                              const llm_part_vtable_t *vtable, int32_t replace) {
  return llm::guard_api([&] {
    using namespace llm;
    if (!category || !kind || !vtable) LLM_THROW(InvalidArg, "llm_register_part: null argument");
    const llm_part_vtable_t vt = *vtable;
    const std::string cat = category;
    PartFactory f;
    if (cat == "mixer") f = [vt](const Json &s, const BuildEnv &e) { return std::unique_ptr<Part>(new PluginMixer(vt, s, e)); };
    else if (cat == "feed_forward") f = [vt](const Json &s, const BuildEnv &e) { return std::unique_ptr<Part>(new PluginFeedForward(vt, s, e)); };
    else if (cat == "position") f = [vt](const Json &s, const BuildEnv &e) { return std::unique_ptr<Part>(new PluginPosition(vt, s, e)); };
    else LLM_THROW(Config, "a plug-in part is a mixer, a feed_forward or a position (norms and blocks are C++ classes), not '%s'", category);
    register_part(cat, kind, f, replace != 0);
  });
}

extern "C" __attribute__((visibility("default"))) int32_t llm_register_architecture(const char *name, llm_json_fn_t parse,
                                                                                      llm_json_fn_t describe,
                                                                                      const char *(*last_error)(void *), void *user,
                                                                                      int32_t replace) {
  return llm::guard_api([&] {
    using namespace llm;
    if (!name) LLM_THROW(InvalidArg, "llm_register_architecture: null name");
    if (!parse || !describe) {
      // without functions nothing can be registered; a name that is taken is said to be taken
      for (const auto &k : known_architectures())
        if (k == name && !replace) LLM_THROW(Config, "architecture '%s' is registered already", name);
      LLM_THROW(InvalidArg, "llm_register_architecture: an architecture needs its parse and describe functions");
    }
    const std::string n = name;
    auto call = [n, last_error, user](llm_json_fn_t fn, const Json &in, const char *what) {
      const char *out = fn(in.dump().c_str(), user);
      if (!out) {
        const char *msg = last_error ? last_error(user) : nullptr;
        throw Error(ErrorKind::Config, std::string(what) + " of architecture '" + n + "'" + (msg && *msg ? std::string(": ") + msg : " failed"));
      }
      return Json::parse(out, std::string(what) + " of architecture '" + n + "'");
    };
    Architecture a;
    a.name = n;
    a.parse = [call, parse](const Json &j) { return call(parse, j, "parse"); };
    a.describe = [call, describe](const Json &j) { return ModelSpec::from_json(call(describe, j, "describe")); };
    register_architecture(std::move(a), replace != 0);
  });
}
