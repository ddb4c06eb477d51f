// The C interface (include/llm.h) over the host library.  Every function catches what the
// library throws, keeps the message for the calling thread and returns the status, as the
// reference does at the same boundary (src/libllm/llm.cc:60-71, 134-152).
#include <cstring>
#include <functional>
#include <memory>

#include "cache/kv_cache.h"
#include "config/config.h"
#include "csrc/kernels.h"
#include "engine/generate.h"
#include "engine/model.h"
#include "engine/step.h"
#include "include/llm.h"
#include "sampling/rng.h"
#include "util/log.h"

#define LLM_API extern "C" __attribute__((visibility("default")))

using namespace llm;

struct llm_json_impl_t {
  Json value;
};
struct llm_model_impl_t {
  std::unique_ptr<Engine> engine;
  WeightsReport report;
  std::string path;
};
struct llm_completion_impl_t {
  std::unique_ptr<Completion> completion;
};
struct llm_pending_impl_t {
  PendingTokens pending;
};
struct llm_cachebook_impl_t {
  std::unique_ptr<KVCache> cache;
};

namespace {
thread_local std::string g_message, g_details = "{}";
thread_local int g_kind = 0;

void keep_error(const Error &e) {
  g_message = e.what();
  g_kind = (int)e.kind();
  g_details = "{}";
  if (const WeightsError *w = dynamic_cast<const WeightsError *>(&e)) {
    Json d = Json::object();
    d.set("missing", Json::list(w->report.missing));
    d.set("unexpected", Json::list(w->report.unexpected));
    Json wrong = Json::array();
    for (const auto &ws : w->report.wrong_shape) {
      Json t = Json::array();
      t.push(ws.name);
      t.push(Json::list(ws.expected));
      t.push(Json::list(ws.found));
      wrong.push(t);
    }
    d.set("wrong_shape", wrong);
    g_details = d.dump();
  }
}

Engine &engine_of(llm_model_t *m) {
  if (!m || !*m) LLM_THROW(InvalidArg, "the model handle is null");
  if (!(*m)->engine) LLM_THROW(InvalidArg, "the model is not loaded");
  return *(*m)->engine;
}
Json &json_of(llm_json_t *j, const char *what) {
  if (!j || !*j) LLM_THROW(InvalidArg, "the %s handle is null", what);
  return (*j)->value;
}

// Options may only carry keys that the call knows (the reference checks its kwargs the same way,
// src/libllm/llm.cc:73-96).
void check_keys(const Json &kwargs, std::initializer_list<const char *> known, const char *what) {
  if (!kwargs.is_object()) LLM_THROW(InvalidArg, "%s: the options must be a JSON object", what);
  for (const auto &m : kwargs.members()) {
    bool ok = false;
    for (const char *k : known) ok = ok || m.first == k;
    if (!ok) LLM_THROW(InvalidArg, "%s: unexpected key '%s' in the options", what, m.first.c_str());
  }
}

std::vector<int> int_list(const Json &j, const char *what) {
  if (!j.is_array()) LLM_THROW(InvalidArg, "%s must be a list of integers", what);
  std::vector<int> out;
  for (const auto &v : j.items()) {
    if (!v.is_int()) LLM_THROW(InvalidArg, "%s must be a list of integers", what);
    out.push_back((int)v.as_int());
  }
  return out;
}

SamplingParams sampling_of(const Json &kwargs) {
  ConfigReader r(kwargs, "options", ErrorKind::InvalidArg);
  SamplingParams s;
  s.temperature = (float)r.number_or("temperature", 1.0, false);
  s.top_k = (int)r.integer_or("top_k", 50, -(1 << 30));
  s.top_p = (float)r.number_or("top_p", 0.8, false);
  s.validate();
  return s;
}

Engine::Options engine_options(const Json &kwargs) {
  ConfigReader r(kwargs, "options", ErrorKind::InvalidArg);
  Engine::Options o;
  o.max_tokens = r.integer_or("max_tokens", 65536);
  o.max_seq_len = r.integer_or("max_seq_len", 0, 0);
  o.max_slots = (int)r.integer_or("max_slots", 0, 0);
  o.max_step_tokens = (int)r.integer_or("max_step_tokens", 8192);
  o.use_graphs = r.boolean_or("use_graphs", true);
  o.device = (int)r.integer_or("cuda_device", 0, 0);
  const std::string device = r.string_or("device", "auto");
  if (device == "cpu") LLM_THROW(InvalidArg, "this library has no CPU path: device must be cuda or auto");
  if (device != "auto" && device != "cuda") LLM_THROW(InvalidArg, "invalid device '%s' (auto or cuda)", device.c_str());
  return o;
}

void build_items(int32_t n_items, const int32_t *slots, const int32_t *n_tokens, const int32_t *tokens, const int32_t *fed_rows,
                 const int32_t *n_want, const int32_t *want, std::vector<StepItem> *items) {
  if (n_items < 0 || (n_items > 0 && (!slots || !n_tokens || !tokens))) LLM_THROW(InvalidArg, "step: null argument");
  size_t t = 0, w = 0;
  for (int i = 0; i < n_items; ++i) {
    StepItem it;
    it.slot = slots[i];
    if (n_tokens[i] < 0) LLM_THROW(InvalidArg, "step: a negative number of tokens");
    it.tokens.assign(tokens + t, tokens + t + n_tokens[i]);
    t += (size_t)n_tokens[i];
    const int nw = n_want ? n_want[i] : 1;
    if (nw < 0 || (nw > 0 && !want)) LLM_THROW(InvalidArg, "step: wanted places are missing");
    it.want.assign(want + w, want + w + nw);
    w += (size_t)nw;
    it.fed_row = fed_rows ? fed_rows[i] : -1;
    items->push_back(std::move(it));
  }
}
}  // namespace

namespace llm {
int guard_api(const std::function<void()> &body) {
  try {
    body();
    return STATUS_OK;
  } catch (const Error &e) {
    keep_error(e);
    return e.status();
  } catch (const std::exception &e) {
    g_message = e.what();
    g_kind = (int)ErrorKind::Aborted;
    g_details = "{}";
    return STATUS_ABORTED;
  } catch (...) {
    g_message = "an unknown failure";
    g_kind = (int)ErrorKind::Aborted;
    g_details = "{}";
    return STATUS_ABORTED;
  }
}
}  // namespace llm

// ---------------------------------------------------------------- global state
LLM_API void llm_init(void) { known_architectures(); }
LLM_API const char *llm_get_last_error_message(void) { return g_message.c_str(); }
LLM_API int32_t llm_get_last_error_kind(void) { return g_kind; }
LLM_API const char *llm_get_last_error_details(void) { return g_details.c_str(); }

// ---------------------------------------------------------------- JSON
LLM_API int32_t llm_json_init(llm_json_t *j) {
  return guard_api([&] {
    if (!j) LLM_THROW(InvalidArg, "the JSON handle is null");
    *j = new llm_json_impl_t();
  });
}
LLM_API int32_t llm_json_destroy(llm_json_t *j) {
  if (j && *j) {
    delete *j;
    *j = nullptr;
  }
  return STATUS_OK;
}
LLM_API int32_t llm_json_parse(llm_json_t *j, const char *json_str) {
  return guard_api([&] {
    if (!json_str) LLM_THROW(InvalidArg, "the JSON text is null");
    json_of(j, "JSON") = Json::parse(json_str);
  });
}
LLM_API int64_t llm_json_dump_size(llm_json_t *j) { return (j && *j) ? (int64_t)(*j)->value.dump().size() + 1 : 0; }
LLM_API int32_t llm_json_dump(llm_json_t *j, char *buf, int64_t buf_size) {
  int insufficient = 0;
  const int rc = guard_api([&] {
    const std::string text = json_of(j, "JSON").dump();
    if (!buf) LLM_THROW(InvalidArg, "the buffer is null");
    if ((int64_t)text.size() + 1 > buf_size) {
      insufficient = 1;
      LLM_THROW(InvalidArg, "the buffer holds %lld bytes, the text needs %zu", (long long)buf_size, text.size() + 1);
    }
    memcpy(buf, text.c_str(), text.size() + 1);
  });
  return insufficient ? STATUS_INSUFFICIENT_BUFFER : rc;
}

// ---------------------------------------------------------------- model
LLM_API int32_t llm_model_init(llm_model_t *m) {
  return guard_api([&] {
    if (!m) LLM_THROW(InvalidArg, "the model handle is null");
    *m = new llm_model_impl_t();
  });
}
LLM_API int32_t llm_model_destroy(llm_model_t *m) {
  return guard_api([&] {
    if (m && *m) {
      delete *m;
      *m = nullptr;
    }
  });
}

namespace {
const std::initializer_list<const char *> LOAD_KEYS = {"filename", "device", "dtype", "max_tokens", "max_seq_len", "max_slots",
                                                       "max_step_tokens", "use_graphs", "cuda_device", "strict", "random", "config"};

int64_t positions_for(const Json &kwargs, const Engine::Options &o) {
  // the rotary table is as long as the longest sequence this engine can hold, not as long as the
  // architecture allows
  const int64_t by_cache = (o.max_tokens + o.page_size - 1) / o.page_size * o.page_size;
  (void)kwargs;
  return o.max_seq_len > 0 ? std::min(o.max_seq_len, by_cache) : by_cache;
}
}  // namespace

LLM_API int32_t llm_model_load(llm_model_t *m, llm_json_t *kwargs) {
  return guard_api([&] {
    if (!m || !*m) LLM_THROW(InvalidArg, "the model handle is null");
    const Json &kw = json_of(kwargs, "options");
    check_keys(kw, LOAD_KEYS, "llm_model_load");
    ConfigReader r(kw, "options", ErrorKind::InvalidArg);
    const Engine::Options o = engine_options(kw);
    const DType dtype = parse_dtype(r.string_or("dtype", "bfloat16"));
    LLM_CUDA(cudaSetDevice(o.device));
    std::unique_ptr<Model> model;
    (*m)->engine.reset();
    if (kw.has("random")) {
      const Json &rnd = r.object("random");
      ConfigReader rr(rnd, "options: random", ErrorKind::InvalidArg);
      model = model_from_config(rr.object("config"), dtype, positions_for(kw, o));
      model->load_random((uint64_t)rr.integer_or("seed", 0, 0));
      (*m)->path = "<random>";
    } else {
      const std::string folder = r.string("filename");
      model = model_from_config(read_config_json(folder), dtype, positions_for(kw, o));
      std::unique_ptr<StateMap> state = StateMap::from_folder(folder);
      (*m)->report = model->load(*state, r.boolean_or("strict", true));
      (*m)->path = folder;
    }
    (*m)->engine.reset(new Engine(std::move(model), o));
  });
}

LLM_API int32_t llm_model_load_tensors(llm_model_t *m, llm_json_t *kwargs, int32_t n, const char *const *names,
                                       const char *const *dtypes, const int64_t *const *shapes, const int32_t *ndims,
                                       const void *const *data) {
  return guard_api([&] {
    if (!m || !*m) LLM_THROW(InvalidArg, "the model handle is null");
    const Json &kw = json_of(kwargs, "options");
    check_keys(kw, LOAD_KEYS, "llm_model_load_tensors");
    ConfigReader r(kw, "options", ErrorKind::InvalidArg);
    const Engine::Options o = engine_options(kw);
    const DType dtype = parse_dtype(r.string_or("dtype", "bfloat16"));
    LLM_CUDA(cudaSetDevice(o.device));
    (*m)->engine.reset();
    std::unique_ptr<Model> model = model_from_config(r.object("config"), dtype, positions_for(kw, o));
    std::unique_ptr<StateMap> state = StateMap::in_memory();
    for (int i = 0; i < n; ++i) {
      StoredTensor t;
      t.dtype = stored_type_from_name(dtypes[i], std::string("tensor '") + names[i] + "'");
      t.shape.assign(shapes[i], shapes[i] + ndims[i]);
      t.data = (const uint8_t *)data[i];
      t.nbytes = (size_t)t.numel() * stored_type_size(t.dtype);
      state->add(names[i], t);
    }
    (*m)->report = model->load(*state, r.boolean_or("strict", true));
    (*m)->path = "<memory>";
    (*m)->engine.reset(new Engine(std::move(model), o));
  });
}

LLM_API int32_t llm_model_get_info(llm_model_t *m, llm_json_t *info) {
  return guard_api([&] {
    Engine &e = engine_of(m);
    Json j = Json::object();
    j.set("name", e.model().spec().name);
    j.set("path", (*m)->path);
    j.set("config", e.model().config());
    j.set("dtype", dtype_name(e.model().dtype()));
    j.set("vocab_size", e.vocab());
    j.set("max_seq_len", e.max_seq_len());
    j.set("capacity_tokens", (int64_t)e.cache().n_pages() * e.cache().page_size());
    j.set("page_size", e.cache().page_size());
    j.set("max_step_tokens", e.options().max_step_tokens);
    j.set("use_graphs", e.options().use_graphs && e.model().capturable());
    j.set("stop_tokens", Json::list(e.model().spec().stop_tokens));
    j.set("cuda_device", e.device());
    j.set("steps_run", (int64_t)e.steps_run());
    j.set("graphs_captured", (int64_t)e.graphs_captured());
    j.set("graph_replays", (int64_t)e.graph_replays());
    j.set("chain_launches", (int64_t)e.chain_launches());
    j.set("last_tokens_capacity", e.last_tokens_capacity());
    j.set("last_step_h2d_bytes", (int64_t)e.last_step_h2d_bytes());
    j.set("last_step_d2h_bytes", (int64_t)e.last_step_d2h_bytes());
    j.set("unexpected_tensors", Json::list((*m)->report.unexpected));
    j.set("ignored_tensors", Json::list((*m)->report.ignored));
    j.set("kernel_families", Json::list(e.model().kernel_families()));
    json_of(info, "info") = j;
  });
}

// ---------------------------------------------------------------- completion
LLM_API int32_t llm_completion_init(llm_completion_t *c) {
  return guard_api([&] {
    if (!c) LLM_THROW(InvalidArg, "the completion handle is null");
    *c = new llm_completion_impl_t();
  });
}
LLM_API int32_t llm_completion_destroy(llm_completion_t *c) {
  return guard_api([&] {
    if (c && *c) {
      delete *c;
      *c = nullptr;
    }
  });
}
LLM_API int32_t llm_model_complete(llm_model_t *m, llm_json_t *kwargs, llm_completion_t *comp) {
  return guard_api([&] {
    Engine &e = engine_of(m);
    if (!comp || !*comp) LLM_THROW(InvalidArg, "the completion handle is null");
    const Json &kw = json_of(kwargs, "options");
    check_keys(kw, {"temperature", "top_k", "top_p", "prompt_ids", "max_new_tokens", "seed", "stop_token_ids"}, "llm_model_complete");
    ConfigReader r(kw, "options", ErrorKind::InvalidArg);
    std::set<int> stops;
    if (kw.has("stop_token_ids") && !kw.get("stop_token_ids").is_null())
      for (int t : int_list(kw.get("stop_token_ids"), "stop_token_ids")) stops.insert(t);
    else
      stops.insert(e.model().spec().stop_tokens.begin(), e.model().spec().stop_tokens.end());
    (*comp)->completion.reset(new Completion(e, int_list(kw.get("prompt_ids"), "prompt_ids"),
                                             (int)r.integer_or("max_new_tokens", 1 << 30, 0), sampling_of(kw),
                                             (uint64_t)r.integer_or("seed", 0, 0), stops));
  });
}
LLM_API int32_t llm_completion_get_next_chunk(llm_completion_t *c, llm_json_t *chunk) {
  return guard_api([&] {
    if (!c || !*c || !(*c)->completion) LLM_THROW(InvalidArg, "the completion has not been started");
    int token = 0;
    if (!(*c)->completion->next(&token)) throw Error(ErrorKind::Eof, "the completion has ended");
    Json j = Json::object();
    j.set("token", token);
    j.set("text", "<" + std::to_string(token) + ">");
    json_of(chunk, "chunk") = j;
  });
}

// ---------------------------------------------------------------- batched generation
LLM_API int32_t llm_model_generate(llm_model_t *m, llm_json_t *kwargs, llm_token_fn_t on_token, void *user, llm_json_t *result) {
  return guard_api([&] {
    Engine &e = engine_of(m);
    const Json &kw = json_of(kwargs, "options");
    check_keys(kw, {"prompts", "max_new_tokens", "temperature", "top_k", "top_p", "seed", "stop_token_ids", "max_batch"},
               "llm_model_generate");
    ConfigReader r(kw, "options", ErrorKind::InvalidArg);
    const Json &ps = kw.get("prompts");
    if (!ps.is_array()) LLM_THROW(InvalidArg, "prompts must be a list of lists of token ids");
    std::vector<std::vector<int>> prompts;
    for (const auto &p : ps.items()) prompts.push_back(int_list(p, "a prompt"));
    std::vector<int> limits;
    const Json &mn = kw.get("max_new_tokens");
    if (mn.is_array()) limits = int_list(mn, "max_new_tokens");
    else limits = {(int)r.integer_or("max_new_tokens", 64, -(1 << 30))};
    GenerateOptions go;
    go.sampling = sampling_of(kw);
    go.seed = (uint64_t)r.integer_or("seed", 0, 0);
    go.max_batch = (int)r.integer_or("max_batch", 64);
    if (kw.has("stop_token_ids") && !kw.get("stop_token_ids").is_null()) {
      go.use_model_stop_tokens = false;
      go.stop_tokens = int_list(kw.get("stop_token_ids"), "stop_token_ids");
    }
    if (on_token) go.on_token = [on_token, user](int req, int tok) { on_token(req, tok, user); };
    const auto out = generate(e, prompts, limits, go);
    Json toks = Json::array();
    for (const auto &o : out) toks.push(Json::list(o));
    Json j = Json::object();
    j.set("tokens", toks);
    json_of(result, "result") = j;
  });
}

// ---------------------------------------------------------------- sequences and steps
LLM_API int32_t llm_model_open_sequence(llm_model_t *m, int32_t *slot) {
  return guard_api([&] { *slot = engine_of(m).open_sequence(); });
}
LLM_API int32_t llm_model_close_sequence(llm_model_t *m, int32_t slot) {
  return guard_api([&] { engine_of(m).close_sequence(slot); });
}
LLM_API int32_t llm_model_sequence_length(llm_model_t *m, int32_t slot, int32_t *length) {
  return guard_api([&] { *length = engine_of(m).sequence_length(slot); });
}

LLM_API int32_t llm_model_step(llm_model_t *m, int32_t n_items, const int32_t *slots, const int32_t *n_tokens, const int32_t *tokens,
                               const int32_t *fed_rows, const int32_t *n_want, const int32_t *want, const char *sampling_json,
                               const float *uniforms, float *logits, int32_t *sampled) {
  return guard_api([&] {
    Engine &e = engine_of(m);
    std::vector<StepItem> items;
    build_items(n_items, slots, n_tokens, tokens, fed_rows, n_want, want, &items);
    if (sampling_json) {
      const SamplingParams s = sampling_of(Json::parse(sampling_json, "sampling"));
      const StepResult r = e.step(items, &s, uniforms);
      if (logits) e.read_logits(r, logits);
      if (sampled) e.read_tokens(r, sampled);
      if (!logits && !sampled) e.check_status();
    } else {
      const StepResult r = e.step(items);
      if (logits) e.read_logits(r, logits);
      else e.check_status();
    }
  });
}

LLM_API int32_t llm_model_step_tokens(llm_model_t *m, int32_t n_items, const int32_t *slots, const int32_t *n_tokens,
                                      const int32_t *tokens, const int32_t *fed_rows, const int32_t *want, const char *sampling_json,
                                      const float *uniforms, llm_pending_t *pending) {
  return guard_api([&] {
    Engine &e = engine_of(m);
    if (!pending) LLM_THROW(InvalidArg, "step_tokens: the pending handle is null");
    std::vector<StepItem> items;
    build_items(n_items, slots, n_tokens, tokens, fed_rows, nullptr, want, &items);
    const SamplingParams s = sampling_of(sampling_json ? Json::parse(sampling_json, "sampling") : Json::object());
    std::unique_ptr<llm_pending_impl_t> p(new llm_pending_impl_t());
    p->pending = e.step_tokens(items, s, uniforms);
    *pending = p.release();
  });
}
LLM_API int32_t llm_pending_result(llm_pending_t *pending, int32_t *tokens) {
  return guard_api([&] {
    if (!pending || !*pending) LLM_THROW(InvalidArg, "the pending handle is null");
    std::unique_ptr<llm_pending_impl_t> p(*pending);
    *pending = nullptr;
    const std::vector<int> t = p->pending.result();
    if (tokens) std::copy(t.begin(), t.end(), tokens);
  });
}
LLM_API int32_t llm_pending_destroy(llm_pending_t *pending) {
  if (pending && *pending) {
    delete *pending;
    *pending = nullptr;
  }
  return STATUS_OK;
}
LLM_API int32_t llm_model_synchronize(llm_model_t *m) {
  return guard_api([&] { engine_of(m).synchronize(); });
}
LLM_API int32_t llm_model_stream(llm_model_t *m, void **cuda_stream) {
  return guard_api([&] { *cuda_stream = (void *)engine_of(m).stream(); });
}

// ---------------------------------------------------------------- cache
LLM_API int32_t llm_model_cache_info(llm_model_t *m, llm_json_t *info) {
  return guard_api([&] { json_of(info, "info") = engine_of(m).cache().info(); });
}
LLM_API int32_t llm_model_cache_check(llm_model_t *m) {
  return guard_api([&] { engine_of(m).cache().check(); });
}
LLM_API int32_t llm_model_debug_set_status(llm_model_t *m, int32_t code) {
  return guard_api([&] {
    Engine &e = engine_of(m);
    e.make_current();
    LLM_CUDA(cudaMemcpyAsync(e.status_word(), &code, sizeof(int), cudaMemcpyHostToDevice, e.stream()));
    LLM_CUDA(cudaStreamSynchronize(e.stream()));
  });
}
LLM_API int32_t llm_model_debug_wait_probe(llm_model_t *m, int64_t limit_ns) {
  return guard_api([&] {
    Engine &e = engine_of(m);
    e.make_current();
    kernels::gemm_tc_wait_probe(limit_ns, e.status_word(), e.stream());
  });
}

// ---------------------------------------------------------------- configuration, registries, weights
LLM_API int32_t llm_known_architectures(llm_json_t *out) {
  return guard_api([&] { json_of(out, "out") = Json::list(known_architectures()); });
}
LLM_API int32_t llm_load_config(const char *folder, llm_json_t *out) {
  return guard_api([&] { json_of(out, "out") = load_config(folder ? folder : ""); });
}
LLM_API int32_t llm_parse_config(llm_json_t *config_json, llm_json_t *out) {
  return guard_api([&] {
    const Json parsed = parse_config(json_of(config_json, "config"));
    json_of(out, "out") = parsed;
  });
}

namespace {
Json needs_json(const std::vector<TensorNeed> &needs) {
  Json a = Json::array();
  for (const auto &n : needs) {
    Json o = Json::object();
    o.set("name", n.name);
    o.set("shape", Json::list(n.shape));
    o.set("role", n.role == TensorRole::Vector ? "vector" : n.role == TensorRole::Table ? "table" : "matrix");
    o.set("optional", n.optional);
    a.push(o);
  }
  return a;
}
std::vector<TensorNeed> needs_from(const Json &j) {
  if (!j.is_array()) LLM_THROW(InvalidArg, "tensor needs must be a list");
  std::vector<TensorNeed> out;
  for (const auto &e : j.items()) {
    ConfigReader r(e, "a tensor need", ErrorKind::InvalidArg);
    TensorNeed n;
    n.name = r.string("name");
    for (const auto &d : e.get("shape").items()) n.shape.push_back(d.as_int());
    const std::string role = r.string_or("role", "matrix");
    n.role = role == "vector" ? TensorRole::Vector : role == "table" ? TensorRole::Table : TensorRole::Matrix;
    n.optional = r.boolean_or("optional", false);
    out.push_back(n);
  }
  return out;
}
}  // namespace

LLM_API int32_t llm_describe_model(llm_json_t *config_json, const char *dtype, llm_json_t *out) {
  return guard_api([&] {
    std::unique_ptr<Model> model = model_from_config(json_of(config_json, "config"), parse_dtype(dtype ? dtype : "bfloat16"));
    Json j = Json::object();
    j.set("spec", model->spec().to_json());
    j.set("config", model->config());
    j.set("tensor_needs", needs_json(model->tensor_needs()));
    j.set("kernel_families", Json::list(model->kernel_families()));
    j.set("capturable", model->capturable());
    json_of(out, "out") = j;
  });
}
LLM_API int32_t llm_create_random_model(const char *folder, llm_json_t *config_json, uint64_t seed, const char *dtype) {
  return guard_api([&] {
    if (!folder) LLM_THROW(InvalidArg, "the folder is null");
    create_random_model(folder, json_of(config_json, "config"), seed, dtype ? dtype : "bfloat16");
  });
}
LLM_API int32_t llm_check_weights(const char *folder, llm_json_t *needs, llm_json_t *ignore, int32_t strict, llm_json_t *report) {
  return guard_api([&] {
    std::unique_ptr<StateMap> state = StateMap::from_folder(folder ? folder : "");
    std::vector<std::string> ign;
    if (ignore && *ignore && (*ignore)->value.is_array())
      for (const auto &p : (*ignore)->value.items()) ign.push_back(p.as_string());
    const WeightsReport r = state->check(needs_from(json_of(needs, "needs")), ign, strict != 0);
    Json j = Json::object();
    j.set("missing", Json::list(r.missing));
    j.set("unexpected", Json::list(r.unexpected));
    j.set("ignored", Json::list(r.ignored));
    j.set("names", Json::list(state->names()));
    if (report && *report) (*report)->value = j;
  });
}
LLM_API int32_t llm_read_safetensors_header(const char *path, llm_json_t *out) {
  return guard_api([&] {
    SafetensorsFile f(path ? path : "");
    Json j = Json::object();
    for (const auto &n : f.names()) {
      Json e = Json::object();
      e.set("dtype", stored_type_name(f.tensor(n).dtype));
      e.set("shape", Json::list(f.tensor(n).shape));
      e.set("nbytes", f.tensor(n).nbytes);
      j.set(n, e);
    }
    json_of(out, "out") = j;
  });
}
LLM_API int32_t llm_set_kernel_library(const char *family, const char *path) {
  return guard_api([&] {
    if (!family || !path) LLM_THROW(InvalidArg, "llm_set_kernel_library: null argument");
    kernels::set_library(family, path);
  });
}
LLM_API int32_t llm_loaded_kernel_libraries(llm_json_t *out) {
  return guard_api([&] { json_of(out, "out") = Json::list(kernels::loaded_libraries()); });
}
LLM_API int64_t llm_kernel_launches(void) { return kernels::launches(); }
LLM_API int32_t llm_rotary_frequencies(int64_t rotary_dim, double theta, llm_json_t *scaling, double *out) {
  return guard_api([&] {
    const Json s = (scaling && *scaling) ? (*scaling)->value : Json();
    const std::vector<double> f = rotary_frequencies(rotary_dim, theta, s);
    std::copy(f.begin(), f.end(), out);
  });
}
LLM_API float llm_uniform(uint64_t seed, uint64_t sequence, uint64_t step) { return uniform(seed, sequence, step); }
LLM_API int32_t llm_plan_batches(llm_json_t *in, llm_json_t *out) {
  return guard_api([&] {
    const Json &j = json_of(in, "in");
    ConfigReader r(j, "plan_batches", ErrorKind::InvalidArg);
    const auto batches = plan_batches(int_list(j.get("prompt_lengths"), "prompt_lengths"), int_list(j.get("max_new_tokens"), "max_new_tokens"),
                                      r.integer("capacity_tokens"), (int)r.integer("max_batch"), (int)r.integer_or("page_size", 64),
                                      r.integer_or("max_seq_len", 0, 0));
    Json a = Json::array();
    for (const auto &b : batches) a.push(Json::list(b));
    json_of(out, "out") = a;
  });
}
LLM_API int32_t llm_should_stop(int32_t token, int32_t n_generated, int32_t max_new_tokens, llm_json_t *stop_tokens, llm_json_t *out) {
  return guard_api([&] {
    std::set<int> stops;
    for (int t : int_list(json_of(stop_tokens, "stop_tokens"), "stop_tokens")) stops.insert(t);
    const StopDecision d = should_stop(token, n_generated, max_new_tokens, stops);
    Json j = Json::object();
    j.set("ends", d.ends);
    j.set("emit", d.emit);
    json_of(out, "out") = j;
  });
}
LLM_API int32_t llm_validate_sampling(double temperature, int32_t top_k, double top_p) {
  return guard_api([&] {
    SamplingParams s;
    s.temperature = (float)temperature;
    s.top_k = top_k;
    s.top_p = (float)top_p;
    s.validate();
  });
}

// ---------------------------------------------------------------- the cache's bookkeeping alone
LLM_API int32_t llm_cachebook_init(llm_cachebook_t *c, llm_json_t *spec) {
  return guard_api([&] {
    if (!c) LLM_THROW(InvalidArg, "the handle is null");
    const Json &j = json_of(spec, "spec");
    ConfigReader r(j, "cache description", ErrorKind::InvalidArg);
    std::vector<CacheNeed> needs;
    std::vector<char> has;
    if (!j.get("runs").is_array()) LLM_THROW(InvalidArg, "cache description: 'runs' must be a list");
    for (const auto &e : j.get("runs").items()) {
      CacheNeed n;
      if (e.is_object()) {
        ConfigReader er(e, "cache need", ErrorKind::InvalidArg);
        n.kind = er.string_or("kind", "full");
        n.n_kv_heads = (int)er.integer("n_kv_heads");
        n.k_dim = (int)er.integer("k_dim");
        n.v_dim = (int)er.integer_or("v_dim", n.k_dim, 0);
        n.window = (int)er.integer_or("window", 0, 0);
      }
      needs.push_back(n);
      has.push_back(e.is_object() ? 1 : 0);
    }
    std::vector<std::vector<StateNeed>> states(needs.size());
    const Json &st = j.get("states");
    if (st.is_array())
      for (size_t i = 0; i < st.size() && i < states.size(); ++i)
        for (const auto &e : st.at(i).items()) {
          StateNeed n;
          n.name = e.get("name").as_string();
          for (const auto &d : e.get("shape").items()) n.shape.push_back(d.as_int());
          states[i].push_back(n);
        }
    std::unique_ptr<llm_cachebook_impl_t> impl(new llm_cachebook_impl_t());
    impl->cache.reset(new KVCache(needs, has, states, r.integer("capacity_tokens", -(1ll << 40)), DType::F32, (int)r.integer_or("page_size", 64, -(1 << 30)),
                                  (int)r.integer_or("max_slots", 0, 0), false));
    *c = impl.release();
  });
}
LLM_API int32_t llm_cachebook_destroy(llm_cachebook_t *c) {
  if (c && *c) {
    delete *c;
    *c = nullptr;
  }
  return STATUS_OK;
}
namespace {
KVCache &book(llm_cachebook_t *c) {
  if (!c || !*c || !(*c)->cache) LLM_THROW(InvalidArg, "the cache handle is null");
  return *(*c)->cache;
}
}  // namespace
LLM_API int32_t llm_cachebook_open(llm_cachebook_t *c, int32_t *slot) {
  return guard_api([&] { *slot = book(c).open(); });
}
LLM_API int32_t llm_cachebook_close(llm_cachebook_t *c, int32_t slot) {
  return guard_api([&] { book(c).close(slot); });
}
LLM_API int32_t llm_cachebook_reserve(llm_cachebook_t *c, int32_t n, const int32_t *slots, const int32_t *new_lengths) {
  return guard_api([&] {
    std::vector<std::pair<int, int>> growth;
    for (int i = 0; i < n; ++i) growth.push_back({slots[i], new_lengths[i]});
    book(c).reserve(growth);
  });
}
LLM_API int32_t llm_cachebook_commit(llm_cachebook_t *c, int32_t slot, int32_t new_length) {
  return guard_api([&] { book(c).commit(slot, new_length); });
}
LLM_API int32_t llm_cachebook_page_table(llm_cachebook_t *c, int32_t group, int32_t n, const int32_t *slots, int32_t width, int32_t *out) {
  return guard_api([&] {
    KVCache &k = book(c);
    if (group < 0 || group >= (int)k.groups().size()) LLM_THROW(InvalidArg, "group %d does not exist", group);
    k.page_table(group, std::vector<int>(slots, slots + n), width, out);
  });
}
LLM_API int32_t llm_cachebook_check(llm_cachebook_t *c) {
  return guard_api([&] { book(c).check(); });
}
LLM_API int32_t llm_cachebook_info(llm_cachebook_t *c, llm_json_t *info) {
  return guard_api([&] { json_of(info, "info") = book(c).info(); });
}

// A script of operations on a page pool or a slot table, for tests of their checks.
// in: {"kind": "pages" | "slots", "n": N, "ops": [{"op": "take", "n": k} | {"op": "give_back", "pages": [...] | "slot": s} | {"op": "check"}]}
// out: [{"result": ..., "error": null | message, "available": a, "in_use": u}]
LLM_API int32_t llm_debug_pool_script(llm_json_t *in, llm_json_t *out) {
  return guard_api([&] {
    const Json &j = json_of(in, "in");
    const bool pages = j.get("kind").as_string() == "pages";
    std::unique_ptr<PagePool> pool;
    std::unique_ptr<SlotTable> slots;
    if (pages) pool.reset(new PagePool((int)j.get("n").as_int()));
    else slots.reset(new SlotTable((int)j.get("n").as_int()));
    Json results = Json::array();
    for (const auto &op : j.get("ops").items()) {
      Json r = Json::object();
      r.set("result", Json());
      r.set("error", Json());
      try {
        const std::string name = op.get("op").as_string();
        if (name == "take") {
          if (pages) r.set("result", Json::list(pool->take((int)op.get("n").as_int())));
          else r.set("result", slots->take());
        } else if (name == "give_back") {
          if (pages) pool->give_back(int_list(op.get("pages"), "pages"));
          else slots->give_back((int)op.get("slot").as_int());
        } else if (name == "check") {
          if (pages) pool->check();
        } else if (name == "held") {
          if (!pages) r.set("result", Json::list(slots->held()));
        }
      } catch (const Error &e) {
        r.set("error", std::string(e.what()));
      }
      r.set("available", pages ? pool->available() : slots->available());
      r.set("in_use", pages ? pool->in_use() : slots->n_slots() - slots->available());
      results.push(r);
    }
    json_of(out, "out") = results;
  });
}
