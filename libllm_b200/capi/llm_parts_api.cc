// One part alone, through the C interface: built from its description, given its tensors, and
// run on device memory that the caller brings.  It is how the tests check each part of a layer
// against the plain implementation's function for it, and how a part in the making can be tried
// without a model around it.  The step's arrays, the input and the cache are the caller's device
// pointers (as integers in the call's JSON); what the part returns lies in memory of the handle's
// own and stays valid until the next call on the same handle.  Everything runs on the default
// stream.
#include <cstring>
#include <functional>
#include <memory>

#include "include/llm.h"
#include "parts/part.h"
#include "engine/model.h"
#include "config/config.h"

#define LLM_API extern "C" __attribute__((visibility("default")))

using namespace llm;

struct llm_json_impl_t {
  Json value;
};

struct llm_part_impl_t {
  std::string category;
  BuildEnv env;
  std::map<std::string, std::shared_ptr<Weight>> shared;
  std::unique_ptr<Part> part;
  Arena arena{(size_t)8 << 20};
  DeviceBuffer status, counters;
};
typedef llm_part_impl_t *llm_part_t;

namespace llm {
int guard_api(const std::function<void()> &body);
}

namespace {
class MapLoader : public Loader {
 public:
  MapLoader(const StateMap &s, DType engine) : Loader(engine), state_(s) {}
  void fetch_into(const TensorNeed &need, DType target, void *dst) const override { state_.fetch_into(need, target, dst); }
  bool has(const std::string &name) const override { return state_.has(name); }

 private:
  const StateMap &state_;
};

void *ptr_of(const Json &j) { return j.is_null() ? nullptr : (void *)(uintptr_t)j.as_int(); }

Act act_from(const Json &j) {
  Act a;
  if (!j.is_object()) return a;
  a.data = ptr_of(j.get("ptr"));
  a.dtype = parse_dtype(j.get("dtype").as_string());
  a.rows = j.get("rows").as_int();
  a.cols = j.get("cols").as_int();
  a.ld = j.has("ld") ? j.get("ld").as_int() : a.cols;
  a.parts = j.has("parts") ? (int)j.get("parts").as_int() : 1;
  a.part_stride = j.has("part_stride") ? j.get("part_stride").as_int() : a.rows * a.cols;
  return a;
}

Json act_json(const Act &a) {
  if (!a.data) return Json();
  Json j = Json::object();
  j.set("ptr", (int64_t)(uintptr_t)a.data);
  j.set("dtype", dtype_name(a.dtype));
  j.set("rows", a.rows);
  j.set("cols", a.cols);
  j.set("ld", a.ld);
  j.set("parts", a.parts);
  j.set("part_stride", a.part_stride);
  return j;
}

std::vector<int> ints(const Json &j) {
  std::vector<int> out;
  if (j.is_array())
    for (const auto &v : j.items()) out.push_back((int)v.as_int());
  return out;
}

llm_part_impl_t &part_of(llm_part_t *p) {
  if (!p || !*p || !(*p)->part) LLM_THROW(InvalidArg, "the part handle is null");
  return **p;
}
}  // namespace

LLM_API int32_t llm_part_build(llm_part_t *p, const char *category, llm_json_t *spec, const char *dtype, int64_t max_positions) {
  return guard_api([&] {
    if (!p || !category || !spec || !*spec) LLM_THROW(InvalidArg, "llm_part_build: null argument");
    std::unique_ptr<llm_part_impl_t> impl(new llm_part_impl_t());
    impl->category = category;
    impl->env.dtype = parse_dtype(dtype ? dtype : "bfloat16");
    impl->env.max_positions = max_positions;
    impl->env.shared = &impl->shared;
    impl->part = build_part(category, (*spec)->value, impl->env);
    *p = impl.release();
  });
}

LLM_API int32_t llm_part_destroy(llm_part_t *p) {
  return guard_api([&] {
    if (p && *p) {
      delete *p;
      *p = nullptr;
    }
  });
}

// out: {"tensor_needs": [...], "kernel_families": [...], "capturable": bool,
//       "cache": null | {...}, "state": [...]} (the last two for mixers)
LLM_API int32_t llm_part_describe(llm_part_t *p, llm_json_t *out) {
  return guard_api([&] {
    llm_part_impl_t &h = part_of(p);
    Json j = Json::object();
    Json needs = Json::array();
    for (const auto &n : h.part->tensor_needs()) {
      Json o = Json::object();
      o.set("name", n.name);
      o.set("shape", Json::list(n.shape));
      o.set("role", n.role == TensorRole::Vector ? "vector" : n.role == TensorRole::Table ? "table" : "matrix");
      o.set("optional", n.optional);
      needs.push(o);
    }
    j.set("tensor_needs", needs);
    j.set("kernel_families", Json::list(h.part->kernel_families()));
    j.set("capturable", h.part->capturable());
    if (Mixer *m = dynamic_cast<Mixer *>(h.part.get())) {
      if (m->wants_cache()) {
        const CacheNeed c = m->cache_need();
        Json cj = Json::object();
        cj.set("kind", c.kind);
        cj.set("n_kv_heads", c.n_kv_heads);
        cj.set("k_dim", c.k_dim);
        cj.set("v_dim", c.v_dim);
        cj.set("window", c.window > 0 ? Json(c.window) : Json());
        j.set("cache", cj);
      } else {
        j.set("cache", Json());
      }
      Json st = Json::array();
      for (const auto &s : m->state_need()) {
        Json o = Json::object();
        o.set("name", s.name);
        o.set("shape", Json::list(s.shape));
        o.set("dtype", dtype_name(s.dtype));
        st.push(o);
      }
      j.set("state", st);
    }
    if (!out || !*out) LLM_THROW(InvalidArg, "the out handle is null");
    (*out)->value = j;
  });
}

LLM_API int32_t llm_part_load(llm_part_t *p, int32_t n, const char *const *names, const char *const *dtypes,
                              const int64_t *const *shapes, const int32_t *ndims, const void *const *data) {
  return guard_api([&] {
    llm_part_impl_t &h = part_of(p);
    std::unique_ptr<StateMap> state = StateMap::in_memory();
    for (int i = 0; i < n; ++i) {
      StoredTensor t;
      t.dtype = stored_type_from_name(dtypes[i], std::string("tensor '") + names[i] + "'");
      t.shape.assign(shapes[i], shapes[i] + ndims[i]);
      t.data = (const uint8_t *)data[i];
      t.nbytes = (size_t)t.numel() * stored_type_size(t.dtype);
      state->add(names[i], t);
    }
    state->check(h.part->tensor_needs(), {}, true);
    h.part->load(MapLoader(*state, h.env.dtype));
    LLM_CUDA(cudaDeviceSynchronize());
  });
}

// call: {"step": {"n_tokens", "n_seqs", "tokens", "tok_seq", "tok_pos", "seq_start", "seq_past", "seq_slot" (device
//         pointers), "q_lens", "past_lens", "slots" (lists), "max_q_len", "max_kv_len", "decode_only"},
//        "x": {"ptr", "dtype", "rows", "cols"},                      mixers, feed-forwards
//        "resid": ptr, "pending": null | {...}, "rows": null | ptr, "n_rows": n        norms, blocks
//        "cache": null | {"k", "v", "n_pages", "page_table", "table_width", "page_size", "writes"},
//        "state": [{"name", "ptr", "shape", "dtype", "n_slots"}]}
// result: {"out": {...}} (norm, mixer, feed_forward), {"pending": {...}} (norm, block),
//         {"table": {"ptr", "rows", "rotary_dim"}} (position)
LLM_API int32_t llm_part_forward(llm_part_t *p, llm_json_t *call, llm_json_t *result) {
  return guard_api([&] {
    llm_part_impl_t &h = part_of(p);
    if (!call || !*call || !result || !*result) LLM_THROW(InvalidArg, "llm_part_forward: null argument");
    const Json &c = (*call)->value;
    const Json &s = c.get("step");
    if (!h.status) {
      h.status.allocate(sizeof(int), true);
      h.counters.allocate(sizeof(int) << 16, true);
    }
    h.arena.reset();
    StepContext ctx;
    ctx.dtype = h.env.dtype;
    ctx.stream = nullptr;
    ctx.n_tokens = (int)s.get("n_tokens").as_int();
    ctx.n_seqs = (int)s.get("n_seqs").as_int();
    ctx.tokens = (const int *)ptr_of(s.get("tokens"));
    ctx.tok_seq = (const int *)ptr_of(s.get("tok_seq"));
    ctx.tok_pos = (const int *)ptr_of(s.get("tok_pos"));
    ctx.seq_start = (const int *)ptr_of(s.get("seq_start"));
    ctx.seq_past = (const int *)ptr_of(s.get("seq_past"));
    ctx.seq_slot = (const int *)ptr_of(s.get("seq_slot"));
    ctx.q_lens = ints(s.get("q_lens"));
    ctx.past_lens = ints(s.get("past_lens"));
    ctx.slots = ints(s.get("slots"));
    ctx.max_q_len = (int)s.get("max_q_len").as_int();
    ctx.max_kv_len = (int)s.get("max_kv_len").as_int();
    ctx.decode_only = s.get("decode_only").as_bool();
    ctx.arena = &h.arena;
    ctx.tc_status = h.status.as<int>();
    ctx.zero_counters = h.counters.as<int>();
    ctx.n_zero_counters = 1 << 16;
    int dev = 0;
    LLM_CUDA(cudaGetDevice(&dev));
    LLM_CUDA(cudaDeviceGetAttribute(&ctx.sm_count, cudaDevAttrMultiProcessorCount, dev));

    LayerCache lc;
    bool has_cache = false;
    if (c.get("cache").is_object()) {
      const Json &cj = c.get("cache");
      has_cache = true;
      lc.k = ptr_of(cj.get("k"));
      lc.v = ptr_of(cj.get("v"));
      lc.n_pages = cj.get("n_pages").as_int();
      lc.page_table = (const int *)ptr_of(cj.get("page_table"));
      lc.table_width = (int)cj.get("table_width").as_int();
      lc.page_size = cj.has("page_size") ? (int)cj.get("page_size").as_int() : h.env.page_size;
      lc.writes = !cj.has("writes") || cj.get("writes").as_bool();
      lc.dtype = h.env.dtype;
      if (Mixer *m = dynamic_cast<Mixer *>(h.part.get())) lc.need = m->cache_need();
      if (Block *b = dynamic_cast<Block *>(h.part.get()))
        if (b->mixer_part()) lc.need = b->mixer_part()->cache_need();
    }
    StateView state;
    if (c.get("state").is_array())
      for (const auto &e : c.get("state").items()) {
        StateTensor t;
        t.name = e.get("name").as_string();
        t.data = ptr_of(e.get("ptr"));
        for (const auto &d : e.get("shape").items()) t.shape.push_back(d.as_int());
        t.dtype = parse_dtype(e.get("dtype").as_string());
        t.n_slots = e.get("n_slots").as_int();
        state.push_back(t);
      }

    Json out = Json::object();
    ResidualStream stream;
    stream.resid = (float *)ptr_of(c.get("resid"));
    stream.rows = ctx.n_tokens;
    stream.pending = act_from(c.get("pending"));
    if (Norm *norm = dynamic_cast<Norm *>(h.part.get())) {
      stream.hidden = c.get("hidden").as_int();
      const int *rows = (const int *)ptr_of(c.get("rows"));
      out.set("out", act_json(norm->forward(ctx, stream, rows, rows ? (int)c.get("n_rows").as_int() : 0)));
      out.set("pending", act_json(stream.pending));
    } else if (Mixer *mixer = dynamic_cast<Mixer *>(h.part.get())) {
      out.set("out", act_json(mixer->forward(ctx, act_from(c.get("x")), has_cache ? &lc : nullptr, state.empty() ? nullptr : &state)));
    } else if (FeedForward *ff = dynamic_cast<FeedForward *>(h.part.get())) {
      out.set("out", act_json(ff->forward(ctx, act_from(c.get("x")))));
    } else if (Block *block = dynamic_cast<Block *>(h.part.get())) {
      stream.hidden = c.get("hidden").as_int();
      block->forward(ctx, stream, has_cache ? &lc : nullptr, state.empty() ? nullptr : &state);
      out.set("pending", act_json(stream.pending));
    } else if (PositionEncoding *pos = dynamic_cast<PositionEncoding *>(h.part.get())) {
      int rows = 0, rot = 0;
      const float *t = pos->half_split_table(&rows, &rot);
      Json tj = Json::object();
      tj.set("ptr", (int64_t)(uintptr_t)t);
      tj.set("rows", rows);
      tj.set("rotary_dim", rot);
      out.set("table", tj);
    }
    LLM_CUDA(cudaDeviceSynchronize());
    int code = 0;
    LLM_CUDA(cudaMemcpy(&code, h.status.get(), sizeof(int), cudaMemcpyDeviceToHost));
    if (code) {
      cudaMemset(h.status.get(), 0, sizeof(int));
      LLM_THROW(Extension, "a tensor-core kernel gave up waiting on a barrier (code %d)", code);
    }
    (*result)->value = out;
  });
}
