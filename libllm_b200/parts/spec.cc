#include "parts/spec.h"

#include "config/config.h"

namespace llm {

Json ModelSpec::to_json() const {
  Json j = Json::object();
  j.set("name", name);
  j.set("vocab_size", vocab_size);
  j.set("hidden", hidden);
  j.set("embedding", embedding);
  Json ls = Json::array();
  for (const auto &l : layers) ls.push(l);
  j.set("layers", ls);
  Json sch = Json::array();
  for (const auto &e : schedule) {
    Json o = Json::object();
    o.set("layer", e.layer);
    o.set("cache_from", e.cache_from < 0 ? Json() : Json(e.cache_from));
    sch.push(o);
  }
  j.set("schedule", sch);
  j.set("final_norm", final_norm);
  j.set("head", head.empty() ? Json() : Json(head));
  j.set("max_positions", max_positions);
  j.set("stop_tokens", Json::list(stop_tokens));
  j.set("embedding_scale", embedding_scale);
  j.set("logit_scale", logit_scale);
  j.set("logit_softcap", logit_softcap);
  j.set("ignore_tensors", Json::list(ignore_tensors));
  return j;
}

ModelSpec ModelSpec::from_json(const Json &j) {
  if (!j.is_object()) LLM_THROW(Config, "a model description must be an object");
  ConfigReader r(j, "model description");
  ModelSpec s;
  s.name = r.string_or("name", "");
  s.vocab_size = r.integer("vocab_size");
  s.hidden = r.integer("hidden");
  s.embedding = r.string("embedding");
  const Json &ls = j.get("layers");
  if (!ls.is_array()) r.fail("'layers' must be a list of block descriptions");
  for (const auto &l : ls.items()) {
    if (!l.is_object() || !l.get("kind").is_string()) r.fail("every layer is an object with a 'kind'");
    s.layers.push_back(l);
  }
  const Json &sch = j.get("schedule");
  if (sch.is_null()) {
    for (size_t i = 0; i < s.layers.size(); ++i) s.schedule.push_back({(int)i, -1});
  } else {
    if (!sch.is_array()) r.fail("'schedule' must be a list");
    for (const auto &e : sch.items()) {
      ScheduleEntry se;
      if (e.is_int()) {
        se.layer = (int)e.as_int();
      } else if (e.is_object()) {
        ConfigReader er(e, "model description: schedule entry");
        se.layer = (int)er.integer("layer", 0);
        se.cache_from = (int)er.integer_or("cache_from", -1, 0);
      } else {
        r.fail("a schedule entry is a layer number or {layer, cache_from}");
      }
      s.schedule.push_back(se);
    }
  }
  s.final_norm = r.object("final_norm");
  s.head = r.string_or("head", "");
  s.max_positions = r.integer("max_positions");
  const Json &st = j.get("stop_tokens");
  if (st.is_array())
    for (const auto &t : st.items()) {
      if (!t.is_int()) r.fail("'stop_tokens' must be integers");
      s.stop_tokens.push_back((int)t.as_int());
    }
  s.embedding_scale = r.number_or("embedding_scale", 1.0);
  s.logit_scale = r.number_or("logit_scale", 1.0);
  s.logit_softcap = r.number_or("logit_softcap", 0.0, false);
  const Json &ig = j.get("ignore_tensors");
  if (ig.is_array())
    for (const auto &t : ig.items())
      if (t.is_string()) s.ignore_tensors.push_back(t.as_string());
  return s;
}

}  // namespace llm
