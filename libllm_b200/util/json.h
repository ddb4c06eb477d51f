// A small JSON value: what config.json, the header of a safetensors file, the options of the C
// API and the description of a model are read from and written to.  The reference brings
// nlohmann's header for the same jobs (src/libllm/llm.cc:73-96); this one keeps the order of an
// object's keys, tells integers from other numbers (config.json's sizes must be integers) and
// reports the position of a syntax error.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "util/error.h"

namespace llm {

class Json {
 public:
  enum Type { Null, Bool, Int, Real, String, Array, Object };
  using Member = std::pair<std::string, Json>;

  Json() : type_(Null) {}
  Json(std::nullptr_t) : type_(Null) {}
  Json(bool b) : type_(Bool), int_(b) {}
  Json(int v) : type_(Int), int_(v) {}
  Json(int64_t v) : type_(Int), int_(v) {}
  Json(size_t v) : type_(Int), int_((int64_t)v) {}
  Json(double v) : type_(Real), real_(v) {}
  Json(const char *s) : type_(String), str_(s) {}
  Json(const std::string &s) : type_(String), str_(s) {}
  static Json array() { Json j; j.type_ = Array; return j; }
  static Json object() { Json j; j.type_ = Object; return j; }
  template <typename T>
  static Json list(const std::vector<T> &v) {
    Json j = array();
    for (const auto &x : v) j.push(Json(x));
    return j;
  }

  Type type() const { return type_; }
  bool is_null() const { return type_ == Null; }
  bool is_bool() const { return type_ == Bool; }
  bool is_int() const { return type_ == Int; }
  bool is_number() const { return type_ == Int || type_ == Real; }
  bool is_string() const { return type_ == String; }
  bool is_array() const { return type_ == Array; }
  bool is_object() const { return type_ == Object; }
  const char *type_name() const;

  bool as_bool() const { return int_ != 0; }
  int64_t as_int() const { return type_ == Real ? (int64_t)real_ : int_; }
  double as_number() const { return type_ == Int ? (double)int_ : real_; }
  const std::string &as_string() const { return str_; }

  // arrays
  size_t size() const { return type_ == Array ? items_.size() : members_.size(); }
  const Json &at(size_t i) const { return items_.at(i); }
  Json &at(size_t i) { return items_.at(i); }
  void push(Json v) { items_.push_back(std::move(v)); }
  const std::vector<Json> &items() const { return items_; }

  // objects (insertion order kept)
  bool has(const std::string &key) const { return find(key) != nullptr; }
  const Json *find(const std::string &key) const;
  const Json &get(const std::string &key) const;       // a shared null when absent
  Json &set(const std::string &key, Json v);
  const std::vector<Member> &members() const { return members_; }

  std::string dump(int indent = -1) const;
  // Throws Error(InvalidArg) naming `where` and the byte offset of the fault.
  static Json parse(const std::string &text, const std::string &where = "JSON");

 private:
  void dump_to(std::string &out, int indent, int depth) const;
  Type type_;
  int64_t int_ = 0;
  double real_ = 0;
  std::string str_;
  std::vector<Json> items_;
  std::vector<Member> members_;
};

}  // namespace llm
