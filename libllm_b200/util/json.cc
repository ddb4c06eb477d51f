#include "util/json.h"

#include <cmath>
#include <cstdlib>
#include <cstring>

namespace llm {

const char *Json::type_name() const {
  static const char *names[] = {"null", "a boolean", "an integer", "a number", "a string", "an array", "an object"};
  return names[type_];
}

const Json *Json::find(const std::string &key) const {
  for (const auto &m : members_)
    if (m.first == key) return &m.second;
  return nullptr;
}

const Json &Json::get(const std::string &key) const {
  static const Json null_value;
  const Json *p = find(key);
  return p ? *p : null_value;
}

Json &Json::set(const std::string &key, Json v) {
  if (type_ == Null) type_ = Object;
  for (auto &m : members_)
    if (m.first == key) {
      m.second = std::move(v);
      return m.second;
    }
  members_.emplace_back(key, std::move(v));
  return members_.back().second;
}

// ---------------------------------------------------------------- writing
static void dump_string(std::string &out, const std::string &s) {
  out.push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\r': out += "\\r"; break;
      case '\t': out += "\\t"; break;
      default:
        if (c < 0x20) {
          char buf[8];
          snprintf(buf, sizeof(buf), "\\u%04x", c);
          out += buf;
        } else {
          out.push_back((char)c);
        }
    }
  }
  out.push_back('"');
}

void Json::dump_to(std::string &out, int indent, int depth) const {
  auto newline = [&](int d) {
    if (indent < 0) return;
    out.push_back('\n');
    out.append((size_t)(indent * d), ' ');
  };
  switch (type_) {
    case Null: out += "null"; break;
    case Bool: out += int_ ? "true" : "false"; break;
    case Int: out += std::to_string(int_); break;
    case Real: {
      if (!std::isfinite(real_)) {
        out += "null";
        break;
      }
      char buf[40];
      snprintf(buf, sizeof(buf), "%.17g", real_);
      // the shortest form that reads back to the same number
      for (int p = 1; p < 17; ++p) {
        char t[40];
        snprintf(t, sizeof(t), "%.*g", p, real_);
        if (strtod(t, nullptr) == real_) {
          memcpy(buf, t, sizeof(t));
          break;
        }
      }
      out += buf;
      if (!strpbrk(buf, ".eEn")) out += ".0";
      break;
    }
    case String: dump_string(out, str_); break;
    case Array:
      out.push_back('[');
      for (size_t i = 0; i < items_.size(); ++i) {
        if (i) out += indent < 0 ? "," : ",";
        newline(depth + 1);
        items_[i].dump_to(out, indent, depth + 1);
      }
      if (!items_.empty()) newline(depth);
      out.push_back(']');
      break;
    case Object:
      out.push_back('{');
      for (size_t i = 0; i < members_.size(); ++i) {
        if (i) out.push_back(',');
        newline(depth + 1);
        dump_string(out, members_[i].first);
        out += indent < 0 ? ":" : ": ";
        members_[i].second.dump_to(out, indent, depth + 1);
      }
      if (!members_.empty()) newline(depth);
      out.push_back('}');
      break;
  }
}

std::string Json::dump(int indent) const {
  std::string out;
  dump_to(out, indent, 0);
  return out;
}

// ---------------------------------------------------------------- reading
namespace {
struct Parser {
  const std::string &s;
  const std::string &where;
  size_t i = 0;
  int depth = 0;

  [[noreturn]] void fail(const char *what) const {
    LLM_THROW(InvalidArg, "%s: not valid JSON (%s at byte %zu)", where.c_str(), what, i);
  }
  void skip() {
    while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i;
  }
  bool eat(const char *word) {
    const size_t n = strlen(word);
    if (s.compare(i, n, word) == 0) {
      i += n;
      return true;
    }
    return false;
  }
  static void put_utf8(std::string &out, unsigned cp) {
    if (cp < 0x80) out.push_back((char)cp);
    else if (cp < 0x800) {
      out.push_back((char)(0xC0 | (cp >> 6)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    } else if (cp < 0x10000) {
      out.push_back((char)(0xE0 | (cp >> 12)));
      out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    } else {
      out.push_back((char)(0xF0 | (cp >> 18)));
      out.push_back((char)(0x80 | ((cp >> 12) & 0x3F)));
      out.push_back((char)(0x80 | ((cp >> 6) & 0x3F)));
      out.push_back((char)(0x80 | (cp & 0x3F)));
    }
  }
  unsigned hex4() {
    if (i + 4 > s.size()) fail("a short \\u escape");
    unsigned v = 0;
    for (int k = 0; k < 4; ++k) {
      const char c = s[i++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= (unsigned)(c - '0');
      else if (c >= 'a' && c <= 'f') v |= (unsigned)(c - 'a' + 10);
      else if (c >= 'A' && c <= 'F') v |= (unsigned)(c - 'A' + 10);
      else fail("a bad \\u escape");
    }
    return v;
  }
  std::string string() {
    std::string out;
    ++i;  // the opening quote
    for (;;) {
      if (i >= s.size()) fail("an unterminated string");
      const char c = s[i++];
      if (c == '"') return out;
      if ((unsigned char)c < 0x20) fail("a control character in a string");
      if (c != '\\') {
        out.push_back(c);
        continue;
      }
      if (i >= s.size()) fail("an unterminated escape");
      const char e = s[i++];
      switch (e) {
        case '"': out.push_back('"'); break;
        case '\\': out.push_back('\\'); break;
        case '/': out.push_back('/'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'n': out.push_back('\n'); break;
        case 'r': out.push_back('\r'); break;
        case 't': out.push_back('\t'); break;
        case 'u': {
          unsigned cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && s.compare(i, 2, "\\u") == 0) {
            i += 2;
            const unsigned lo = hex4();
            if (lo >= 0xDC00 && lo < 0xE000) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          put_utf8(out, cp);
          break;
        }
        default: fail("an unknown escape");
      }
    }
  }
  Json number() {
    const size_t start = i;
    bool real = false;
    if (s[i] == '-') ++i;
    if (i >= s.size() || !(s[i] >= '0' && s[i] <= '9')) fail("a malformed number");
    while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
    if (i < s.size() && s[i] == '.') {
      real = true;
      ++i;
      if (i >= s.size() || !(s[i] >= '0' && s[i] <= '9')) fail("a malformed number");
      while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
    }
    if (i < s.size() && (s[i] == 'e' || s[i] == 'E')) {
      real = true;
      ++i;
      if (i < s.size() && (s[i] == '+' || s[i] == '-')) ++i;
      if (i >= s.size() || !(s[i] >= '0' && s[i] <= '9')) fail("a malformed number");
      while (i < s.size() && s[i] >= '0' && s[i] <= '9') ++i;
    }
    const std::string text = s.substr(start, i - start);
    if (!real && text.size() <= 18) return Json((int64_t)strtoll(text.c_str(), nullptr, 10));
    return Json(strtod(text.c_str(), nullptr));
  }
  Json value() {
    skip();
    if (i >= s.size()) fail("an unexpected end");
    if (++depth > 200) fail("nesting too deep");
    Json out;
    const char c = s[i];
    if (c == '{') {
      ++i;
      out = Json::object();
      skip();
      if (i < s.size() && s[i] == '}') {
        ++i;
      } else {
        for (;;) {
          skip();
          if (i >= s.size() || s[i] != '"') fail("a key expected");
          std::string key = string();
          skip();
          if (i >= s.size() || s[i] != ':') fail("':' expected");
          ++i;
          out.set(key, value());
          skip();
          if (i < s.size() && s[i] == ',') {
            ++i;
            continue;
          }
          if (i < s.size() && s[i] == '}') {
            ++i;
            break;
          }
          fail("',' or '}' expected");
        }
      }
    } else if (c == '[') {
      ++i;
      out = Json::array();
      skip();
      if (i < s.size() && s[i] == ']') {
        ++i;
      } else {
        for (;;) {
          out.push(value());
          skip();
          if (i < s.size() && s[i] == ',') {
            ++i;
            continue;
          }
          if (i < s.size() && s[i] == ']') {
            ++i;
            break;
          }
          fail("',' or ']' expected");
        }
      }
    } else if (c == '"') {
      out = Json(string());
    } else if (c == '-' || (c >= '0' && c <= '9')) {
      out = number();
    } else if (eat("true")) {
      out = Json(true);
    } else if (eat("false")) {
      out = Json(false);
    } else if (eat("null")) {
      out = Json();
    } else if (eat("NaN")) {
      out = Json(std::nan(""));
    } else if (eat("Infinity")) {
      out = Json(HUGE_VAL);
    } else if (eat("-Infinity")) {
      out = Json(-HUGE_VAL);
    } else {
      fail("an unexpected character");
    }
    --depth;
    return out;
  }
};
}  // namespace

Json Json::parse(const std::string &text, const std::string &where) {
  Parser p{text, where};
  Json v = p.value();
  p.skip();
  if (p.i != text.size()) p.fail("text after the value");
  return v;
}

}  // namespace llm
