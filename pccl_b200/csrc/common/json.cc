#include "json.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>

namespace pccl {
namespace json {
namespace {

class Parser {
 public:
  explicit Parser(const std::string& t) : t_(t) {}
  Value run() {
    Value v = value();
    ws();
    if (p_ != t_.size()) fail("trailing characters");
    return v;
  }

 private:
  [[noreturn]] void fail(const std::string& what) const {
    throw std::runtime_error("json: " + what + " at byte " + std::to_string(p_));
  }
  void ws() { while (p_ < t_.size() && (t_[p_] == ' ' || t_[p_] == '\n' || t_[p_] == '\t' || t_[p_] == '\r')) ++p_; }
  char peek() { ws(); if (p_ >= t_.size()) fail("unexpected end"); return t_[p_]; }
  void expect(char c) { if (peek() != c) fail(std::string("expected '") + c + "'"); ++p_; }
  bool literal(const char* word) {
    size_t n = 0; while (word[n]) ++n;
    if (t_.compare(p_, n, word) == 0) { p_ += n; return true; }
    return false;
  }

  Value value() {
    char c = peek();
    if (c == '{') return object();
    if (c == '[') return array();
    if (c == '"') return Value(string());
    if (literal("true")) return Value(true);
    if (literal("false")) return Value(false);
    if (literal("null")) return Value();
    return number();
  }
  Value object() {
    Value v = Value::object();
    expect('{');
    if (peek() == '}') { ++p_; return v; }
    for (;;) {
      if (peek() != '"') fail("expected a string key");
      std::string key = string();
      expect(':');
      v.set(key, value());
      char c = peek();
      ++p_;
      if (c == '}') return v;
      if (c != ',') fail("expected ',' or '}'");
    }
  }
  Value array() {
    Value v = Value::array();
    expect('[');
    if (peek() == ']') { ++p_; return v; }
    for (;;) {
      v.push(value());
      char c = peek();
      ++p_;
      if (c == ']') return v;
      if (c != ',') fail("expected ',' or ']'");
    }
  }
  std::string string() {
    expect('"');
    std::string out;
    while (p_ < t_.size()) {
      char c = t_[p_++];
      if (c == '"') return out;
      if (c != '\\') { out.push_back(c); continue; }
      if (p_ >= t_.size()) break;
      char e = t_[p_++];
      switch (e) {
        case 'n': out.push_back('\n'); break;
        case 't': out.push_back('\t'); break;
        case 'r': out.push_back('\r'); break;
        case 'b': out.push_back('\b'); break;
        case 'f': out.push_back('\f'); break;
        case 'u': {
          if (p_ + 4 > t_.size()) fail("short \\u escape");
          unsigned code = static_cast<unsigned>(std::strtoul(t_.substr(p_, 4).c_str(), nullptr, 16));
          p_ += 4;
          if (code < 0x80) out.push_back(static_cast<char>(code));
          else if (code < 0x800) { out.push_back(static_cast<char>(0xC0 | (code >> 6))); out.push_back(static_cast<char>(0x80 | (code & 0x3F))); }
          else { out.push_back(static_cast<char>(0xE0 | (code >> 12))); out.push_back(static_cast<char>(0x80 | ((code >> 6) & 0x3F))); out.push_back(static_cast<char>(0x80 | (code & 0x3F))); }
          break;
        }
        default: out.push_back(e);
      }
    }
    fail("unterminated string");
  }
  Value number() {
    size_t start = p_;
    bool integral = true;
    if (p_ < t_.size() && (t_[p_] == '-' || t_[p_] == '+')) ++p_;
    while (p_ < t_.size()) {
      char c = t_[p_];
      if (c >= '0' && c <= '9') { ++p_; continue; }
      if (c == '.' || c == 'e' || c == 'E' || c == '-' || c == '+') { integral = false; ++p_; continue; }
      break;
    }
    if (p_ == start) fail("unexpected character");
    std::string tok = t_.substr(start, p_ - start);
    if (integral) return Value(static_cast<int64_t>(std::strtoll(tok.c_str(), nullptr, 10)));
    return Value(std::strtod(tok.c_str(), nullptr));
  }

  const std::string& t_;
  size_t p_ = 0;
};

void escape(const std::string& s, std::string* out) {
  out->push_back('"');
  for (unsigned char c : s) {
    switch (c) {
      case '"': *out += "\\\""; break;
      case '\\': *out += "\\\\"; break;
      case '\n': *out += "\\n"; break;
      case '\t': *out += "\\t"; break;
      case '\r': *out += "\\r"; break;
      default:
        if (c < 0x20) { char buf[8]; std::snprintf(buf, sizeof buf, "\\u%04x", c); *out += buf; }
        else out->push_back(static_cast<char>(c));
    }
  }
  out->push_back('"');
}

void dump_into(const Value& v, std::string* out) {
  switch (v.type()) {
    case Value::kNull: *out += "null"; break;
    case Value::kBool: *out += v.as_bool() ? "true" : "false"; break;
    case Value::kInt: *out += std::to_string(v.as_int()); break;
    case Value::kDouble: { char buf[40]; std::snprintf(buf, sizeof buf, "%.17g", v.as_double()); *out += buf; break; }
    case Value::kString: escape(v.as_string(), out); break;
    case Value::kArray: {
      out->push_back('[');
      bool first = true;
      for (const auto& item : v.items()) { if (!first) out->push_back(','); first = false; dump_into(item, out); }
      out->push_back(']');
      break;
    }
    case Value::kObject: {
      out->push_back('{');
      bool first = true;
      for (const auto& kv : v.members()) {
        if (!first) out->push_back(',');
        first = false;
        escape(kv.first, out);
        out->push_back(':');
        dump_into(kv.second, out);
      }
      out->push_back('}');
      break;
    }
  }
}

}  // namespace

Value parse(const std::string& text) { return Parser(text).run(); }

std::string Value::dump() const {
  std::string out;
  dump_into(*this, &out);
  return out;
}

}  // namespace json
}  // namespace pccl
