// A small JSON reader/writer: enough for plan files and endpoint records.
// Numbers keep an exact int64 when the text is integral.  Objects preserve
// key order.  Parse errors throw std::runtime_error with the byte offset.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace pccl {
namespace json {

class Value {
 public:
  enum Type { kNull, kBool, kInt, kDouble, kString, kArray, kObject };
  using Array = std::vector<Value>;
  using Object = std::vector<std::pair<std::string, Value>>;

  Value() = default;
  Value(bool b) : type_(kBool), i_(b) {}
  Value(int v) : type_(kInt), i_(v) {}
  Value(int64_t v) : type_(kInt), i_(v) {}
  Value(uint64_t v) : type_(kInt), i_(static_cast<int64_t>(v)) {}
  Value(double v) : type_(kDouble), d_(v) {}
  Value(const char* s) : type_(kString), s_(s) {}
  Value(std::string s) : type_(kString), s_(std::move(s)) {}
  static Value array() { Value v; v.type_ = kArray; return v; }
  static Value object() { Value v; v.type_ = kObject; return v; }

  Type type() const { return type_; }
  bool is_null() const { return type_ == kNull; }
  bool is_number() const { return type_ == kInt || type_ == kDouble; }
  bool is_string() const { return type_ == kString; }
  bool is_array() const { return type_ == kArray; }
  bool is_object() const { return type_ == kObject; }

  bool as_bool() const { need(kBool); return i_ != 0; }
  int64_t as_int() const {
    if (type_ == kDouble) return static_cast<int64_t>(d_);
    need(kInt);
    return i_;
  }
  double as_double() const { return type_ == kInt ? static_cast<double>(i_) : (need(kDouble), d_); }
  const std::string& as_string() const { need(kString); return s_; }
  const Array& items() const { need(kArray); return a_; }
  Array& items() { need(kArray); return a_; }
  const Object& members() const { need(kObject); return o_; }

  bool contains(const std::string& key) const { return find(key) != nullptr; }
  const Value* find(const std::string& key) const {
    if (type_ != kObject) return nullptr;
    for (const auto& kv : o_) if (kv.first == key) return &kv.second;
    return nullptr;
  }
  const Value& at(const std::string& key) const {
    const Value* v = find(key);
    if (!v) throw std::runtime_error("json: missing key '" + key + "'");
    return *v;
  }
  int64_t get_int(const std::string& key, int64_t fallback) const {
    const Value* v = find(key);
    return v && v->is_number() ? v->as_int() : fallback;
  }
  std::string get_string(const std::string& key, const std::string& fallback) const {
    const Value* v = find(key);
    return v && v->is_string() ? v->as_string() : fallback;
  }
  void set(const std::string& key, Value v) {
    need(kObject);
    for (auto& kv : o_) if (kv.first == key) { kv.second = std::move(v); return; }
    o_.emplace_back(key, std::move(v));
  }
  void push(Value v) { need(kArray); a_.push_back(std::move(v)); }

  std::string dump() const;

 private:
  void need(Type t) const {
    if (type_ != t) throw std::runtime_error("json: value has a different type than requested");
  }
  Type type_ = kNull;
  int64_t i_ = 0;
  double d_ = 0;
  std::string s_;
  Array a_;
  Object o_;
};

Value parse(const std::string& text);

}  // namespace json
}  // namespace pccl
