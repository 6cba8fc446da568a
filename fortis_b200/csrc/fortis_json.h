// Minimal JSON reader for the layout descriptors (gather.json, scatter.json, loop.json, kdist.json, lift2d.json).
// Header-only, no dependencies.  Numbers are kept as double (and as text, so that "1.0e-30" keeps its spelling).
#pragma once
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace fortis {

struct JValue {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;                       // string value, or the literal text of a number
  std::vector<JValue> arr;
  std::vector<std::pair<std::string, JValue>> obj;

  bool is_null() const { return kind == Null; }
  bool truthy() const { return kind == Bool ? b : kind == Num ? num != 0.0 : kind != Null; }
  const JValue* find(const std::string& k) const {
    if (kind != Obj) return nullptr;
    for (auto& kv : obj) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  const JValue& at(const std::string& k) const {
    const JValue* v = find(k);
    if (!v) throw std::runtime_error("descriptor: missing key \"" + k + "\"");
    return *v;
  }
  const JValue& at(size_t i) const {
    if (kind != Arr || i >= arr.size()) throw std::runtime_error("descriptor: array index out of range");
    return arr[i];
  }
  long as_long() const {
    if (kind != Num) throw std::runtime_error("descriptor: expected a number");
    return (long)num;
  }
  const std::string& as_str() const {
    if (kind != Str) throw std::runtime_error("descriptor: expected a string");
    return str;
  }
  size_t size() const { return kind == Arr ? arr.size() : kind == Obj ? obj.size() : 0; }
};

class JParser {
 public:
  explicit JParser(const std::string& s) : s_(s) {}
  JValue parse() {
    JValue v = value();
    ws();
    if (p_ != s_.size()) fail("trailing characters");
    return v;
  }

 private:
  const std::string& s_;
  size_t p_ = 0;
  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string("descriptor JSON: ") + what + " at byte " + std::to_string(p_));
  }
  void ws() { while (p_ < s_.size() && (s_[p_] == ' ' || s_[p_] == '\n' || s_[p_] == '\t' || s_[p_] == '\r')) p_++; }
  JValue value() {
    ws();
    if (p_ >= s_.size()) fail("unexpected end");
    char c = s_[p_];
    JValue v;
    if (c == '{') {
      v.kind = JValue::Obj; p_++; ws();
      if (p_ < s_.size() && s_[p_] == '}') { p_++; return v; }
      for (;;) {
        ws();
        JValue k = string_();
        ws();
        if (p_ >= s_.size() || s_[p_] != ':') fail("expected ':'");
        p_++;
        v.obj.emplace_back(k.str, value());
        ws();
        if (p_ < s_.size() && s_[p_] == ',') { p_++; continue; }
        if (p_ < s_.size() && s_[p_] == '}') { p_++; return v; }
        fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      v.kind = JValue::Arr; p_++; ws();
      if (p_ < s_.size() && s_[p_] == ']') { p_++; return v; }
      for (;;) {
        v.arr.push_back(value());
        ws();
        if (p_ < s_.size() && s_[p_] == ',') { p_++; continue; }
        if (p_ < s_.size() && s_[p_] == ']') { p_++; return v; }
        fail("expected ',' or ']'");
      }
    }
    if (c == '"') return string_();
    if (s_.compare(p_, 4, "true") == 0) { p_ += 4; v.kind = JValue::Bool; v.b = true; return v; }
    if (s_.compare(p_, 5, "false") == 0) { p_ += 5; v.kind = JValue::Bool; v.b = false; return v; }
    if (s_.compare(p_, 4, "null") == 0) { p_ += 4; return v; }
    // number
    size_t b = p_;
    while (p_ < s_.size() && (std::string("+-0123456789.eE").find(s_[p_]) != std::string::npos)) p_++;
    if (b == p_) fail("unexpected character");
    v.kind = JValue::Num; v.str = s_.substr(b, p_ - b); v.num = std::strtod(v.str.c_str(), nullptr);
    return v;
  }
  JValue string_() {
    if (p_ >= s_.size() || s_[p_] != '"') fail("expected string");
    p_++;
    JValue v; v.kind = JValue::Str;
    while (p_ < s_.size() && s_[p_] != '"') {
      char c = s_[p_++];
      if (c == '\\' && p_ < s_.size()) {
        char e = s_[p_++];
        switch (e) {
          case 'n': v.str += '\n'; break;
          case 't': v.str += '\t'; break;
          case 'r': v.str += '\r'; break;
          case 'b': v.str += '\b'; break;
          case 'f': v.str += '\f'; break;
          case 'u': v.str += '?'; p_ += 4; break;   // descriptors are ASCII; non-ASCII names are not interpreted
          default: v.str += e;
        }
      } else {
        v.str += c;
      }
    }
    if (p_ >= s_.size()) fail("unterminated string");
    p_++;
    return v;
  }
};

inline JValue parse_json(const std::string& text) { return JParser(text).parse(); }

}  // namespace fortis
