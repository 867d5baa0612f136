// A small JSON reader: enough for config.json and the header of a safetensors file (objects, arrays,
// strings with the usual escapes, numbers, true / false / null).  The reference reads its model
// metadata from GGUF key-value pairs (runtime/src/model_config.cpp:74-95); a model folder here
// carries the same facts as JSON.
#pragma once
#include <cmath>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace qv {

struct JsonError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;      // in file order

  bool is_null() const { return kind == Null; }
  const Json* find(const std::string& key) const {
    if (kind != Object) return nullptr;
    for (const auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  bool has(const std::string& key) const {
    const Json* j = find(key);
    return j && !j->is_null();
  }
  const Json& at(const std::string& key) const {
    const Json* j = find(key);
    if (!j) throw JsonError("missing key '" + key + "'");
    return *j;
  }
  double number() const {
    if (kind != Number) throw JsonError("not a number");
    return num;
  }
  long long integer() const {
    if (kind != Number || std::floor(num) != num) throw JsonError("not an integer");
    return (long long)num;
  }
  const std::string& string() const {
    if (kind != String) throw JsonError("not a string");
    return str;
  }
  bool boolean() const {
    if (kind != Bool) throw JsonError("not true or false");
    return b;
  }
};

class JsonParser {
 public:
  JsonParser(const char* p, size_t n) : p_(p), end_(p + n) {}
  Json parse() {
    Json v = value();
    ws();
    if (p_ != end_) fail("text after the value");
    return v;
  }

 private:
  const char* p_;
  const char* end_;
  [[noreturn]] void fail(const std::string& what) const { throw JsonError("JSON: " + what); }
  void ws() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }
  bool eat(char c) {
    ws();
    if (p_ < end_ && *p_ == c) { ++p_; return true; }
    return false;
  }
  void word(const char* w) {
    for (; *w; ++w, ++p_)
      if (p_ >= end_ || *p_ != *w) fail("unknown word");
  }
  Json value() {
    ws();
    if (p_ >= end_) fail("ends early");
    Json v;
    const char c = *p_;
    if (c == '{') {
      ++p_;
      v.kind = Json::Object;
      if (eat('}')) return v;
      do {
        ws();
        if (p_ >= end_ || *p_ != '"') fail("an object key must be a string");
        std::string k = text();
        if (!eat(':')) fail("':' expected");
        v.obj.emplace_back(std::move(k), value());
      } while (eat(','));
      if (!eat('}')) fail("'}' expected");
    } else if (c == '[') {
      ++p_;
      v.kind = Json::Array;
      if (eat(']')) return v;
      do v.arr.push_back(value());
      while (eat(','));
      if (!eat(']')) fail("']' expected");
    } else if (c == '"') {
      v.kind = Json::String;
      v.str = text();
    } else if (c == 't') { word("true"); v.kind = Json::Bool; v.b = true;
    } else if (c == 'f') { word("false"); v.kind = Json::Bool; v.b = false;
    } else if (c == 'n') { word("null");
    } else if (c == 'N') { word("NaN"); v.kind = Json::Number; v.num = NAN;      // written by some exporters
    } else if (c == 'I') { word("Infinity"); v.kind = Json::Number; v.num = INFINITY;
    } else {
      char* e = nullptr;
      std::string tmp(p_, (size_t)std::min<ptrdiff_t>(end_ - p_, 64));
      v.num = std::strtod(tmp.c_str(), &e);
      if (e == tmp.c_str()) fail("a value was expected");
      p_ += e - tmp.c_str();
      v.kind = Json::Number;
    }
    return v;
  }
  static void utf8(std::string& out, unsigned cp) {
    if (cp < 0x80) out += (char)cp;
    else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
  }
  unsigned hex4() {
    if (end_ - p_ < 4) fail("short \\u escape");
    unsigned v = 0;
    for (int i = 0; i < 4; ++i, ++p_) {
      const char c = *p_;
      v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : (fail("bad \\u escape"), 0));
    }
    return v;
  }
  std::string text() {
    ++p_;                                             // the opening quote
    std::string out;
    while (true) {
      if (p_ >= end_) fail("a string does not end");
      const char c = *p_++;
      if (c == '"') break;
      if (c != '\\') { out += c; continue; }
      if (p_ >= end_) fail("a string does not end");
      const char e = *p_++;
      switch (e) {
        case 'n': out += '\n'; break;
        case 't': out += '\t'; break;
        case 'r': out += '\r'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'u': {
          unsigned cp = hex4();
          if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
            p_ += 2;
            cp = 0x10000 + ((cp - 0xD800) << 10) + (hex4() - 0xDC00);
          }
          utf8(out, cp);
          break;
        }
        default: out += e;                            // \" \\ \/
      }
    }
    return out;
  }
};

inline Json parse_json(const std::string& text) { return JsonParser(text.data(), text.size()).parse(); }

}  // namespace qv
