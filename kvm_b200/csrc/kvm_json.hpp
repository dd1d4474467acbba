// A small JSON reader for bundle metadata (metadata.json, golden.json): objects, arrays, strings, numbers, booleans, null.
// Numbers keep their text as well as their double value, so 64-bit seeds survive (a double holds 53 bits).
// Malformed input throws std::runtime_error with the byte offset; nesting is limited so hostile files cannot exhaust the stack.
// Used by the bundle loader inside the library and by the kvm_exec command-line tool (host code only).
#pragma once
#include <cmath>
#include <cstdlib>
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

struct KvmJson {
  enum Type { Null, Bool, Num, Str, Arr, Obj } type = Null;
  bool b = false;
  double n = 0.0;
  std::string s;                                   // string value, or the literal text of a number
  std::vector<KvmJson> a;
  std::vector<std::pair<std::string, KvmJson>> o;  // members in file order

  const KvmJson* get(const std::string& key) const {
    if (type != Obj) return nullptr;
    for (auto& kv : o) if (kv.first == key) return &kv.second;
    return nullptr;
  }
  const KvmJson& need(const std::string& key) const {
    const KvmJson* v = get(key);
    if (!v) throw std::runtime_error("missing key '" + key + "'");
    return *v;
  }
  double num(const std::string& key, double dflt) const {
    const KvmJson* v = get(key);
    return v && v->type == Num ? v->n : dflt;
  }
  long long integer(const std::string& key, long long dflt) const {
    const KvmJson* v = get(key);
    if (!v || v->type != Num) return dflt;
    if (v->s.find_first_of(".eE") == std::string::npos) return strtoll(v->s.c_str(), nullptr, 10);
    return (long long)v->n;
  }
  unsigned long long u64(const std::string& key, unsigned long long dflt) const {
    const KvmJson* v = get(key);
    if (!v) return dflt;
    if (v->type == Str || (v->type == Num && v->s.find_first_of(".eE-") == std::string::npos)) return strtoull(v->s.c_str(), nullptr, 10);
    return v->type == Num ? (unsigned long long)v->n : dflt;
  }
  std::string str(const std::string& key, const std::string& dflt = "") const {
    const KvmJson* v = get(key);
    return v && v->type == Str ? v->s : dflt;
  }
};

class KvmJsonParser {
 public:
  explicit KvmJsonParser(const std::string& text) : t_(text) {}
  KvmJson parse() {
    KvmJson v = value(0);
    ws();
    if (p_ != t_.size()) fail("trailing characters");
    return v;
  }

 private:
  const std::string& t_;
  size_t p_ = 0;
  [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("JSON: ") + what + " at byte " + std::to_string(p_)); }
  void ws() { while (p_ < t_.size() && (t_[p_] == ' ' || t_[p_] == '\n' || t_[p_] == '\t' || t_[p_] == '\r')) ++p_; }
  bool lit(const char* w) {
    size_t n = 0;
    while (w[n]) ++n;
    if (t_.compare(p_, n, w) != 0) return false;
    p_ += n;
    return true;
  }
  std::string string_() {
    std::string out;
    ++p_;                                          // opening quote
    while (true) {
      if (p_ >= t_.size()) fail("unterminated string");
      const char c = t_[p_++];
      if (c == '"') return out;
      if ((unsigned char)c < 0x20) fail("control character in string");
      if (c != '\\') { out += c; continue; }
      if (p_ >= t_.size()) fail("unterminated escape");
      const char e = t_[p_++];
      switch (e) {
        case '"': out += '"'; break; case '\\': out += '\\'; break; case '/': out += '/'; break;
        case 'b': out += '\b'; break; case 'f': out += '\f'; break; case 'n': out += '\n'; break; case 'r': out += '\r'; break; case 't': out += '\t'; break;
        case 'u': {
          if (p_ + 4 > t_.size()) fail("short \\u escape");
          unsigned cp = 0;
          for (int i = 0; i < 4; ++i) {
            const char h = t_[p_++];
            cp = cp * 16 + (h >= '0' && h <= '9' ? h - '0' : h >= 'a' && h <= 'f' ? h - 'a' + 10 : h >= 'A' && h <= 'F' ? h - 'A' + 10 : (fail("bad \\u escape"), 0));
          }
          if (cp < 0x80) out += (char)cp;
          else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
          else { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
          break;
        }
        default: fail("bad escape");
      }
    }
  }
  KvmJson value(int depth) {
    if (depth > 64) fail("nesting too deep");
    ws();
    if (p_ >= t_.size()) fail("unexpected end");
    KvmJson v;
    const char c = t_[p_];
    if (c == '{') {
      v.type = KvmJson::Obj;
      ++p_; ws();
      if (p_ < t_.size() && t_[p_] == '}') { ++p_; return v; }
      while (true) {
        ws();
        if (p_ >= t_.size() || t_[p_] != '"') fail("object key expected");
        std::string k = string_();
        ws();
        if (p_ >= t_.size() || t_[p_] != ':') fail("':' expected");
        ++p_;
        v.o.emplace_back(std::move(k), value(depth + 1));
        ws();
        if (p_ < t_.size() && t_[p_] == ',') { ++p_; continue; }
        if (p_ < t_.size() && t_[p_] == '}') { ++p_; return v; }
        fail("',' or '}' expected");
      }
    }
    if (c == '[') {
      v.type = KvmJson::Arr;
      ++p_; ws();
      if (p_ < t_.size() && t_[p_] == ']') { ++p_; return v; }
      while (true) {
        v.a.push_back(value(depth + 1));
        ws();
        if (p_ < t_.size() && t_[p_] == ',') { ++p_; continue; }
        if (p_ < t_.size() && t_[p_] == ']') { ++p_; return v; }
        fail("',' or ']' expected");
      }
    }
    if (c == '"') { v.type = KvmJson::Str; v.s = string_(); return v; }
    if (lit("true")) { v.type = KvmJson::Bool; v.b = true; return v; }
    if (lit("false")) { v.type = KvmJson::Bool; return v; }
    if (lit("null")) return v;
    if (lit("NaN")) { v.type = KvmJson::Num; v.n = NAN; v.s = "NaN"; return v; }                 // Python's json module writes these
    if (lit("Infinity")) { v.type = KvmJson::Num; v.n = INFINITY; v.s = "Infinity"; return v; }
    if (lit("-Infinity")) { v.type = KvmJson::Num; v.n = -INFINITY; v.s = "-Infinity"; return v; }
    const size_t start = p_;
    if (p_ < t_.size() && (t_[p_] == '-' || t_[p_] == '+')) ++p_;
    while (p_ < t_.size() && ((t_[p_] >= '0' && t_[p_] <= '9') || t_[p_] == '.' || t_[p_] == 'e' || t_[p_] == 'E' || t_[p_] == '-' || t_[p_] == '+')) ++p_;
    if (p_ == start) fail("value expected");
    v.type = KvmJson::Num;
    v.s = t_.substr(start, p_ - start);
    char* end = nullptr;
    v.n = strtod(v.s.c_str(), &end);
    if (!end || *end) { p_ = start; fail("bad number"); }
    return v;
  }
};
