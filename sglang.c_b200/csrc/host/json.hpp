// A small JSON reader for config.json, the safetensors header and the shard index: objects keep
// their keys in file order, numbers keep whether they were written as integers.  The reference
// has a reader of its own for the same files (src/json.c; used at src/gpt2.c:37-42 and
// src/safetensors.c:676-843).
#pragma once
#include <cstdlib>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

namespace sglc {

struct Json {
  enum Kind { Null, Bool, Int, Real, Str, Arr, Obj } kind = Null;
  bool b = false;
  long long i = 0;
  double d = 0.0;
  std::string s;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  const Json* get(const std::string& key) const {
    if (kind != Obj) return nullptr;
    for (const auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  bool is_number() const { return kind == Int || kind == Real; }
  double number() const { return kind == Int ? (double)i : d; }
};

class JsonParser {
 public:
  JsonParser(const char* p, size_t n) : p_(p), end_(p + n) {}
  // false with `err` set (what was expected, and the byte offset) on malformed input
  bool parse(Json* out, std::string* err) {
    begin_ = p_;
    if (!value(out, 0)) {
      *err = err_ + " at byte " + std::to_string((long long)(p_ - begin_));
      return false;
    }
    ws();
    if (p_ != end_) {
      *err = "text after the JSON value at byte " + std::to_string((long long)(p_ - begin_));
      return false;
    }
    return true;
  }

 private:
  const char *p_, *end_, *begin_ = nullptr;
  std::string err_;
  void ws() {
    while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_;
  }
  bool fail(const char* what) {
    if (err_.empty()) err_ = what;
    return false;
  }
  bool lit(const char* w) {
    const size_t n = strlen(w);
    if ((size_t)(end_ - p_) < n || memcmp(p_, w, n) != 0) return fail("unknown literal");
    p_ += n;
    return true;
  }
  static void utf8(unsigned cp, std::string* s) {
    if (cp < 0x80) s->push_back((char)cp);
    else if (cp < 0x800) { s->push_back((char)(0xC0 | (cp >> 6))); s->push_back((char)(0x80 | (cp & 63))); }
    else if (cp < 0x10000) {
      s->push_back((char)(0xE0 | (cp >> 12))); s->push_back((char)(0x80 | ((cp >> 6) & 63)));
      s->push_back((char)(0x80 | (cp & 63)));
    } else {
      s->push_back((char)(0xF0 | (cp >> 18))); s->push_back((char)(0x80 | ((cp >> 12) & 63)));
      s->push_back((char)(0x80 | ((cp >> 6) & 63))); s->push_back((char)(0x80 | (cp & 63)));
    }
  }
  bool hex4(unsigned* v) {
    if (end_ - p_ < 4) return fail("short \\u escape");
    unsigned x = 0;
    for (int k = 0; k < 4; ++k) {
      const char c = *p_++;
      x <<= 4;
      if (c >= '0' && c <= '9') x |= c - '0';
      else if (c >= 'a' && c <= 'f') x |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') x |= c - 'A' + 10;
      else return fail("bad \\u escape");
    }
    *v = x;
    return true;
  }
  bool string(std::string* s) {
    if (p_ >= end_ || *p_ != '"') return fail("expected a string");
    ++p_;
    while (p_ < end_ && *p_ != '"') {
      char c = *p_++;
      if (c != '\\') { s->push_back(c); continue; }
      if (p_ >= end_) return fail("unterminated escape");
      c = *p_++;
      switch (c) {
        case 'n': s->push_back('\n'); break;
        case 't': s->push_back('\t'); break;
        case 'r': s->push_back('\r'); break;
        case 'b': s->push_back('\b'); break;
        case 'f': s->push_back('\f'); break;
        case 'u': {
          unsigned cp;
          if (!hex4(&cp)) return false;
          if (cp >= 0xD800 && cp < 0xDC00 && end_ - p_ >= 6 && p_[0] == '\\' && p_[1] == 'u') {
            p_ += 2;
            unsigned lo;
            if (!hex4(&lo)) return false;
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          utf8(cp, s);
          break;
        }
        default: s->push_back(c);      // \" \\ \/
      }
    }
    if (p_ >= end_) return fail("unterminated string");
    ++p_;
    return true;
  }
  bool value(Json* out, int depth) {
    if (depth > 64) return fail("nested too deep");
    ws();
    if (p_ >= end_) return fail("unexpected end");
    const char c = *p_;
    if (c == '{') {
      ++p_;
      out->kind = Json::Obj;
      ws();
      if (p_ < end_ && *p_ == '}') { ++p_; return true; }
      for (;;) {
        ws();
        std::string key;
        if (!string(&key)) return false;
        ws();
        if (p_ >= end_ || *p_ != ':') return fail("expected ':'");
        ++p_;
        out->obj.emplace_back(std::move(key), Json());
        if (!value(&out->obj.back().second, depth + 1)) return false;
        ws();
        if (p_ < end_ && *p_ == ',') { ++p_; continue; }
        if (p_ < end_ && *p_ == '}') { ++p_; return true; }
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      ++p_;
      out->kind = Json::Arr;
      ws();
      if (p_ < end_ && *p_ == ']') { ++p_; return true; }
      for (;;) {
        out->arr.emplace_back();
        if (!value(&out->arr.back(), depth + 1)) return false;
        ws();
        if (p_ < end_ && *p_ == ',') { ++p_; continue; }
        if (p_ < end_ && *p_ == ']') { ++p_; return true; }
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') { out->kind = Json::Str; return string(&out->s); }
    if (c == 't') { out->kind = Json::Bool; out->b = true; return lit("true"); }
    if (c == 'f') { out->kind = Json::Bool; out->b = false; return lit("false"); }
    if (c == 'n') { out->kind = Json::Null; return lit("null"); }
    // a number: an integer if it has no fraction or exponent and fits 64 bits
    const char* q = p_;
    if (q < end_ && (*q == '-' || *q == '+')) ++q;
    bool digits = false, real = false;
    while (q < end_ && ((*q >= '0' && *q <= '9') || *q == '.' || *q == 'e' || *q == 'E' || *q == '-' || *q == '+')) {
      if (*q >= '0' && *q <= '9') digits = true;
      else real = true;
      ++q;
    }
    if (!digits) return fail("expected a value");
    const std::string text(p_, q);
    p_ = q;
    if (!real && text.size() <= 18) {
      out->kind = Json::Int;
      out->i = strtoll(text.c_str(), nullptr, 10);
    } else {
      out->kind = Json::Real;
      out->d = strtod(text.c_str(), nullptr);
    }
    return true;
  }
};

inline bool json_parse(const std::string& text, Json* out, std::string* err) {
  JsonParser p(text.data(), text.size());
  return p.parse(out, err);
}

}  // namespace sglc
