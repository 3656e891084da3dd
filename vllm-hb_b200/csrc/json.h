// Minimal JSON reader: enough for HuggingFace config.json and safetensors headers.
#pragma once

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace hb {

struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;  // insertion order kept

  const Json* get(const std::string& key) const {
    if (kind != Obj) return nullptr;
    for (auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
  double number_or(const std::string& key, double dflt) const {
    const Json* j = get(key);
    return (j && j->kind == Num) ? j->num : dflt;
  }
  std::string string_or(const std::string& key, const std::string& dflt) const {
    const Json* j = get(key);
    return (j && j->kind == Str) ? j->str : dflt;
  }
};

class JsonParser {
 public:
  JsonParser(const char* s, size_t n) : p_(s), end_(s + n) {}
  bool parse(Json* out, std::string* err) {
    skip();
    if (!value(out)) { *err = err_; return false; }
    skip();
    if (p_ != end_) { *err = "trailing characters after JSON value"; return false; }
    return true;
  }

 private:
  const char* p_;
  const char* end_;
  std::string err_;

  void skip() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
  bool fail(const char* m) { err_ = m; return false; }
  bool lit(const char* w) {
    size_t n = strlen(w);
    if ((size_t)(end_ - p_) < n || strncmp(p_, w, n) != 0) return false;
    p_ += n;
    return true;
  }
  bool string(std::string* out) {
    if (p_ >= end_ || *p_ != '"') return fail("expected string");
    ++p_;
    out->clear();
    while (p_ < end_ && *p_ != '"') {
      if (*p_ == '\\') {
        if (++p_ >= end_) return fail("bad escape");
        switch (*p_) {
          case 'n': out->push_back('\n'); break;
          case 't': out->push_back('\t'); break;
          case 'r': out->push_back('\r'); break;
          case 'b': out->push_back('\b'); break;
          case 'f': out->push_back('\f'); break;
          case 'u': {
            if (end_ - p_ < 5) return fail("bad \\u escape");
            unsigned cp = (unsigned)strtoul(std::string(p_ + 1, 4).c_str(), nullptr, 16);
            p_ += 4;
            if (cp < 0x80) out->push_back((char)cp);
            else if (cp < 0x800) { out->push_back((char)(0xC0 | (cp >> 6))); out->push_back((char)(0x80 | (cp & 0x3F))); }
            else { out->push_back((char)(0xE0 | (cp >> 12))); out->push_back((char)(0x80 | ((cp >> 6) & 0x3F))); out->push_back((char)(0x80 | (cp & 0x3F))); }
            break;
          }
          default: out->push_back(*p_);
        }
        ++p_;
      } else {
        out->push_back(*p_++);
      }
    }
    if (p_ >= end_) return fail("unterminated string");
    ++p_;
    return true;
  }
  bool value(Json* out) {
    skip();
    if (p_ >= end_) return fail("unexpected end of input");
    const char c = *p_;
    if (c == '{') {
      ++p_;
      out->kind = Json::Obj;
      skip();
      if (p_ < end_ && *p_ == '}') { ++p_; return true; }
      for (;;) {
        skip();
        std::string key;
        if (!string(&key)) return false;
        skip();
        if (p_ >= end_ || *p_ != ':') return fail("expected ':'");
        ++p_;
        Json v;
        if (!value(&v)) return false;
        out->obj.emplace_back(std::move(key), std::move(v));
        skip();
        if (p_ < end_ && *p_ == ',') { ++p_; continue; }
        if (p_ < end_ && *p_ == '}') { ++p_; return true; }
        return fail("expected ',' or '}'");
      }
    }
    if (c == '[') {
      ++p_;
      out->kind = Json::Arr;
      skip();
      if (p_ < end_ && *p_ == ']') { ++p_; return true; }
      for (;;) {
        Json v;
        if (!value(&v)) return false;
        out->arr.push_back(std::move(v));
        skip();
        if (p_ < end_ && *p_ == ',') { ++p_; continue; }
        if (p_ < end_ && *p_ == ']') { ++p_; return true; }
        return fail("expected ',' or ']'");
      }
    }
    if (c == '"') { out->kind = Json::Str; return string(&out->str); }
    if (lit("true")) { out->kind = Json::Bool; out->b = true; return true; }
    if (lit("false")) { out->kind = Json::Bool; out->b = false; return true; }
    if (lit("null")) { out->kind = Json::Null; return true; }
    char* e = nullptr;
    std::string tmp(p_, (size_t)std::min<ptrdiff_t>(end_ - p_, 64));
    double d = strtod(tmp.c_str(), &e);
    if (e == tmp.c_str()) return fail("unexpected character");
    p_ += (e - tmp.c_str());
    out->kind = Json::Num;
    out->num = d;
    return true;
  }
};

}  // namespace hb
