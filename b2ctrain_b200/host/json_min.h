// A small JSON reader for the files the host front end takes (cameras.json): objects, arrays, numbers, strings, true /
// false / null; no comments, UTF-8 passed through, \uXXXX escapes kept only for the Basic Latin range. Values are
// held in one tagged struct; lookups throw std::runtime_error with the missing key, like the rest of the host.
#pragma once
#include <cstdlib>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace b2c {

struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool b = false;
  double num = 0.0;
  std::string str;
  std::vector<Json> items;
  std::map<std::string, Json> fields;

  const Json& at(const std::string& key) const {
    auto it = fields.find(key);
    if (kind != Object || it == fields.end()) throw std::runtime_error("json: missing key '" + key + "'");
    return it->second;
  }
  bool has(const std::string& key) const { return kind == Object && fields.count(key) > 0; }
  const Json& operator[](size_t i) const {
    if (kind != Array || i >= items.size()) throw std::runtime_error("json: index out of range");
    return items[i];
  }
  double number() const { if (kind != Number) throw std::runtime_error("json: not a number"); return num; }
  const std::string& string() const { if (kind != String) throw std::runtime_error("json: not a string"); return str; }

  static Json parse(const std::string& text) {
    size_t at = 0;
    Json v = value(text, at);
    skip(text, at);
    if (at != text.size()) throw std::runtime_error("json: trailing characters at offset " + std::to_string(at));
    return v;
  }

 private:
  static void skip(const std::string& t, size_t& at) { while (at < t.size() && (t[at] == ' ' || t[at] == '\n' || t[at] == '\t' || t[at] == '\r')) at++; }
  [[noreturn]] static void bad(size_t at, const char* what) { throw std::runtime_error(std::string("json: ") + what + " at offset " + std::to_string(at)); }
  static std::string quoted(const std::string& t, size_t& at) {
    std::string out;
    at++;   // opening quote
    while (at < t.size() && t[at] != '"') {
      char ch = t[at++];
      if (ch == '\\') {
        if (at >= t.size()) bad(at, "unterminated escape");
        const char e = t[at++];
        switch (e) {
          case 'n': ch = '\n'; break; case 't': ch = '\t'; break; case 'r': ch = '\r'; break; case 'b': ch = '\b'; break; case 'f': ch = '\f'; break;
          case 'u': {
            if (at + 4 > t.size()) bad(at, "short \\u escape");
            const long code = std::strtol(t.substr(at, 4).c_str(), nullptr, 16);
            at += 4;
            ch = code < 128 ? (char)code : '?';
            break;
          }
          default: ch = e;   // quote, backslash, slash
        }
      }
      out.push_back(ch);
    }
    if (at >= t.size()) bad(at, "unterminated string");
    at++;   // closing quote
    return out;
  }
  static Json value(const std::string& t, size_t& at) {
    skip(t, at);
    if (at >= t.size()) bad(at, "unexpected end");
    Json v;
    const char ch = t[at];
    if (ch == '{') {
      v.kind = Object; at++;
      skip(t, at);
      if (at < t.size() && t[at] == '}') { at++; return v; }
      for (;;) {
        skip(t, at);
        if (at >= t.size() || t[at] != '"') bad(at, "expected a key");
        std::string key = quoted(t, at);
        skip(t, at);
        if (at >= t.size() || t[at] != ':') bad(at, "expected ':'");
        at++;
        v.fields[key] = value(t, at);
        skip(t, at);
        if (at < t.size() && t[at] == ',') { at++; continue; }
        if (at < t.size() && t[at] == '}') { at++; return v; }
        bad(at, "expected ',' or '}'");
      }
    }
    if (ch == '[') {
      v.kind = Array; at++;
      skip(t, at);
      if (at < t.size() && t[at] == ']') { at++; return v; }
      for (;;) {
        v.items.push_back(value(t, at));
        skip(t, at);
        if (at < t.size() && t[at] == ',') { at++; continue; }
        if (at < t.size() && t[at] == ']') { at++; return v; }
        bad(at, "expected ',' or ']'");
      }
    }
    if (ch == '"') { v.kind = String; v.str = quoted(t, at); return v; }
    if (t.compare(at, 4, "true") == 0) { v.kind = Bool; v.b = true; at += 4; return v; }
    if (t.compare(at, 5, "false") == 0) { v.kind = Bool; at += 5; return v; }
    if (t.compare(at, 4, "null") == 0) { at += 4; return v; }
    char* end = nullptr;
    v.num = std::strtod(t.c_str() + at, &end);
    if (end == t.c_str() + at) bad(at, "unexpected character");
    v.kind = Number;
    at = (size_t)(end - t.c_str());
    return v;
  }
};

}  // namespace b2c
