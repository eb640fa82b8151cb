// Minimal JSON reader/writer helpers for plan sidecars (host only, no dependencies).
#pragma once
#include <cctype>
#include <cstdlib>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace tmb {

class Json {
 public:
  enum Kind { kNull, kBool, kNumber, kString, kArray, kObject };
  Kind kind = kNull;
  bool boolean = false;
  double number = 0.0;
  std::string text;
  std::vector<Json> items;
  std::map<std::string, Json> fields;

  static Json Parse(const std::string& source) {
    size_t at = 0;
    Json value = ParseValue(source, at);
    SkipSpace(source, at);
    if (at != source.size()) throw std::invalid_argument("trailing characters after JSON value");
    return value;
  }

  bool has(const std::string& key) const { return kind == kObject && fields.count(key) != 0; }
  const Json& at(const std::string& key) const {
    auto found = fields.find(key);
    if (kind != kObject || found == fields.end()) throw std::invalid_argument("missing JSON field " + key);
    return found->second;
  }
  double num(const std::string& key, double fallback) const {
    return has(key) && at(key).kind == kNumber ? at(key).number : fallback;
  }
  long long integer(const std::string& key, long long fallback) const {
    return static_cast<long long>(num(key, static_cast<double>(fallback)));
  }
  bool flag(const std::string& key, bool fallback) const {
    if (!has(key)) return fallback;
    const Json& v = at(key);
    return v.kind == kBool ? v.boolean : (v.kind == kNumber ? v.number != 0.0 : fallback);
  }
  std::string str(const std::string& key, const std::string& fallback) const {
    return has(key) && at(key).kind == kString ? at(key).text : fallback;
  }

  static std::string Quote(const std::string& s) {
    std::string out = "\"";
    for (char ch : s) {
      if (ch == '"' || ch == '\\') out += '\\';
      out += ch;
    }
    return out + "\"";
  }

 private:
  static void SkipSpace(const std::string& s, size_t& at) {
    while (at < s.size() && std::isspace(static_cast<unsigned char>(s[at]))) ++at;
  }
  static Json ParseValue(const std::string& s, size_t& at) {
    SkipSpace(s, at);
    if (at >= s.size()) throw std::invalid_argument("unexpected end of JSON");
    Json value;
    const char ch = s[at];
    if (ch == '{') {
      value.kind = kObject;
      ++at;
      SkipSpace(s, at);
      if (at < s.size() && s[at] == '}') { ++at; return value; }
      for (;;) {
        SkipSpace(s, at);
        std::string key = ParseString(s, at);
        SkipSpace(s, at);
        if (at >= s.size() || s[at] != ':') throw std::invalid_argument("expected ':' in JSON object");
        ++at;
        value.fields[key] = ParseValue(s, at);
        SkipSpace(s, at);
        if (at < s.size() && s[at] == ',') { ++at; continue; }
        if (at < s.size() && s[at] == '}') { ++at; return value; }
        throw std::invalid_argument("expected ',' or '}' in JSON object");
      }
    }
    if (ch == '[') {
      value.kind = kArray;
      ++at;
      SkipSpace(s, at);
      if (at < s.size() && s[at] == ']') { ++at; return value; }
      for (;;) {
        value.items.push_back(ParseValue(s, at));
        SkipSpace(s, at);
        if (at < s.size() && s[at] == ',') { ++at; continue; }
        if (at < s.size() && s[at] == ']') { ++at; return value; }
        throw std::invalid_argument("expected ',' or ']' in JSON array");
      }
    }
    if (ch == '"') {
      value.kind = kString;
      value.text = ParseString(s, at);
      return value;
    }
    if (s.compare(at, 4, "true") == 0) { value.kind = kBool; value.boolean = true; at += 4; return value; }
    if (s.compare(at, 5, "false") == 0) { value.kind = kBool; at += 5; return value; }
    if (s.compare(at, 4, "null") == 0) { at += 4; return value; }
    char* end = nullptr;
    value.number = std::strtod(s.c_str() + at, &end);
    if (end == s.c_str() + at) throw std::invalid_argument("invalid JSON token");
    value.kind = kNumber;
    at = static_cast<size_t>(end - s.c_str());
    return value;
  }
  static std::string ParseString(const std::string& s, size_t& at) {
    if (at >= s.size() || s[at] != '"') throw std::invalid_argument("expected JSON string");
    ++at;
    std::string out;
    while (at < s.size() && s[at] != '"') {
      if (s[at] == '\\' && at + 1 < s.size()) {
        ++at;
        switch (s[at]) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': at += 4; out += '?'; break;  // plan sidecars are ASCII
          default: out += s[at];
        }
        ++at;
      } else {
        out += s[at++];
      }
    }
    if (at >= s.size()) throw std::invalid_argument("unterminated JSON string");
    ++at;
    return out;
  }
};

}  // namespace tmb
