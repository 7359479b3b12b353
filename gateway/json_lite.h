// Minimal JSON support for the gateway: find the raw text span of a top-level member of an object, replace or add
// members, and decode string / integer values.  It never builds a DOM; request bodies are forwarded almost verbatim.
#pragma once
#include <cctype>
#include <map>
#include <optional>
#include <string>
#include <string_view>
#include <utility>
#include <vector>

namespace jl {

inline size_t skip_ws(std::string_view s, size_t i) { while (i < s.size() && std::isspace((unsigned char)s[i])) i++; return i; }

// Returns the index one past the JSON value starting at i, or npos on malformed input.
inline size_t skip_value(std::string_view s, size_t i) {
  i = skip_ws(s, i);
  if (i >= s.size()) return std::string_view::npos;
  char c = s[i];
  if (c == '"') {
    for (i++; i < s.size(); i++) {
      if (s[i] == '\\') { i++; continue; }
      if (s[i] == '"') return i + 1;
    }
    return std::string_view::npos;
  }
  if (c == '{' || c == '[') {
    int depth = 0;
    for (; i < s.size(); i++) {
      char d = s[i];
      if (d == '"') { size_t e = skip_value(s, i); if (e == std::string_view::npos) return e; i = e - 1; continue; }
      if (d == '{' || d == '[') depth++;
      else if (d == '}' || d == ']') { if (--depth == 0) return i + 1; }
    }
    return std::string_view::npos;
  }
  size_t j = i;
  while (j < s.size() && s[j] != ',' && s[j] != '}' && s[j] != ']' && !std::isspace((unsigned char)s[j])) j++;
  return j == i ? std::string_view::npos : j;
}

struct Member { std::string key; size_t key_begin, value_begin, value_end; };

// Top-level members of the object in `s` (empty if `s` is not an object).
inline std::vector<Member> members(std::string_view s) {
  std::vector<Member> out;
  size_t i = skip_ws(s, 0);
  if (i >= s.size() || s[i] != '{') return out;
  i++;
  while (true) {
    i = skip_ws(s, i);
    if (i >= s.size() || s[i] == '}') break;
    if (s[i] != '"') return {};
    size_t kb = i, ke = skip_value(s, i);
    if (ke == std::string_view::npos) return {};
    i = skip_ws(s, ke);
    if (i >= s.size() || s[i] != ':') return {};
    size_t vb = skip_ws(s, i + 1), ve = skip_value(s, vb);
    if (ve == std::string_view::npos) return {};
    out.push_back({std::string(s.substr(kb + 1, ke - kb - 2)), kb, vb, ve});
    i = skip_ws(s, ve);
    if (i < s.size() && s[i] == ',') i++;
  }
  return out;
}

inline std::optional<std::string> raw(std::string_view s, const std::string& key) {
  for (auto& m : members(s)) if (m.key == key) return std::string(s.substr(m.value_begin, m.value_end - m.value_begin));
  return std::nullopt;
}

inline std::string unquote(std::string_view v) {
  std::string out;
  if (v.size() < 2 || v.front() != '"') return std::string(v);
  for (size_t i = 1; i + 1 < v.size(); i++) {
    if (v[i] == '\\' && i + 2 < v.size()) {
      char c = v[++i];
      out += c == 'n' ? '\n' : c == 't' ? '\t' : c == 'r' ? '\r' : c;
    } else out += v[i];
  }
  return out;
}

inline std::string quote(const std::string& s) {
  std::string o = "\"";
  for (char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += c; }
    else if (c == '\n') o += "\\n";
    else if (c == '\r') o += "\\r";
    else if (c == '\t') o += "\\t";
    else o += c;
  }
  return o + "\"";
}

// Copy of object `s` with `key` set to the raw JSON text `value` (replaced if present, appended otherwise).
inline std::string with_member(std::string_view s, const std::string& key, const std::string& value) {
  auto ms = members(s);
  for (auto& m : ms) {
    if (m.key == key) return std::string(s.substr(0, m.value_begin)) + value + std::string(s.substr(m.value_end));
  }
  size_t close = s.rfind('}');
  if (close == std::string_view::npos) return "{" + quote(key) + ":" + value + "}";
  std::string head(s.substr(0, close));
  return head + (ms.empty() ? "" : ",") + quote(key) + ":" + value + std::string(s.substr(close));
}

inline bool is_true(std::string_view s, const std::string& key) {
  auto v = raw(s, key);
  return v && *v == "true";
}

}  // namespace jl
