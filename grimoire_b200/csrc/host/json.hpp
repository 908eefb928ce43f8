// Strict JSON parser + string escaping for the host runtime (tokenizer.json, config.json, request
// bodies).  Counterpart of the reference's own parser (include/b70/json.hpp: struct Json,
// json_escape); a recursive-descent parser into a small variant tree.
#pragma once
#include <cstdint>
#include <cstdlib>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace grm {

struct Json {
  enum Type { Null, Bool, Num, Str, Arr, Obj } type = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  const Json* get(const std::string& k) const {
    if (type != Obj) return nullptr;
    for (auto& kv : obj) if (kv.first == k) return &kv.second;
    return nullptr;
  }
  bool is(Type t) const { return type == t; }
};

struct JsonParser {
  const char* p;
  const char* e;
  std::string err;
  int depth = 0;

  explicit JsonParser(const std::string& s) : p(s.data()), e(s.data() + s.size()) {}
  JsonParser(const char* b, const char* en) : p(b), e(en) {}

  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool fail(const char* m) { if (err.empty()) err = m; return false; }

  static void put_utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out += (char)cp;
    else if (cp < 0x800) { out += (char)(0xC0 | (cp >> 6)); out += (char)(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { out += (char)(0xE0 | (cp >> 12)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
    else { out += (char)(0xF0 | (cp >> 18)); out += (char)(0x80 | ((cp >> 12) & 0x3F)); out += (char)(0x80 | ((cp >> 6) & 0x3F)); out += (char)(0x80 | (cp & 0x3F)); }
  }
  bool hex4(uint32_t& v) {
    if (e - p < 4) return false;
    v = 0;
    for (int i = 0; i < 4; ++i) {
      const char c = p[i];
      uint32_t d;
      if (c >= '0' && c <= '9') d = c - '0';
      else if (c >= 'a' && c <= 'f') d = c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') d = c - 'A' + 10;
      else return false;
      v = v * 16 + d;
    }
    p += 4;
    return true;
  }
  bool parse_string(std::string& out) {
    if (p >= e || *p != '"') return fail("expected string");
    ++p;
    while (p < e && *p != '"') {
      const unsigned char c = (unsigned char)*p;
      if (c < 0x20) return fail("control character in string");
      if (c == '\\') {
        ++p;
        if (p >= e) return fail("bad escape");
        switch (*p++) {
          case '"': out += '"'; break;
          case '\\': out += '\\'; break;
          case '/': out += '/'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'n': out += '\n'; break;
          case 'r': out += '\r'; break;
          case 't': out += '\t'; break;
          case 'u': {
            uint32_t cp;
            if (!hex4(cp)) return fail("bad \\u escape");
            if (cp >= 0xD800 && cp <= 0xDBFF) {
              uint32_t lo;
              if (e - p < 6 || p[0] != '\\' || p[1] != 'u') return fail("lone surrogate");
              p += 2;
              if (!hex4(lo) || lo < 0xDC00 || lo > 0xDFFF) return fail("bad surrogate pair");
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            } else if (cp >= 0xDC00 && cp <= 0xDFFF) {
              return fail("lone surrogate");
            }
            put_utf8(out, cp);
            break;
          }
          default: return fail("bad escape");
        }
      } else {
        out += *p++;
      }
    }
    if (p >= e) return fail("unterminated string");
    ++p;
    return true;
  }
  bool parse(Json& j) {
    if (++depth > 256) return fail("nesting too deep");
    ws();
    if (p >= e) return fail("unexpected end");
    bool ok = true;
    const char c = *p;
    if (c == '{') {
      j.type = Json::Obj;
      ++p; ws();
      if (p < e && *p == '}') { ++p; }
      else {
        for (;;) {
          ws();
          std::string k;
          if (!parse_string(k)) { ok = false; break; }
          ws();
          if (p >= e || *p != ':') { ok = fail("expected ':'"); break; }
          ++p;
          j.obj.emplace_back(std::move(k), Json());
          if (!parse(j.obj.back().second)) { ok = false; break; }
          ws();
          if (p < e && *p == ',') { ++p; continue; }
          if (p < e && *p == '}') { ++p; break; }
          ok = fail("expected ',' or '}'");
          break;
        }
      }
    } else if (c == '[') {
      j.type = Json::Arr;
      ++p; ws();
      if (p < e && *p == ']') { ++p; }
      else {
        for (;;) {
          j.arr.emplace_back();
          if (!parse(j.arr.back())) { ok = false; break; }
          ws();
          if (p < e && *p == ',') { ++p; continue; }
          if (p < e && *p == ']') { ++p; break; }
          ok = fail("expected ',' or ']'");
          break;
        }
      }
    } else if (c == '"') {
      j.type = Json::Str;
      ok = parse_string(j.str);
    } else if (c == 't' && e - p >= 4 && std::string(p, 4) == "true") { j.type = Json::Bool; j.b = true; p += 4; }
    else if (c == 'f' && e - p >= 5 && std::string(p, 5) == "false") { j.type = Json::Bool; j.b = false; p += 5; }
    else if (c == 'n' && e - p >= 4 && std::string(p, 4) == "null") { j.type = Json::Null; p += 4; }
    else if (c == '-' || (c >= '0' && c <= '9')) {
      const char* s = p;
      if (*p == '-') ++p;
      if (p >= e) return fail("bad number");
      if (*p == '0') ++p;
      else if (*p >= '1' && *p <= '9') { while (p < e && *p >= '0' && *p <= '9') ++p; }
      else return fail("bad number");
      if (p < e && *p == '.') { ++p; if (p >= e || *p < '0' || *p > '9') return fail("bad number"); while (p < e && *p >= '0' && *p <= '9') ++p; }
      if (p < e && (*p == 'e' || *p == 'E')) { ++p; if (p < e && (*p == '+' || *p == '-')) ++p; if (p >= e || *p < '0' || *p > '9') return fail("bad number"); while (p < e && *p >= '0' && *p <= '9') ++p; }
      j.type = Json::Num;
      j.num = std::strtod(std::string(s, p).c_str(), nullptr);
    } else {
      ok = fail("unexpected character");
    }
    --depth;
    return ok;
  }
  bool parse_document(Json& j) {
    if (!parse(j)) return false;
    ws();
    if (p != e) return fail("trailing characters");
    return true;
  }
};

inline std::string json_escape(const std::string& s) {
  std::string o;
  o.reserve(s.size() + 8);
  static const char* hex = "0123456789abcdef";
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      case '\b': o += "\\b"; break;
      case '\f': o += "\\f"; break;
      default:
        if (c < 0x20) { o += "\\u00"; o += hex[c >> 4]; o += hex[c & 15]; }
        else o += (char)c;
    }
  }
  return o;
}

}  // namespace grm
