// Byte-level BPE tokenizer over a HF tokenizer.json: Qwen2 / GPT-2 style pre-tokenisation written
// as a scanner (no regex engine), byte <-> unicode mapping, rank-ordered merges, added / special
// tokens split out before pre-tokenisation, decode back to bytes.
// Reference: Tokenizer::{load,encode,decode,special_id} (src/tokenizer.cpp:168-1860,
// include/b70/tokenizer.hpp); chat templates live in grimoire_b200/tokenizer.py.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "json.hpp"
#include "unicode_tables.hpp"

namespace {

using grm::Json;

bool in_ranges(const uint32_t (*tbl)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    const int mid = (lo + hi) >> 1;
    if (cp < tbl[mid][0]) hi = mid - 1;
    else if (cp > tbl[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}
bool is_L(uint32_t c) {
  if (c < 0x80) return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z');
  return in_ranges(grm::kUnicodeL, grm::kUnicodeL_count, c);
}
bool is_N(uint32_t c) {
  if (c < 0x80) return c >= '0' && c <= '9';
  return in_ranges(grm::kUnicodeN, grm::kUnicodeN_count, c);
}
bool is_S(uint32_t c) {   // White_Space
  return (c >= 9 && c <= 13) || c == 32 || c == 0x85 || c == 0xA0 || c == 0x1680 || (c >= 0x2000 && c <= 0x200A) || c == 0x2028 ||
         c == 0x2029 || c == 0x202F || c == 0x205F || c == 0x3000;
}
bool is_nl(uint32_t c) { return c == '\r' || c == '\n'; }

void decode_utf8(const char* s, int n, std::vector<uint32_t>& cps, std::vector<int>& offs) {
  int i = 0;
  while (i < n) {
    const unsigned char c = (unsigned char)s[i];
    uint32_t cp;
    int len;
    if (c < 0x80) { cp = c; len = 1; }
    else if ((c >> 5) == 6 && i + 1 < n) { cp = ((c & 31) << 6) | (s[i + 1] & 63); len = 2; }
    else if ((c >> 4) == 14 && i + 2 < n) { cp = ((c & 15) << 12) | ((s[i + 1] & 63) << 6) | (s[i + 2] & 63); len = 3; }
    else if ((c >> 3) == 30 && i + 3 < n) { cp = ((c & 7) << 18) | ((s[i + 1] & 63) << 12) | ((s[i + 2] & 63) << 6) | (s[i + 3] & 63); len = 4; }
    else { cp = 0xFFFD; len = 1; }   // invalid byte: its own piece, bytes preserved by offsets
    cps.push_back(cp);
    offs.push_back(i);
    i += len;
  }
  offs.push_back(n);
}

struct PairHash {
  size_t operator()(const std::pair<int, int>& p) const { return ((size_t)(uint32_t)p.first << 32) ^ (uint32_t)p.second; }
};

struct Tok {
  std::unordered_map<std::string, int> vocab;
  std::vector<std::string> id_to_tok;
  std::unordered_map<std::pair<int, int>, int, PairHash> merges;   // (left id, right id) -> rank
  std::unordered_map<std::pair<int, int>, int, PairHash> merged;   // (left id, right id) -> merged id
  std::vector<std::pair<std::string, int>> added;                  // content -> id, longest first
  std::vector<char> added_special;                                 // indexed like `added`
  std::unordered_map<int, int> special_ids;                        // id -> 1
  std::string byte_sym[256];                                       // byte -> utf8 of its mapped code point
  std::unordered_map<uint32_t, int> sym_byte;                      // mapped code point -> byte
  int byte_id[256];
  std::unordered_map<std::string, std::vector<int>> cache;
  bool ignore_merges = false;
};

void build_byte_map(Tok& t) {
  std::vector<int> bs;
  for (int b = 33; b <= 126; ++b) bs.push_back(b);
  for (int b = 161; b <= 172; ++b) bs.push_back(b);
  for (int b = 174; b <= 255; ++b) bs.push_back(b);
  std::vector<int> cs(bs.begin(), bs.end());
  int n = 0;
  for (int b = 0; b < 256; ++b)
    if (std::find(bs.begin(), bs.end(), b) == bs.end()) { bs.push_back(b); cs.push_back(256 + n++); }
  for (size_t i = 0; i < bs.size(); ++i) {
    std::string u;
    grm::JsonParser::put_utf8(u, (uint32_t)cs[i]);
    t.byte_sym[bs[i]] = u;
    t.sym_byte[(uint32_t)cs[i]] = bs[i];
  }
}

// one pre-token [i, j) in code points, following the alternatives of the Qwen2 pattern in order
int next_piece(const std::vector<uint32_t>& c, int i) {
  const int n = (int)c.size();
  const uint32_t a = c[i];
  // 1. contractions, case-insensitive
  if (a == '\'' && i + 1 < n) {
    const uint32_t b = c[i + 1] | 32;
    if (b == 's' || b == 't' || b == 'm' || b == 'd') return i + 2;
    if (i + 2 < n) {
      const uint32_t d = c[i + 2] | 32;
      if ((b == 'r' && d == 'e') || (b == 'v' && d == 'e') || (b == 'l' && d == 'l')) return i + 3;
    }
  }
  // 2. [^\r\n\p{L}\p{N}]?\p{L}+
  {
    int j = i;
    if (!is_L(a)) { if (!is_nl(a) && !is_N(a) && i + 1 < n && is_L(c[i + 1])) j = i + 1; else j = -1; }
    if (j >= 0) {
      while (j < n && is_L(c[j])) ++j;
      return j;
    }
  }
  // 3. \p{N}
  if (is_N(a)) return i + 1;
  // 4.  ?[^\s\p{L}\p{N}]+[\r\n]*
  {
    int k = i + (a == ' ' ? 1 : 0);
    if (k < n && !is_S(c[k]) && !is_L(c[k]) && !is_N(c[k])) {
      while (k < n && !is_S(c[k]) && !is_L(c[k]) && !is_N(c[k])) ++k;
      while (k < n && is_nl(c[k])) ++k;
      return k;
    }
  }
  if (is_S(a)) {
    int e = i;
    while (e < n && is_S(c[e])) ++e;
    // 5. \s*[\r\n]+ : up to and including the last newline of the run
    int last_nl = -1;
    for (int q = i; q < e; ++q) if (is_nl(c[q])) last_nl = q;
    if (last_nl >= 0) return last_nl + 1;
    // 6. \s+(?!\S)
    if (e == n) return e;
    if (e - i >= 2) return e - 1;
    // 7. \s+
    return e;
  }
  return i + 1;
}

void bpe_word(Tok& t, const std::string& bytes, std::vector<int>& out) {
  auto it = t.cache.find(bytes);
  if (it != t.cache.end()) { out.insert(out.end(), it->second.begin(), it->second.end()); return; }
  std::vector<int> ids;
  if (t.ignore_merges) {
    std::string mapped;
    for (unsigned char b : bytes) mapped += t.byte_sym[b];
    auto v = t.vocab.find(mapped);
    if (v != t.vocab.end()) ids.push_back(v->second);
  }
  if (ids.empty()) {
    ids.reserve(bytes.size());
    for (unsigned char b : bytes) ids.push_back(t.byte_id[b]);
    while (ids.size() > 1) {
      int best = -1, best_rank = INT32_MAX;
      for (size_t k = 0; k + 1 < ids.size(); ++k) {
        auto m = t.merges.find({ids[k], ids[k + 1]});
        if (m != t.merges.end() && m->second < best_rank) { best_rank = m->second; best = (int)k; }
      }
      if (best < 0) break;
      const int merged = t.merged[{ids[best], ids[best + 1]}];
      ids[best] = merged;
      ids.erase(ids.begin() + best + 1);
    }
  }
  if (t.cache.size() < 200000) t.cache[bytes] = ids;
  out.insert(out.end(), ids.begin(), ids.end());
}

void encode_plain(Tok& t, const char* s, int n, std::vector<int>& out) {
  std::vector<uint32_t> cps;
  std::vector<int> offs;
  decode_utf8(s, n, cps, offs);
  int i = 0;
  const int m = (int)cps.size();
  while (i < m) {
    const int j = next_piece(cps, i);
    bpe_word(t, std::string(s + offs[i], s + offs[j]), out);
    i = j;
  }
}

}  // namespace

extern "C" {

void* grm_tok_load(const char* path, char* err, int cap) {
  auto fail = [&](const std::string& m) -> void* {
    if (err && cap > 0) { std::strncpy(err, m.c_str(), cap - 1); err[cap - 1] = 0; }
    return nullptr;
  };
  std::ifstream f(path, std::ios::binary);
  if (!f) return fail(std::string("cannot open ") + path);
  std::stringstream ss;
  ss << f.rdbuf();
  const std::string text = ss.str();
  Json root;
  grm::JsonParser ps(text);
  if (!ps.parse_document(root)) return fail("tokenizer.json: " + ps.err);
  const Json* model = root.get("model");
  if (!model || !model->get("vocab") || !model->get("merges")) return fail("tokenizer.json: no BPE model");
  Tok* t = new Tok();
  build_byte_map(*t);
  const Json* vocab = model->get("vocab");
  size_t max_id = 0;
  for (auto& kv : vocab->obj) max_id = std::max(max_id, (size_t)kv.second.num);
  const Json* added = root.get("added_tokens");
  if (added) for (auto& a : added->arr) if (a.get("id")) max_id = std::max(max_id, (size_t)a.get("id")->num);
  t->id_to_tok.assign(max_id + 1, "");
  for (auto& kv : vocab->obj) { t->vocab[kv.first] = (int)kv.second.num; t->id_to_tok[(size_t)kv.second.num] = kv.first; }
  if (const Json* im = model->get("ignore_merges")) t->ignore_merges = im->type == Json::Bool && im->b;
  int rank = 0;
  for (auto& m : model->get("merges")->arr) {
    std::string l, r;
    if (m.type == Json::Arr && m.arr.size() == 2) { l = m.arr[0].str; r = m.arr[1].str; }
    else if (m.type == Json::Str) { const size_t sp = m.str.find(' '); if (sp == std::string::npos) continue; l = m.str.substr(0, sp); r = m.str.substr(sp + 1); }
    else continue;
    auto li = t->vocab.find(l), ri = t->vocab.find(r), mi = t->vocab.find(l + r);
    if (li == t->vocab.end() || ri == t->vocab.end() || mi == t->vocab.end()) { ++rank; continue; }
    t->merges[{li->second, ri->second}] = rank++;
    t->merged[{li->second, ri->second}] = mi->second;
  }
  for (int b = 0; b < 256; ++b) {
    auto v = t->vocab.find(t->byte_sym[b]);
    t->byte_id[b] = v == t->vocab.end() ? 0 : v->second;
  }
  if (added) {
    for (auto& a : added->arr) {
      const Json* c = a.get("content");
      const Json* id = a.get("id");
      if (!c || !id) continue;
      const bool special = a.get("special") && a.get("special")->b;
      t->added.emplace_back(c->str, (int)id->num);
      if ((size_t)id->num < t->id_to_tok.size()) t->id_to_tok[(size_t)id->num] = c->str;
      if (special) t->special_ids[(int)id->num] = 1;
      t->vocab[c->str] = (int)id->num;
    }
    std::stable_sort(t->added.begin(), t->added.end(), [](auto& x, auto& y) { return x.first.size() > y.first.size(); });
  }
  return t;
}

void grm_tok_free(void* h) { delete static_cast<Tok*>(h); }
int grm_tok_vocab_size(void* h) { return (int)static_cast<Tok*>(h)->id_to_tok.size(); }

int grm_tok_token_id(void* h, const char* s) {
  Tok* t = static_cast<Tok*>(h);
  auto it = t->vocab.find(s);
  return it == t->vocab.end() ? -1 : it->second;
}

int grm_tok_is_special(void* h, int id) { return static_cast<Tok*>(h)->special_ids.count(id) ? 1 : 0; }

// Returns the number of ids (written up to cap); allow_special = 0 encodes special-token text as plain text.
int grm_tok_encode(void* h, const char* s, int n, int* out, int cap, int allow_special) {
  Tok* t = static_cast<Tok*>(h);
  std::vector<int> ids;
  int i = 0, seg = 0;
  while (i < n) {
    int hit = -1;
    if (allow_special) {
      for (size_t a = 0; a < t->added.size(); ++a) {
        const std::string& c = t->added[a].first;
        if (!c.empty() && (int)c.size() <= n - i && s[i] == c[0] && std::memcmp(s + i, c.data(), c.size()) == 0) { hit = (int)a; break; }
      }
    }
    if (hit >= 0) {
      if (i > seg) encode_plain(*t, s + seg, i - seg, ids);
      ids.push_back(t->added[hit].second);
      i += (int)t->added[hit].first.size();
      seg = i;
    } else {
      ++i;
    }
  }
  if (n > seg) encode_plain(*t, s + seg, n - seg, ids);
  for (int k = 0; k < (int)ids.size() && k < cap; ++k) out[k] = ids[k];
  return (int)ids.size();
}

// Returns the number of bytes (written up to cap).  Byte-level tokens are mapped back to raw bytes;
// added tokens are emitted verbatim (or skipped when skip_special and marked special).
int grm_tok_decode(void* h, const int* ids, int n, char* out, int cap, int skip_special) {
  Tok* t = static_cast<Tok*>(h);
  std::string o;
  for (int k = 0; k < n; ++k) {
    const int id = ids[k];
    if (id < 0 || id >= (int)t->id_to_tok.size()) continue;
    if (t->special_ids.count(id)) { if (!skip_special) o += t->id_to_tok[id]; continue; }
    const std::string& tok = t->id_to_tok[id];
    bool is_added = false;
    for (auto& a : t->added) if (a.second == id) { is_added = true; break; }
    if (is_added) { o += tok; continue; }
    std::vector<uint32_t> cps;
    std::vector<int> offs;
    decode_utf8(tok.data(), (int)tok.size(), cps, offs);
    for (uint32_t cp : cps) {
      auto b = t->sym_byte.find(cp);
      if (b != t->sym_byte.end()) o += (char)b->second;
    }
  }
  const int m = (int)o.size();
  std::memcpy(out, o.data(), std::min(m, cap));
  return m;
}

}  // extern "C"
