// safetensors reader: mmap the file, parse the JSON header with a small strict parser, hand out
// (name, dtype, shape, byte range) records.  Same role as the reference's SafeTensors / HFModel
// (include/b70/safetensors.hpp:42-119, src/safetensors.cpp:252-400): zero-copy access to shards.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct TensorRec {
  std::string name, dtype;
  std::vector<int64_t> shape;
  int64_t begin = 0, end = 0;
};

struct StFile {
  int fd = -1;
  uint8_t* map = nullptr;
  size_t size = 0;
  uint64_t header_len = 0;
  std::vector<TensorRec> tensors;
  std::string metadata;   // raw JSON of __metadata__ ("" when absent)
  std::string error;
};

struct Parser {
  const char* p;
  const char* e;
  bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  std::string str() {
    ws();
    std::string out;
    if (p >= e || *p != '"') { ok = false; return out; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        switch (*p) {
          case 'n': out += '\n'; break;
          case 't': out += '\t'; break;
          case 'r': out += '\r'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'u': {   // keep ASCII escapes, pass others through as '?'
            if (p + 4 < e) { unsigned v = 0; for (int i = 1; i <= 4; ++i) { char c = p[i]; v = v * 16 + (c <= '9' ? c - '0' : (c | 32) - 'a' + 10); } out += v < 128 ? (char)v : '?'; p += 4; }
            break;
          }
          default: out += *p;
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= e) { ok = false; return out; }
    ++p;
    return out;
  }
  int64_t num() {
    ws();
    bool neg = false;
    if (p < e && *p == '-') { neg = true; ++p; }
    if (p >= e || *p < '0' || *p > '9') { ok = false; return 0; }
    int64_t v = 0;
    while (p < e && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0');
    return neg ? -v : v;
  }
  // skip any JSON value, returning its raw text
  std::string skip() {
    ws();
    const char* s = p;
    int depth = 0;
    bool in_str = false;
    while (p < e) {
      const char c = *p;
      if (in_str) { if (c == '\\') ++p; else if (c == '"') in_str = false; }
      else if (c == '"') in_str = true;
      else if (c == '{' || c == '[') ++depth;
      else if (c == '}' || c == ']') { if (depth == 0) break; --depth; if (depth == 0) { ++p; break; } }
      else if (c == ',' && depth == 0) break;
      ++p;
    }
    return std::string(s, p);
  }
};

bool parse_header(StFile& f) {
  Parser ps{reinterpret_cast<const char*>(f.map + 8), reinterpret_cast<const char*>(f.map + 8 + f.header_len)};
  if (!ps.eat('{')) { f.error = "header is not a JSON object"; return false; }
  if (ps.eat('}')) return true;
  do {
    std::string key = ps.str();
    if (!ps.ok || !ps.eat(':')) { f.error = "bad key"; return false; }
    if (key == "__metadata__") { f.metadata = ps.skip(); continue; }
    TensorRec t;
    t.name = key;
    if (!ps.eat('{')) { f.error = "tensor entry is not an object: " + key; return false; }
    do {
      std::string k = ps.str();
      if (!ps.ok || !ps.eat(':')) { f.error = "bad field in " + key; return false; }
      if (k == "dtype") t.dtype = ps.str();
      else if (k == "shape") {
        if (!ps.eat('[')) { f.error = "bad shape in " + key; return false; }
        if (!ps.eat(']')) { do { t.shape.push_back(ps.num()); } while (ps.eat(',')); if (!ps.eat(']')) { f.error = "bad shape in " + key; return false; } }
      } else if (k == "data_offsets") {
        if (!ps.eat('[')) { f.error = "bad offsets in " + key; return false; }
        t.begin = ps.num(); if (!ps.eat(',')) { f.error = "bad offsets in " + key; return false; }
        t.end = ps.num(); if (!ps.eat(']')) { f.error = "bad offsets in " + key; return false; }
      } else ps.skip();
      if (!ps.ok) { f.error = "bad value in " + key; return false; }
    } while (ps.eat(','));
    if (!ps.eat('}')) { f.error = "unterminated entry " + key; return false; }
    const int64_t data_len = (int64_t)f.size - 8 - (int64_t)f.header_len;
    if (t.begin < 0 || t.end < t.begin || t.end > data_len) { f.error = "data offsets out of range: " + key; return false; }
    // the byte range must be exactly shape x element size (a mismatch would otherwise surface as a reshape error, or as a
    // read past the tensor when a caller trusts the shape)
    {
      static const struct { const char* n; int64_t b; } kDt[] = {{"F64", 8}, {"F32", 4}, {"F16", 2}, {"BF16", 2}, {"I64", 8}, {"I32", 4},
                                                               {"I16", 2}, {"I8", 1}, {"U8", 1}, {"BOOL", 1}, {"F8_E4M3", 1}, {"F8_E5M2", 1},
                                                               {"U16", 2}, {"U32", 4}, {"U64", 8}, {"F8_E8M0", 1}};
      int64_t esz = 0;
      for (const auto& d : kDt) if (t.dtype == d.n) esz = d.b;
      if (esz) {
        int64_t n = esz;
        bool bad = false;
        for (int64_t d : t.shape) bad = bad || d < 0 || __builtin_mul_overflow(n, d, &n);
        if (bad || n != t.end - t.begin) { f.error = "byte length does not match shape x dtype: " + key; return false; }
      }
    }
    f.tensors.push_back(std::move(t));
  } while (ps.eat(','));
  if (!ps.eat('}')) { f.error = "unterminated header"; return false; }
  return true;
}

}  // namespace

extern "C" {

void* grm_st_open(const char* path, char* err, int err_cap) {
  StFile* f = new StFile();
  auto fail = [&](const std::string& m) -> void* {
    if (err && err_cap > 0) { std::strncpy(err, m.c_str(), err_cap - 1); err[err_cap - 1] = 0; }
    if (f->map) munmap(f->map, f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
    return nullptr;
  };
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) return fail(std::string("cannot open ") + path);
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 8) return fail("file too small for a safetensors header");
  f->size = (size_t)st.st_size;
  f->map = static_cast<uint8_t*>(mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0));
  if (f->map == MAP_FAILED) { f->map = nullptr; return fail("mmap failed"); }
  std::memcpy(&f->header_len, f->map, 8);
  if (f->header_len > f->size - 8 || f->header_len > (1ull << 30)) return fail("header length out of range");
  if (!parse_header(*f)) return fail(f->error);
  return f;
}

void grm_st_close(void* h) {
  StFile* f = static_cast<StFile*>(h);
  if (!f) return;
  if (f->map) munmap(f->map, f->size);
  if (f->fd >= 0) close(f->fd);
  delete f;
}

int grm_st_count(void* h) { return (int)static_cast<StFile*>(h)->tensors.size(); }

// shape: up to 8 dims.  Returns ndim, or -1 on a bad index / too small name buffer.
int grm_st_info(void* h, int i, char* name, int name_cap, char* dtype, int dtype_cap, int64_t* shape, int64_t* begin, int64_t* end) {
  StFile* f = static_cast<StFile*>(h);
  if (i < 0 || i >= (int)f->tensors.size()) return -1;
  const TensorRec& t = f->tensors[i];
  if ((int)t.name.size() >= name_cap || (int)t.dtype.size() >= dtype_cap || t.shape.size() > 8) return -1;
  std::strcpy(name, t.name.c_str());
  std::strcpy(dtype, t.dtype.c_str());
  for (size_t d = 0; d < t.shape.size(); ++d) shape[d] = t.shape[d];
  *begin = t.begin; *end = t.end;
  return (int)t.shape.size();
}

const void* grm_st_data(void* h) { StFile* f = static_cast<StFile*>(h); return f->map + 8 + f->header_len; }
int64_t grm_st_data_len(void* h) { StFile* f = static_cast<StFile*>(h); return (int64_t)f->size - 8 - (int64_t)f->header_len; }
int grm_st_metadata(void* h, char* out, int cap) {
  StFile* f = static_cast<StFile*>(h);
  if ((int)f->metadata.size() >= cap) return -1;
  std::strcpy(out, f->metadata.c_str());
  return (int)f->metadata.size();
}

}  // extern "C"
