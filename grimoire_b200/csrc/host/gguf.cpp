// GGUF v2/v3 container parser and block dequantisers (host).
// Reference: GGUFFile (include/b70/gguf.hpp, src/gguf.cpp) and gguf_dequantize
// (src/gguf_decode.cpp:45).  Block layouts and arithmetic follow the public ggml definitions; the
// decoders are checked against llama.cpp-derived golden vectors when those are available
// (tests/test_gguf.py).  Codebook ("IQ1/IQ2/IQ3") and TQ1_0 types are recognised by the parser but
// not decoded.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "codecs.hpp"
#include "json.hpp"

namespace {

struct TypeInfo { int id, elems, size; const char* name; };
const TypeInfo kTypes[] = {
    {0, 1, 4, "F32"}, {1, 1, 2, "F16"}, {2, 32, 18, "Q4_0"}, {3, 32, 20, "Q4_1"}, {6, 32, 22, "Q5_0"}, {7, 32, 24, "Q5_1"},
    {8, 32, 34, "Q8_0"}, {9, 32, 36, "Q8_1"}, {10, 256, 84, "Q2_K"}, {11, 256, 110, "Q3_K"}, {12, 256, 144, "Q4_K"},
    {13, 256, 176, "Q5_K"}, {14, 256, 210, "Q6_K"}, {15, 256, 292, "Q8_K"}, {16, 256, 66, "IQ2_XXS"}, {17, 256, 74, "IQ2_XS"},
    {18, 256, 98, "IQ3_XXS"}, {19, 256, 50, "IQ1_S"}, {20, 32, 18, "IQ4_NL"}, {21, 256, 110, "IQ3_S"}, {22, 256, 82, "IQ2_S"},
    {23, 256, 136, "IQ4_XS"}, {24, 1, 1, "I8"}, {25, 1, 2, "I16"}, {26, 1, 4, "I32"}, {27, 1, 8, "I64"}, {28, 1, 8, "F64"},
    {29, 256, 56, "IQ1_M"}, {30, 1, 2, "BF16"}, {34, 256, 54, "TQ1_0"}, {35, 256, 66, "TQ2_0"}, {39, 32, 17, "MXFP4"},
};
const TypeInfo* type_info(int id) {
  for (const auto& t : kTypes) if (t.id == id) return &t;
  return nullptr;
}

const int8_t kIQ4NL[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
const int8_t kMXFP4[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

inline float h2f(const uint8_t* p) { uint16_t v; std::memcpy(&v, p, 2); return grm::f16_to_f32(v); }

inline void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) { *d = q[j] & 63; *m = q[j + 4] & 63; }
  else { *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); *m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// Decode `nblocks` blocks of `type` at `src` into fp32.  Returns 0, or -1 for an undecodable type.
int dequant_blocks(int type, const uint8_t* src, int64_t nblocks, float* y) {
  const TypeInfo* ti = type_info(type);
  if (!ti) return -1;
  for (int64_t b = 0; b < nblocks; ++b, src += ti->size) {
    switch (type) {
      case 0: { float v; std::memcpy(&v, src, 4); *y++ = v; break; }
      case 1: *y++ = h2f(src); break;
      case 30: { uint16_t v; std::memcpy(&v, src, 2); *y++ = grm::bf16_to_f32(v); break; }
      case 28: { double v; std::memcpy(&v, src, 8); *y++ = (float)v; break; }
      case 24: *y++ = (float)(int8_t)src[0]; break;
      case 25: { int16_t v; std::memcpy(&v, src, 2); *y++ = (float)v; break; }
      case 26: { int32_t v; std::memcpy(&v, src, 4); *y++ = (float)v; break; }
      case 27: { int64_t v; std::memcpy(&v, src, 8); *y++ = (float)v; break; }
      case 2: {   // Q4_0
        const float d = h2f(src); const uint8_t* qs = src + 2;
        for (int j = 0; j < 16; ++j) { y[j] = ((qs[j] & 0xF) - 8) * d; y[j + 16] = ((qs[j] >> 4) - 8) * d; }
        y += 32; break;
      }
      case 3: {   // Q4_1
        const float d = h2f(src), m = h2f(src + 2); const uint8_t* qs = src + 4;
        for (int j = 0; j < 16; ++j) { y[j] = (qs[j] & 0xF) * d + m; y[j + 16] = (qs[j] >> 4) * d + m; }
        y += 32; break;
      }
      case 6: {   // Q5_0
        const float d = h2f(src); uint32_t qh; std::memcpy(&qh, src + 2, 4); const uint8_t* qs = src + 6;
        for (int j = 0; j < 16; ++j) {
          const uint8_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
          y[j] = (((qs[j] & 0xF) | xh0) - 16) * d; y[j + 16] = (((qs[j] >> 4) | xh1) - 16) * d;
        }
        y += 32; break;
      }
      case 7: {   // Q5_1
        const float d = h2f(src), m = h2f(src + 2); uint32_t qh; std::memcpy(&qh, src + 4, 4); const uint8_t* qs = src + 8;
        for (int j = 0; j < 16; ++j) {
          const uint8_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
          y[j] = ((qs[j] & 0xF) | xh0) * d + m; y[j + 16] = ((qs[j] >> 4) | xh1) * d + m;
        }
        y += 32; break;
      }
      case 8: { const float d = h2f(src); for (int j = 0; j < 32; ++j) y[j] = (int8_t)src[2 + j] * d; y += 32; break; }
      case 9: { const float d = h2f(src); for (int j = 0; j < 32; ++j) y[j] = (int8_t)src[4 + j] * d; y += 32; break; }
      case 10: {  // Q2_K
        const uint8_t* scales = src; const uint8_t* q = src + 16; const float d = h2f(src + 80), mn = h2f(src + 82);
        int is = 0;
        for (int n = 0; n < 256; n += 128) {
          int shift = 0;
          for (int j = 0; j < 4; ++j) {
            uint8_t sc = scales[is++]; float dl = d * (sc & 0xF), ml = mn * (sc >> 4);
            for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l] >> shift) & 3)) - ml;
            sc = scales[is++]; dl = d * (sc & 0xF); ml = mn * (sc >> 4);
            for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l + 16] >> shift) & 3)) - ml;
            shift += 2;
          }
          q += 32;
        }
        break;
      }
      case 11: {  // Q3_K
        const uint8_t* hm = src; const uint8_t* q = src + 32; const float d_all = h2f(src + 108);
        const uint32_t kmask1 = 0x03030303, kmask2 = 0x0f0f0f0f;
        uint32_t aux[4];
        std::memcpy(aux, src + 96, 12);
        const uint32_t tmp = aux[2];
        aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
        aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
        aux[0] = (aux[0] & kmask2) | (((tmp >> 0) & kmask1) << 4);
        aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
        const int8_t* scales = reinterpret_cast<const int8_t*>(aux);
        int is = 0; uint8_t m = 1;
        for (int n = 0; n < 256; n += 128) {
          int shift = 0;
          for (int j = 0; j < 4; ++j) {
            float dl = d_all * (scales[is++] - 32);
            for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l] >> shift) & 3) - ((hm[l] & m) ? 0 : 4));
            dl = d_all * (scales[is++] - 32);
            for (int l = 0; l < 16; ++l) *y++ = dl * ((int8_t)((q[l + 16] >> shift) & 3) - ((hm[l + 16] & m) ? 0 : 4));
            shift += 2; m <<= 1;
          }
          q += 32;
        }
        break;
      }
      case 12: {  // Q4_K
        const float d = h2f(src), mn = h2f(src + 2); const uint8_t* scales = src + 4; const uint8_t* q = src + 16;
        int is = 0; uint8_t sc, m;
        for (int j = 0; j < 256; j += 64) {
          scale_min_k4(is + 0, scales, &sc, &m); const float d1 = d * sc, m1 = mn * m;
          scale_min_k4(is + 1, scales, &sc, &m); const float d2 = d * sc, m2 = mn * m;
          for (int l = 0; l < 32; ++l) *y++ = d1 * (q[l] & 0xF) - m1;
          for (int l = 0; l < 32; ++l) *y++ = d2 * (q[l] >> 4) - m2;
          q += 32; is += 2;
        }
        break;
      }
      case 13: {  // Q5_K
        const float d = h2f(src), mn = h2f(src + 2); const uint8_t* scales = src + 4; const uint8_t* qh = src + 16; const uint8_t* ql = src + 48;
        int is = 0; uint8_t sc, m, u1 = 1, u2 = 2;
        for (int j = 0; j < 256; j += 64) {
          scale_min_k4(is + 0, scales, &sc, &m); const float d1 = d * sc, m1 = mn * m;
          scale_min_k4(is + 1, scales, &sc, &m); const float d2 = d * sc, m2 = mn * m;
          for (int l = 0; l < 32; ++l) *y++ = d1 * ((ql[l] & 0xF) + (qh[l] & u1 ? 16 : 0)) - m1;
          for (int l = 0; l < 32; ++l) *y++ = d2 * ((ql[l] >> 4) + (qh[l] & u2 ? 16 : 0)) - m2;
          ql += 32; is += 2; u1 <<= 2; u2 <<= 2;
        }
        break;
      }
      case 14: {  // Q6_K
        const uint8_t* ql = src; const uint8_t* qh = src + 128; const int8_t* sc = reinterpret_cast<const int8_t*>(src + 192);
        const float d = h2f(src + 208);
        for (int n = 0; n < 256; n += 128) {
          for (int l = 0; l < 32; ++l) {
            const int is = l / 16;
            const int8_t q1 = (int8_t)((ql[l + 0] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
            const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int8_t q3 = (int8_t)((ql[l + 0] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            y[l + 0] = d * sc[is + 0] * q1; y[l + 32] = d * sc[is + 2] * q2; y[l + 64] = d * sc[is + 4] * q3; y[l + 96] = d * sc[is + 6] * q4;
          }
          y += 128; ql += 64; qh += 32; sc += 8;
        }
        break;
      }
      case 15: { float d; std::memcpy(&d, src, 4); for (int j = 0; j < 256; ++j) y[j] = d * (int8_t)src[4 + j]; y += 256; break; }
      case 20: {  // IQ4_NL
        const float d = h2f(src); const uint8_t* qs = src + 2;
        for (int j = 0; j < 16; ++j) { y[j] = d * kIQ4NL[qs[j] & 0xf]; y[j + 16] = d * kIQ4NL[qs[j] >> 4]; }
        y += 32; break;
      }
      case 23: {  // IQ4_XS
        const float d = h2f(src); uint16_t sh; std::memcpy(&sh, src + 2, 2); const uint8_t* sl = src + 4; const uint8_t* qs = src + 8;
        for (int ib = 0; ib < 8; ++ib) {
          const int ls = ((sl[ib / 2] >> 4 * (ib % 2)) & 0xf) | (((sh >> 2 * ib) & 3) << 4);
          const float dl = d * (ls - 32);
          for (int j = 0; j < 16; ++j) { y[j] = dl * kIQ4NL[qs[j] & 0xf]; y[j + 16] = dl * kIQ4NL[qs[j] >> 4]; }
          y += 32; qs += 16;
        }
        break;
      }
      case 35: {  // TQ2_0
        const uint8_t* qs = src; const float d = h2f(src + 64);
        for (int j = 0; j < 64; j += 32)
          for (int l = 0; l < 4; ++l)
            for (int m = 0; m < 32; ++m) *y++ = (float)(((qs[j + m] >> (l * 2)) & 3) - 1) * d;
        break;
      }
      case 39: {  // MXFP4 (ggml): E8M0 scale halved, e2m1 codes doubled
        const uint8_t e = src[0]; const uint8_t* qs = src + 1;
        uint32_t bits = e < 2 ? (0x00200000u << e) : ((uint32_t)(e - 1) << 23);
        const float d = grm::bits_to_f32(bits);
        for (int j = 0; j < 16; ++j) { y[j] = kMXFP4[qs[j] & 0xf] * d; y[j + 16] = kMXFP4[qs[j] >> 4] * d; }
        y += 32; break;
      }
      default: return -1;
    }
  }
  return 0;
}

struct GTensor { std::string name; int type; std::vector<uint64_t> dims; uint64_t offset; uint64_t nbytes; };

struct GFile {
  int fd = -1; uint8_t* map = nullptr; size_t size = 0;
  uint32_t version = 0; uint64_t data_start = 0;
  std::string meta_json;
  std::vector<GTensor> tensors;
};

struct Reader {
  const uint8_t* p; const uint8_t* e; bool ok = true;
  template <typename T> T get() { T v{}; if ((size_t)(e - p) < sizeof(T)) { ok = false; return v; } std::memcpy(&v, p, sizeof(T)); p += sizeof(T); return v; }
  std::string str() { const uint64_t n = get<uint64_t>(); if (!ok || n > (uint64_t)(e - p)) { ok = false; return ""; } std::string s((const char*)p, n); p += n; return s; }
};

bool value_json(Reader& r, uint32_t t, std::string& out, int depth = 0) {
  char buf[64];
  switch (t) {
    case 0: out += std::to_string(r.get<uint8_t>()); break;
    case 1: out += std::to_string(r.get<int8_t>()); break;
    case 2: out += std::to_string(r.get<uint16_t>()); break;
    case 3: out += std::to_string(r.get<int16_t>()); break;
    case 4: out += std::to_string(r.get<uint32_t>()); break;
    case 5: out += std::to_string(r.get<int32_t>()); break;
    case 6: { const float v = r.get<float>(); if (std::isfinite(v)) { snprintf(buf, sizeof buf, "%.9g", v); out += buf; } else out += "null"; break; }
    case 7: out += r.get<uint8_t>() ? "true" : "false"; break;
    case 8: out += "\"" + grm::json_escape(r.str()) + "\""; break;
    case 10: out += std::to_string(r.get<uint64_t>()); break;
    case 11: out += std::to_string(r.get<int64_t>()); break;
    case 12: { const double v = r.get<double>(); if (std::isfinite(v)) { snprintf(buf, sizeof buf, "%.17g", v); out += buf; } else out += "null"; break; }
    case 9: {
      if (depth > 4) return false;
      const uint32_t et = r.get<uint32_t>(); const uint64_t n = r.get<uint64_t>();
      if (!r.ok || n > (1ull << 28)) return false;
      out += "[";
      for (uint64_t i = 0; i < n && r.ok; ++i) { if (i) out += ","; if (!value_json(r, et, out, depth + 1)) return false; }
      out += "]";
      break;
    }
    default: return false;
  }
  return r.ok;
}

}  // namespace

extern "C" {

int grm_gguf_type_info(int type, int* elems, int* size, char* name, int cap) {
  const TypeInfo* t = type_info(type);
  if (!t) return -1;
  *elems = t->elems; *size = t->size;
  std::strncpy(name, t->name, cap - 1); name[cap - 1] = 0;
  return 0;
}

// raw: nbytes of blocks; out: n_elems floats.  -1 unknown/undecodable type, -2 size mismatch.
int grm_gguf_dequant(int type, const void* raw, int64_t nbytes, float* out, int64_t n_elems) {
  const TypeInfo* t = type_info(type);
  if (!t) return -1;
  if (n_elems % t->elems || nbytes != n_elems / t->elems * t->size) return -2;
  return dequant_blocks(type, static_cast<const uint8_t*>(raw), n_elems / t->elems, out);
}

void* grm_gguf_open(const char* path, char* err, int cap) {
  GFile* f = new GFile();
  auto fail = [&](const std::string& m) -> void* {
    if (err && cap > 0) { std::strncpy(err, m.c_str(), cap - 1); err[cap - 1] = 0; }
    if (f->map) munmap(f->map, f->size);
    if (f->fd >= 0) close(f->fd);
    delete f; return nullptr;
  };
  f->fd = open(path, O_RDONLY);
  if (f->fd < 0) return fail(std::string("cannot open ") + path);
  struct stat st;
  if (fstat(f->fd, &st) != 0 || st.st_size < 24) return fail("file too small");
  f->size = (size_t)st.st_size;
  f->map = static_cast<uint8_t*>(mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0));
  if (f->map == MAP_FAILED) { f->map = nullptr; return fail("mmap failed"); }
  Reader r{f->map, f->map + f->size};
  if (std::memcmp(r.p, "GGUF", 4) != 0) return fail("not a GGUF file");
  r.p += 4;
  f->version = r.get<uint32_t>();
  if (f->version != 2 && f->version != 3) return fail("unsupported GGUF version " + std::to_string(f->version));
  const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
  if (n_tensors > (1u << 24) || n_kv > (1u << 24)) return fail("implausible counts");
  uint64_t alignment = 32;
  f->meta_json = "{";
  for (uint64_t i = 0; i < n_kv; ++i) {
    const std::string key = r.str();
    const uint32_t vt = r.get<uint32_t>();
    if (!r.ok) return fail("truncated metadata");
    if (i) f->meta_json += ",";
    f->meta_json += "\"" + grm::json_escape(key) + "\":";
    const uint8_t* before = r.p;
    if (!value_json(r, vt, f->meta_json)) return fail("bad metadata value for " + key);
    if (key == "general.alignment" && vt == 4) {
      uint32_t a; std::memcpy(&a, before, 4);
      // a power of two no larger than a page: anything else is a damaged or hostile header
      if (a == 0 || a > 4096 || (a & (a - 1))) return fail("general.alignment must be a power of two <= 4096");
      alignment = a;
    }
  }
  f->meta_json += "}";
  for (uint64_t i = 0; i < n_tensors; ++i) {
    GTensor t;
    t.name = r.str();
    const uint32_t nd = r.get<uint32_t>();
    if (!r.ok || nd > 8) return fail("bad tensor record");
    uint64_t ne = 1;
    bool overflow = false;
    for (uint32_t d = 0; d < nd; ++d) {
      t.dims.push_back(r.get<uint64_t>());
      overflow = overflow || __builtin_mul_overflow(ne, t.dims.back(), &ne);
    }
    if (overflow) return fail("tensor element count overflows: " + t.name);
    t.type = (int)r.get<uint32_t>();
    t.offset = r.get<uint64_t>();
    const TypeInfo* ti = type_info(t.type);
    if (!r.ok || !ti || ne % ti->elems) return fail("bad tensor type/shape for " + t.name);
    if (__builtin_mul_overflow(ne / ti->elems, (uint64_t)ti->size, &t.nbytes)) return fail("tensor size overflows: " + t.name);
    f->tensors.push_back(std::move(t));
  }
  const uint64_t pos = (uint64_t)(r.p - f->map);
  f->data_start = (pos + alignment - 1) / alignment * alignment;
  if (f->data_start > f->size) return fail("tensor data section starts past the end of the file");
  const uint64_t room = f->size - f->data_start;
  for (auto& t : f->tensors)      // subtraction form: neither side can wrap
    if (t.offset > room || t.nbytes > room - t.offset) return fail("tensor data out of range: " + t.name);
  return f;
}

void grm_gguf_close(void* h) { GFile* f = static_cast<GFile*>(h); if (!f) return; if (f->map) munmap(f->map, f->size); if (f->fd >= 0) close(f->fd); delete f; }
int grm_gguf_version(void* h) { return (int)static_cast<GFile*>(h)->version; }
int grm_gguf_tensor_count(void* h) { return (int)static_cast<GFile*>(h)->tensors.size(); }
int64_t grm_gguf_meta_len(void* h) { return (int64_t)static_cast<GFile*>(h)->meta_json.size(); }
void grm_gguf_meta(void* h, char* out) { GFile* f = static_cast<GFile*>(h); std::memcpy(out, f->meta_json.data(), f->meta_json.size()); }
int grm_gguf_tensor_info(void* h, int i, char* name, int cap, int* type, uint64_t* dims, uint64_t* nbytes) {
  GFile* f = static_cast<GFile*>(h);
  if (i < 0 || i >= (int)f->tensors.size()) return -1;
  const GTensor& t = f->tensors[i];
  if ((int)t.name.size() >= cap) return -1;
  std::strcpy(name, t.name.c_str());
  *type = t.type; *nbytes = t.nbytes;
  for (size_t d = 0; d < t.dims.size(); ++d) dims[d] = t.dims[d];
  return (int)t.dims.size();
}
const void* grm_gguf_tensor_data(void* h, int i) { GFile* f = static_cast<GFile*>(h); return f->map + f->data_start + f->tensors[i].offset; }

}  // extern "C"
