// Element codecs shared by the host runtime (C++17, no CUDA): bf16, fp16, E8M0, E2M1, E4M3, E5M2.
// Counterpart of the reference's SYCL-free codec header (include/b70/formats.hpp:65-232); the
// torch versions in grimoire_b200/formats/codecs.py are the oracle these are tested against.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

namespace grm {

inline float bits_to_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
inline uint32_t f32_to_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

inline float bf16_to_f32(uint16_t b) { return bits_to_f32((uint32_t)b << 16); }
inline uint16_t f32_to_bf16(float f) {
  uint32_t u = f32_to_bits(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
  return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}

inline float f16_to_f32(uint16_t h) {
  const uint32_t s = (uint32_t)(h & 0x8000) << 16;
  uint32_t e = (h >> 10) & 0x1f, m = h & 0x3ff;
  if (e == 0) {
    if (m == 0) return bits_to_f32(s);
    int sh = 0;
    while (!(m & 0x400)) { m <<= 1; ++sh; }
    m &= 0x3ff;
    return bits_to_f32(s | ((uint32_t)(113 - sh) << 23) | (m << 13));
  }
  if (e == 31) return bits_to_f32(s | 0x7f800000u | (m << 13));
  return bits_to_f32(s | ((e + 112) << 23) | (m << 13));
}

inline float e8m0_to_f32(uint8_t e) { return e == 255 ? NAN : std::ldexp(1.0f, (int)e - 127); }

inline float e2m1_to_f32(uint8_t c) {
  static const float tbl[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = tbl[c & 7];
  return (c & 8) ? -v : v;
}
// round to nearest even with saturation
inline uint8_t f32_to_e2m1(float x) {
  const float a = std::fabs(x);
  static const float mids[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  int code = 0;
  for (int i = 0; i < 7; ++i) {
    const int nxt = i + 1;
    if ((nxt & 1) == 0 ? a >= mids[i] : a > mids[i]) code = nxt;
  }
  if (std::isnan(x)) code = 7;
  return (uint8_t)(code | (std::signbit(x) ? 8 : 0));
}

inline float e4m3_to_f32(uint8_t c) {
  const int s = c >> 7, e = (c >> 3) & 0xf, m = c & 7;
  float v;
  if (e == 0) v = std::ldexp((float)m, -9);
  else if (e == 15 && m == 7) v = NAN;
  else v = std::ldexp(1.0f + m / 8.0f, e - 7);
  return s ? -v : v;
}
inline float e5m2_to_f32(uint8_t c) {
  const int s = c >> 7, e = (c >> 2) & 0x1f, m = c & 3;
  float v;
  if (e == 0) v = std::ldexp((float)m, -16);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = std::ldexp(1.0f + m / 4.0f, e - 15);
  return s ? -v : v;
}

}  // namespace grm
