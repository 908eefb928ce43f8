// C ABI over the codec header so python tests can check the C++ codecs against the torch oracle.
#include "codecs.hpp"

extern "C" {
void grm_h_bf16_to_f32(const uint16_t* in, float* out, long n) { for (long i = 0; i < n; ++i) out[i] = grm::bf16_to_f32(in[i]); }
void grm_h_f32_to_bf16(const float* in, uint16_t* out, long n) { for (long i = 0; i < n; ++i) out[i] = grm::f32_to_bf16(in[i]); }
void grm_h_f16_to_f32(const uint16_t* in, float* out, long n) { for (long i = 0; i < n; ++i) out[i] = grm::f16_to_f32(in[i]); }
void grm_h_e2m1_to_f32(const uint8_t* in, float* out, long n) { for (long i = 0; i < n; ++i) out[i] = grm::e2m1_to_f32(in[i]); }
void grm_h_f32_to_e2m1(const float* in, uint8_t* out, long n) { for (long i = 0; i < n; ++i) out[i] = grm::f32_to_e2m1(in[i]); }
void grm_h_e4m3_to_f32(const uint8_t* in, float* out, long n) { for (long i = 0; i < n; ++i) out[i] = grm::e4m3_to_f32(in[i]); }
void grm_h_e5m2_to_f32(const uint8_t* in, float* out, long n) { for (long i = 0; i < n; ++i) out[i] = grm::e5m2_to_f32(in[i]); }
void grm_h_e8m0_to_f32(const uint8_t* in, float* out, long n) { for (long i = 0; i < n; ++i) out[i] = grm::e8m0_to_f32(in[i]); }
}
