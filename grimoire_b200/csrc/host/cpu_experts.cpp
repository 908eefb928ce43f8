// Expert FFN rows on the host: the RAM tier of the tiered-MoE manager.  Experts that do not fit the device budget stay in
// (pinned) host memory as the same block-scaled e4m3 bytes the device kernels read, and the routes that name them are
// computed here while the GPU runs the resident ones; the caller adds the fp32 partial into the layer's output.
// Reference: the host expert pool (src/cpu_experts.cpp; tiered_moe_cpu_rows, src/grimoire.cpp:18784) -- AVX2 rows over
// RAM-resident experts, folded into the MoE sum.
//
// One pair = (token row, host expert, routing weight):  a = silu(Wg x) * (Wu x), rounded to bf16 as the device chain
// stores it;  y = Wd a;  out[row] += weight * y.  Pairs are dealt to threads in blocks that share a token row, so a row
// of ``out`` has exactly one writer; the sum over a row's experts runs in pair order, so the result does not depend on
// the thread count.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <thread>
#include <vector>

#include "codecs.hpp"

namespace {

struct Lut {
  float v[256];
  Lut() {
    for (int i = 0; i < 256; ++i) {
      const float f = grm::e4m3_to_f32((uint8_t)i);
      v[i] = std::isnan(f) ? 0.f : f;
    }
  }
};
const Lut kLut;

// dot of one block-scaled e4m3 row (K bytes, K / 128 fp32 scales) with fp32 x
#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
__attribute__((target_clones("avx512f", "avx2,fma", "default")))
#endif
float dot_fp8_row(const uint8_t* w, const float* s, const float* x, int K) {
  float acc = 0.f;
  for (int b = 0; b < K; b += 128) {
    float part[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < 128; k += 8)
      for (int j = 0; j < 8; ++j) part[j] += kLut.v[w[b + k + j]] * x[b + k + j];
    acc += s[b >> 7] * (((part[0] + part[1]) + (part[2] + part[3])) + ((part[4] + part[5]) + (part[6] + part[7])));
  }
  return acc;
}

struct Job {
  const uint8_t *gu, *dn;
  const float *gus, *dns;
  const uint16_t* x;
  const int *row, *expert;
  const float* weight;
  float* out;
  int ldx, ldo, H, I;
};

void run_pairs(const Job& j, int p0, int p1) {
  std::vector<float> x(j.H), a(j.I), y(j.H);
  const size_t gu_e = (size_t)2 * j.I * j.H, dn_e = (size_t)j.H * j.I;
  const size_t gus_e = (size_t)2 * j.I * (j.H / 128), dns_e = (size_t)j.H * (j.I / 128);
  int last_row = -1;
  for (int p = p0; p < p1; ++p) {
    const int r = j.row[p], e = j.expert[p];
    if (r != last_row) {
      for (int k = 0; k < j.H; ++k) x[k] = grm::bf16_to_f32(j.x[(size_t)r * j.ldx + k]);
      last_row = r;
    }
    const uint8_t* gu = j.gu + e * gu_e;
    const float* gus = j.gus + e * gus_e;
    for (int n = 0; n < j.I; ++n) {
      const float g = dot_fp8_row(gu + (size_t)n * j.H, gus + (size_t)n * (j.H / 128), x.data(), j.H);
      const float u = dot_fp8_row(gu + (size_t)(j.I + n) * j.H, gus + (size_t)(j.I + n) * (j.H / 128), x.data(), j.H);
      a[n] = grm::bf16_to_f32(grm::f32_to_bf16(g / (1.f + std::exp(-g)) * u));
    }
    const uint8_t* dn = j.dn + e * dn_e;
    const float* dns = j.dns + e * dns_e;
    float* o = j.out + (size_t)r * j.ldo;
    const float wt = j.weight[p];
    for (int n = 0; n < j.H; ++n)
      o[n] += wt * dot_fp8_row(dn + (size_t)n * j.I, dns + (size_t)n * (j.I / 128), a.data(), j.I);
  }
}

}  // namespace

extern "C" {

// gu uint8 [E][2I][H] (gate rows then up rows), gus fp32 [E][2I][H/128], dn uint8 [E][H][I], dns fp32 [E][H][I/128];
// x bf16 [rows][ldx]; pairs sorted by row (pair_row non-decreasing); out fp32 [rows][ldo], accumulated into.
// Returns 0, or -2 for a shape the kernel does not serve.
int grm_cx_moe_rows(const void* gu, const void* gus, const void* dn, const void* dns, const void* x, int ldx, const int* pair_row,
                    const int* pair_expert, const float* pair_w, int n_pairs, float* out, int ldo, int H, int I, int threads) {
  if (H <= 0 || I <= 0 || (H & 127) || (I & 127) || n_pairs < 0) return -2;
  for (int p = 1; p < n_pairs; ++p)
    if (pair_row[p] < pair_row[p - 1]) return -2;
  if (n_pairs == 0) return 0;
  Job j{(const uint8_t*)gu, (const uint8_t*)dn, (const float*)gus, (const float*)dns, (const uint16_t*)x,
        pair_row, pair_expert, pair_w, out, ldx, ldo, H, I};
  threads = std::max(1, std::min(threads, n_pairs));
  if (threads == 1) {
    run_pairs(j, 0, n_pairs);
    return 0;
  }
  // cut points only where the token row changes: one writer per output row
  std::vector<int> cuts{0};
  for (int t = 1; t < threads; ++t) {
    int c = (int)((long)n_pairs * t / threads);
    while (c < n_pairs && c > 0 && pair_row[c] == pair_row[c - 1]) ++c;
    if (c > cuts.back() && c < n_pairs) cuts.push_back(c);
  }
  cuts.push_back(n_pairs);
  std::vector<std::thread> pool;
  for (size_t t = 0; t + 1 < cuts.size(); ++t) pool.emplace_back(run_pairs, std::cref(j), cuts[t], cuts[t + 1]);
  for (auto& th : pool) th.join();
  return 0;
}

}  // extern "C"
