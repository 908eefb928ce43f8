// sample_logits: temperature / top-k (<= 64) / nucleus sampling of one token per row, on the device.
// Reference: launch_sample_logits (src/sample_logits.hpp:41-134: 2-stage top-k, softmax, nucleus,
// draw) with the counter-based generator of include/b70/sampling.hpp:10-35 -- the uniform number is
// splitmix64(seed, position), so no generator state lives in a captured graph and a replay with a
// new position draws a new number.
//
// Stage 1: grid (64 chunks, rows); each CTA keeps its vocabulary slice in shared memory and extracts
// its local top-k by k rounds of block arg-max (ties -> lowest index).  Stage 2: the last CTA to
// arrive for a row merges the 64*k candidates, extracts the global top-k in descending order,
// applies softmax(logit / T), cuts the nucleus at top_p and inverts the CDF at u.
#include "common.cuh"

namespace {

constexpr int kChunks = 64;
constexpr int kMaxK = 64;
constexpr int kThreads = 256;
constexpr int kSliceMax = 4096;     // vocabulary <= 64 * 4096 = 262144

struct SampleParams {
  const float* logits; int ld; int V;
  const int* positions;             // [M] counter input of the generator (device resident)
  const float* temperature;         // [M]
  const float* top_p;               // [M]
  const int* top_k;                 // [M]
  const unsigned long long* seeds;  // [M]
  float* cand_val; int* cand_idx;   // [M][64][64]
  unsigned int* counters;           // [M]
  int* out;                         // [M]
};

__device__ __forceinline__ double splitmix_uniform(unsigned long long seed, unsigned long long pos) {
  unsigned long long x = seed ^ (pos * 0x9E3779B97F4A7C15ull);
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  x ^= x >> 31;
  return (double)(x >> 11) * (1.0 / 9007199254740992.0);
}

__device__ __forceinline__ void better(float& bv, int& bi, float ov, int oi) {
  if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
}

// block arg-max over vals[0..n) (entries already taken are -inf); returns (value, position in vals)
__device__ void block_argmax(const float* vals, const int* ids, int n, float* sv, int* si, float& out_v, int& out_p) {
  float bv = -INFINITY; int bi = 0x7fffffff, bp = -1;
  for (int i = threadIdx.x; i < n; i += kThreads) {
    const float v = vals[i];
    const int id = ids ? ids[i] : i;
    if (v > bv || (v == bv && id < bi)) { bv = v; bi = id; bp = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    const int op = __shfl_xor_sync(0xffffffffu, bp, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bp = op; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; si[8 + warp] = bp; }
  __syncthreads();
  bv = sv[0]; bi = si[0]; bp = si[8];
  for (int w = 1; w < kThreads / 32; ++w)
    if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; bp = si[8 + w]; }
  out_v = bv; out_p = bp;
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const SampleParams p) {
  __shared__ float slice[kSliceMax];
  __shared__ int slice_id[kSliceMax];
  __shared__ float sv[8];
  __shared__ int si[16];
  __shared__ int s_last;
  const int row = blockIdx.y, chunk = blockIdx.x;
  const int k = max(1, min(kMaxK, p.top_k[row]));
  const int per = (p.V + kChunks - 1) / kChunks;
  const int lo = chunk * per, hi = min(p.V, lo + per), n = max(0, hi - lo);
  const float* lg = p.logits + (size_t)row * p.ld;
  for (int i = threadIdx.x; i < n; i += kThreads) slice[i] = lg[lo + i];
  __syncthreads();
  float* cv = p.cand_val + ((size_t)row * kChunks + chunk) * kMaxK;
  int* ci = p.cand_idx + ((size_t)row * kChunks + chunk) * kMaxK;
  for (int r = 0; r < k; ++r) {
    float v; int pos;
    block_argmax(slice, nullptr, n, sv, si, v, pos);
    if (threadIdx.x == 0) {
      cv[r] = (pos >= 0) ? v : -INFINITY;
      ci[r] = (pos >= 0) ? lo + pos : 0x7fffffff;
      if (pos >= 0) slice[pos] = -INFINITY;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(&p.counters[row], 1u);
    s_last = (prev == kChunks - 1);
    if (s_last) p.counters[row] = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // ---- stage 2: merge 64*k candidates ----
  const int nc = kChunks * k;
  for (int i = threadIdx.x; i < nc; i += kThreads) {
    const int c = i / k, r = i % k;
    slice[i] = __ldcg(p.cand_val + ((size_t)row * kChunks + c) * kMaxK + r);
    slice_id[i] = __ldcg(p.cand_idx + ((size_t)row * kChunks + c) * kMaxK + r);
  }
  __syncthreads();
  __shared__ float topv[kMaxK];
  __shared__ int topi[kMaxK];
  for (int r = 0; r < k; ++r) {
    float v; int pos;
    block_argmax(slice, slice_id, nc, sv, si, v, pos);
    if (threadIdx.x == 0) {
      topv[r] = v; topi[r] = (pos >= 0) ? slice_id[pos] : 0;
      if (pos >= 0) slice[pos] = -INFINITY;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float T = p.temperature[row];
    int choice = topi[0];
    if (T > 0.f && k > 1) {
      const float inv = 1.f / T;
      const float mx = topv[0];
      float pr[kMaxK];
      float sum = 0.f;
      for (int r = 0; r < k; ++r) { pr[r] = (topv[r] == -INFINITY) ? 0.f : expf((topv[r] - mx) * inv); sum += pr[r]; }
      // nucleus: smallest prefix of the sorted candidates whose mass reaches top_p
      const float tp = p.top_p[row];
      int keep = k;
      if (tp > 0.f && tp < 1.f) {
        float acc = 0.f;
        for (int r = 0; r < k; ++r) { acc += pr[r] / sum; if (acc >= tp) { keep = r + 1; break; } }
      }
      float ksum = 0.f;
      for (int r = 0; r < keep; ++r) ksum += pr[r];
      const float u = (float)splitmix_uniform(p.seeds[row], (unsigned long long)(long long)p.positions[row]) * ksum;
      float acc = 0.f;
      choice = topi[keep - 1];
      for (int r = 0; r < keep; ++r) { acc += pr[r]; if (u < acc) { choice = topi[r]; break; } }
    }
    p.out[row] = choice;
  }
}

}  // namespace

// cand_val / cand_idx: M*64*64 floats / ints of scratch, counters: M zeroed uints (left at zero).
GRM_API int grm_sample_logits(const void* logits, int ld, int V, const void* positions, const void* temperature,
                              const void* top_p, const void* top_k, const void* seeds, void* cand_val, void* cand_idx,
                              void* counters, void* out, int M, void* stream) {
  if (M < 1 || V < 1 || V > kChunks * kSliceMax) return -2;
  SampleParams p;
  p.logits = (const float*)logits; p.ld = ld; p.V = V; p.positions = (const int*)positions;
  p.temperature = (const float*)temperature; p.top_p = (const float*)top_p; p.top_k = (const int*)top_k;
  p.seeds = (const unsigned long long*)seeds; p.cand_val = (float*)cand_val; p.cand_idx = (int*)cand_idx;
  p.counters = (unsigned int*)counters; p.out = (int*)out;
  dim3 grid(kChunks, M);
  sample_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}
