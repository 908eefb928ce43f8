// Operators of the K2-Horizon family (reference: launch_rmsnorm_grouped, launch_softplus_gate, launch_router_topk_k2,
// launch_mova_value_decode -- src/ops.cpp:1963-2350, src/moe_kernels.cpp:465-624; host oracle include/b70/k2_horizon.hpp):
//   * grouped RMSNorm: variance per contiguous group of the row, weight over the whole row (plain w, not 1 + w);
//   * softplus attention gate: attn * softplus(gate, beta) with torch's linear region above beta * x = 20;
//   * sigmoid router with a selection-only bias: top-k on score + bias, weights from the unbiased scores;
//   * MoVA combine: value = sum_j w_j * silu(expert output j).
#include "common.cuh"

namespace {

// one CTA (256 threads) per row; groups walked one after the other
__global__ void __launch_bounds__(256) rmsnorm_grouped_kernel(const float* __restrict__ h, int ldh, const float* __restrict__ w,
                                                              bf16* __restrict__ out, int ldo, int n, int n_groups, float eps) {
  __shared__ float red[8];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = n / n_groups;
  const float* x = h + (size_t)row * ldh;
  for (int k = 0; k < n_groups; ++k) {
    float ss = 0.f;
    for (int i = tid; i < g; i += 256) { const float v = x[k * g + i]; ss = fmaf(v, v, ss); }
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float s = rsqrtf(tot / (float)g + eps);
    for (int i = tid; i < g; i += 256) out[(size_t)row * ldo + k * g + i] = __float2bfloat16(x[k * g + i] * s * w[k * g + i]);
    __syncthreads();
  }
}

__device__ __forceinline__ float softplus_beta(float x, float beta) {
  const float bx = beta * x;
  return bx > 20.f ? x : log1pf(__expf(bx)) / beta;
}

__global__ void softplus_gate_kernel(const bf16* __restrict__ attn, const bf16* __restrict__ gate, bf16* __restrict__ out, long n, float beta) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(__bfloat162float(attn[i]) * softplus_beta(__bfloat162float(gate[i]), beta));
}

// one warp per row; a lane holds experts lane, lane + 32, ...; k rounds of (warp arg-max on the biased score, lower index on ties)
constexpr int kMaxPerLane = 16;      // up to 512 experts
__global__ void __launch_bounds__(128) router_topk_bias_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias, int M,
                                                               int E, int top_k, int sigmoid_score, int normalize, float scaling,
                                                               int* __restrict__ ids, int ld_ids, float* __restrict__ wts, int ld_w) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= M) return;
  float score[kMaxPerLane], sel[kMaxPerLane];
  const float* lg = logits + (size_t)row * ld;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    score[i] = e < E ? lg[e] : -INFINITY;
    mx = fmaxf(mx, score[i]);
  }
  if (sigmoid_score) {
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) score[i] = (lane + 32 * i) < E ? 1.f / (1.f + __expf(-score[i])) : -INFINITY;
  } else {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      score[i] = (lane + 32 * i) < E ? __expf(score[i] - mx) : 0.f;
      sum += score[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) score[i] = (lane + 32 * i) < E ? score[i] / sum : -INFINITY;
  }
#pragma unroll
  for (int i = 0; i < kMaxPerLane; ++i) {
    const int e = lane + 32 * i;
    sel[i] = e < E ? score[i] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  float wsum = 0.f, my_w = 0.f;
  int my_id = 0;
  for (int j = 0; j < top_k; ++j) {
    float best = -INFINITY, bscore = 0.f;
    int bidx = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int e = lane + 32 * i;
      if (sel[i] > best || (sel[i] == best && e < bidx)) { best = sel[i]; bidx = e; bscore = score[i]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, bscore, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      if (ob > best || (ob == best && oi < bidx)) { best = ob; bidx = oi; bscore = os; }
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i)
      if (lane + 32 * i == bidx) sel[i] = -INFINITY;              // taken
    wsum += bscore;
    if (lane == j) { my_w = bscore; my_id = bidx; }
  }
  if (lane < top_k) {
    float w = my_w;
    if (normalize && wsum > 0.f) w /= wsum;
    ids[(size_t)row * ld_ids + lane] = my_id;
    wts[(size_t)row * ld_w + lane] = w * scaling;
  }
}

// out[row][d] = sum_j w[row][j] * silu(y[(row * k + j)][d]);  y fp32 [M * k][dim]
__global__ void mova_combine_kernel(const float* __restrict__ y, const float* __restrict__ w, int ld_w, bf16* __restrict__ out, int ldo, int M,
                                    int top_k, int dim) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)M * dim) return;
  const int row = (int)(i / dim), d = (int)(i - (long)row * dim);
  float acc = 0.f;
  for (int j = 0; j < top_k; ++j) {
    const float v = y[((size_t)row * top_k + j) * dim + d];
    acc = fmaf(w[(size_t)row * ld_w + j], v / (1.f + __expf(-v)), acc);
  }
  out[(size_t)row * ldo + d] = __float2bfloat16(acc);
}

}  // namespace

GRM_API int grm_rmsnorm_grouped(const void* h, int ldh, const void* w, void* out, int ldo, int M, int n, int n_groups, float eps, void* stream) {
  if (M < 1 || n < 1 || n_groups < 1 || n % n_groups) return -2;
  rmsnorm_grouped_kernel<<<M, 256, 0, (cudaStream_t)stream>>>((const float*)h, ldh, (const float*)w, (bf16*)out, ldo, n, n_groups, eps);
  GRM_LAUNCH_RET();
}

GRM_API int grm_softplus_gate(const void* attn, const void* gate, void* out, long n, float beta, void* stream) {
  if (n < 1 || beta <= 0.f) return -2;
  softplus_gate_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)attn, (const bf16*)gate, (bf16*)out, n, beta);
  GRM_LAUNCH_RET();
}

GRM_API int grm_router_topk_bias(const void* logits, int ld, const void* bias, int M, int E, int top_k, int sigmoid_score, int normalize,
                                 float scaling, void* ids, int ld_ids, void* wts, int ld_w, void* stream) {
  if (M < 1 || E < 1 || E > 32 * kMaxPerLane || top_k < 1 || top_k > 32 || top_k > E) return -2;
  const int threads = 128;
  router_topk_bias_kernel<<<(M * 32 + threads - 1) / threads, threads, 0, (cudaStream_t)stream>>>(
      (const float*)logits, ld, (const float*)bias, M, E, top_k, sigmoid_score, normalize, scaling, (int*)ids, ld_ids, (float*)wts, ld_w);
  GRM_LAUNCH_RET();
}

GRM_API int grm_mova_combine(const void* y, const void* w, int ld_w, void* out, int ldo, int M, int top_k, int dim, void* stream) {
  if (M < 1 || top_k < 1 || dim < 1) return -2;
  const long n = (long)M * dim;
  mova_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float*)y, (const float*)w, ld_w, (bf16*)out, ldo, M,
                                                                                      top_k, dim);
  GRM_LAUNCH_RET();
}
