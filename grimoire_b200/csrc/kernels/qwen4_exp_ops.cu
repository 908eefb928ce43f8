// Operators of the Qwen4-Exp family (reference kernels: launch_hc_* src/ops.cpp:2352-3011, launch_qsa_* :3013-3440 with
// flash_decode_qsa_list src/attention.cpp:511, launch_ple_* src/ops.cpp:3441-3630; host oracle include/b70/qwen4_exp.hpp):
//   HyperConnections  per-stream (1 + w) RMSNorm of the [hc * H] residual, the gated mean that collapses the streams into a
//                     block input, and the gated injection of a block output into every stream;
//   QSA               indexer logits over pooled key blocks (relu per head, then the sum over heads, then 1 / sqrt(d)),
//                     block list -> token list with the unconditional tail, attention over a gathered token list;
//   PLE               the per-stream gate of the n-gram value row and the dilated depthwise convolution that finishes the layer.
// The small projections between these pieces (low-rank down / up, injection, indexer q) are ordinary linears.
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + __expf(-x)); }

// block-wide sum over 256 threads (all threads get the result)
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}

// grid (rows, hc): normed = x * rsqrt(mean(x^2) + eps) * (1 + w) per stream; fp32 and bf16 copies
__global__ void __launch_bounds__(256) hc_norm_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ out_f,
                                                      bf16* __restrict__ out_b, int H, int hc, float eps) {
  __shared__ float red[8];
  const int row = blockIdx.x, c = blockIdx.y, tid = threadIdx.x;
  const size_t base = ((size_t)row * hc + c) * H;
  float ss = 0.f;
  for (int i = tid; i < H; i += 256) { const float v = x[base + i]; ss = fmaf(v, v, ss); }
  const float inv = rsqrtf(block_sum_256(ss, red) / (float)H + eps);
  for (int i = tid; i < H; i += 256) {
    const float y = x[base + i] * inv * (1.f + w[(size_t)c * H + i]);
    out_f[base + i] = y;
    if (out_b) out_b[base + i] = __float2bfloat16(y);
  }
}

// g = silu(x / hc) in place -> bf16 (the low-rank gate between the down and the up projection)
__global__ void hc_lowrank_gate_kernel(const float* __restrict__ x, bf16* __restrict__ out, long n, float inv_hc) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(siluf_(x[i] * inv_hc));
}

// out[row][h] = mean_c sigmoid(u[row][c][h]) * normed[row][c][h]
__global__ void hc_mix_finish_kernel(const float* __restrict__ u, const float* __restrict__ normed, bf16* __restrict__ out_b, float* __restrict__ out_f,
                                     int rows, int H, int hc) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)rows * H) return;
  const int row = (int)(i / H), h = (int)(i - (long)row * H);
  float acc = 0.f;
  for (int c = 0; c < hc; ++c) {
    const size_t o = ((size_t)row * hc + c) * H + h;
    acc = fmaf(sigmoidf_(u[o]), normed[o], acc);
  }
  acc /= (float)hc;
  if (out_b) out_b[i] = __float2bfloat16(acc);
  if (out_f) out_f[i] = acc;
}

// hyper[row][c][h] += block[row][h] * 2 sigmoid(inj[row][c] / hc)   (in place on the unnormalised streams)
__global__ void hc_combine_kernel(float* __restrict__ hyper, const float* __restrict__ block, const float* __restrict__ inj, int ld_inj, int rows,
                                  int H, int hc) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)rows * hc * H) return;
  const int h = (int)(i % H);
  const long rc = i / H;
  const int c = (int)(rc % hc), row = (int)(rc / hc);
  hyper[i] += block[(size_t)row * H + h] * 2.f * sigmoidf_(inj[(size_t)row * ld_inj + c] / (float)hc);
}

// one warp per (row, block): logits = sum_heads relu(q_h . key) / sqrt(d); -inf from visible[row] on
__global__ void __launch_bounds__(128) qsa_index_logits_kernel(const bf16* __restrict__ q, const bf16* __restrict__ keys, const int* __restrict__ visible,
                                                               float* __restrict__ logits, int rows, int heads, int d, int blocks) {
  const long wid = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= (long)rows * blocks) return;
  const int row = (int)(wid / blocks), n = (int)(wid - (long)row * blocks);
  if (n >= visible[row]) { if (lane == 0) logits[wid] = -INFINITY; return; }
  const bf16* kn = keys + (size_t)n * d;
  float acc = 0.f;
  for (int h = 0; h < heads; ++h) {
    const bf16* qh = q + ((size_t)row * heads + h) * d;
    float dot = 0.f;
    for (int i = lane; i < d; i += 32) dot = fmaf(__bfloat162float(qh[i]), __bfloat162float(kn[i]), dot);
    dot = warp_sum(dot);
    acc += fmaxf(dot, 0.f);                                   // relu per head, then the sum
  }
  if (lane == 0) logits[wid] = acc * rsqrtf((float)d);
}

// one thread per output slot: block list -> token list (budget slots, then the ratio - 1 tail slots)
__global__ void qsa_expand_kernel(const int* __restrict__ blk, int block_topk, int ratio, int token_topk, const int* __restrict__ seq_len,
                                  const int* __restrict__ query_pos, int* __restrict__ out, int rows) {
  const int width = token_topk + ratio - 1;
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)rows * width) return;
  const int row = (int)(i / width), s = (int)(i - (long)row * width);
  const int sl = seq_len[row];
  int t = -1;
  if (s < token_topk) {
    const int b = s / ratio;
    if (b < block_topk) {
      const int bi = blk[(size_t)row * block_topk + b];
      if (bi >= 0) t = bi * ratio + (s - b * ratio);
    }
  } else {
    const int j = s - token_topk, vis = query_pos[row] + 1, tail0 = vis / ratio * ratio;
    if (j < vis - tail0) t = tail0 + j;
  }
  out[i] = (t >= 0 && t < sl) ? t : -1;
}

// Attention of one query row over a gathered token list.  grid (rows, heads), 128 threads: a warp walks every fourth list
// entry with an online softmax (a lane holds d / 32 of the head dimension, d <= 256), the four warps merge through shared
// memory.  k, v: bf16 [kv_heads][cap][d]; idx [rows][n_idx] with -1 holes.
__global__ void __launch_bounds__(128) qsa_gather_attn_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                                                              const int* __restrict__ idx, bf16* __restrict__ out, int heads, int kv_heads, int d,
                                                              int cap, int n_idx, float scale) {
  __shared__ float s_m[4], s_l[4], s_acc[4][256];
  const int row = blockIdx.x, h = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kvh = h / (heads / kv_heads), per = d >> 5;
  const bf16* qh = q + ((size_t)row * heads + h) * d;
  float qv[8], acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { qv[i] = i < per ? __bfloat162float(qh[lane + 32 * i]) * scale : 0.f; acc[i] = 0.f; }
  float m = -INFINITY, l = 0.f;
  for (int e = warp; e < n_idx; e += 4) {
    const int t = idx[(size_t)row * n_idx + e];
    if (t < 0) continue;                                      // warp-uniform
    const bf16* kk = k + ((size_t)kvh * cap + t) * d;
    const bf16* vv = v + ((size_t)kvh * cap + t) * d;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < per) dot = fmaf(qv[i], __bfloat162float(kk[lane + 32 * i]), dot);
    dot = warp_sum(dot);
    const float mn = fmaxf(m, dot), a = __expf(m - mn), p = __expf(dot - mn);
    l = l * a + p;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < per) acc[i] = acc[i] * a + p * __bfloat162float(vv[lane + 32 * i]);
    m = mn;
  }
  if (lane == 0) { s_m[warp] = m; s_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (i < per) s_acc[warp][lane + 32 * i] = acc[i];
  __syncthreads();
  if (warp == 0) {
    const float M4 = fmaxf(fmaxf(s_m[0], s_m[1]), fmaxf(s_m[2], s_m[3]));
    float L = 0.f, w4[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) { w4[j] = s_m[j] == -INFINITY ? 0.f : __expf(s_m[j] - M4); L += s_l[j] * w4[j]; }
    const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < per) {
        const int c = lane + 32 * i;
        const float o = (s_acc[0][c] * w4[0] + s_acc[1][c] * w4[1] + s_acc[2][c] * w4[2] + s_acc[3][c] * w4[3]) * inv;
        out[((size_t)row * heads + h) * d + c] = __float2bfloat16(o);
      }
  }
}

// grid (rows, hc): d = <norm_k(key), norm_q(query)> / sqrt(H); g = sigmoid(sign(d) sqrt(max(|d|, 1e-6))); gated = g * value;
// conv_in = norm_c(gated).  All norms are (1 + w) with weights over the whole hc * H row.
__global__ void __launch_bounds__(256) ple_gate_kernel(const float* __restrict__ key, const float* __restrict__ value, const float* __restrict__ query,
                                                       const float* __restrict__ nk, const float* __restrict__ nq, const float* __restrict__ ncw,
                                                       float* __restrict__ gated, float* __restrict__ conv_in, int H, int hc, float eps) {
  __shared__ float red[8];
  const int row = blockIdx.x, c = blockIdx.y, tid = threadIdx.x;
  const size_t base = ((size_t)row * hc + c) * H, wb = (size_t)c * H;
  float ks = 0.f, qs = 0.f;
  for (int i = tid; i < H; i += 256) { const float a = key[base + i], b = query[base + i]; ks = fmaf(a, a, ks); qs = fmaf(b, b, qs); }
  const float ki = rsqrtf(block_sum_256(ks, red) / (float)H + eps);
  const float qi = rsqrtf(block_sum_256(qs, red) / (float)H + eps);
  float dot = 0.f;
  for (int i = tid; i < H; i += 256) dot = fmaf(key[base + i] * ki * (1.f + nk[wb + i]), query[base + i] * qi * (1.f + nq[wb + i]), dot);
  const float dd = block_sum_256(dot, red) * rsqrtf((float)H);
  const float g = sigmoidf_((dd < 0.f ? -1.f : 1.f) * sqrtf(fmaxf(fabsf(dd), 1e-6f)));
  float gs = 0.f;
  for (int i = tid; i < H; i += 256) { const float y = g * value[(size_t)row * H + i]; gated[base + i] = y; gs = fmaf(y, y, gs); }
  const float gi = rsqrtf(block_sum_256(gs, red) / (float)H + eps);
  for (int i = tid; i < H; i += 256) conv_in[base + i] = g * value[(size_t)row * H + i] * gi * (1.f + ncw[wb + i]);
}

// out[t][c] = hidden[t][c] + gated[t][c] + silu(sum_k w[c][k] * conv_in[t0 + t - (K - 1 - k) * dil][c]); conv_in holds t0 rows of
// history in front of the T new rows (rows before the start of the sequence read zero)
__global__ void ple_conv_kernel(const float* __restrict__ conv_in, const float* __restrict__ gated, const float* __restrict__ hidden,
                                const float* __restrict__ w, float* __restrict__ out, int T, int t0, int C, int Kn, int dil) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)T * C) return;
  const int t = (int)(i / C), c = (int)(i - (long)t * C);
  float acc = 0.f;
  for (int k = 0; k < Kn; ++k) {
    const int at = t0 + t - (Kn - 1 - k) * dil;
    if (at >= 0) acc = fmaf(w[(size_t)c * Kn + k], conv_in[(size_t)at * C + c], acc);
  }
  out[i] = hidden[i] + gated[i] + siluf_(acc);
}

inline unsigned grid1(long n) { return (unsigned)((n + 255) / 256); }

}  // namespace

GRM_API int grm_hc_norm(const void* x, const void* w, void* out_f, void* out_b, int rows, int H, int hc, float eps, void* stream) {
  if (rows < 1 || H < 1 || hc < 1) return -2;
  hc_norm_kernel<<<dim3(rows, hc), 256, 0, (cudaStream_t)stream>>>((const float*)x, (const float*)w, (float*)out_f, (bf16*)out_b, H, hc, eps);
  GRM_LAUNCH_RET();
}
GRM_API int grm_hc_lowrank_gate(const void* x, void* out, long n, int hc, void* stream) {
  if (n < 1 || hc < 1) return -2;
  hc_lowrank_gate_kernel<<<grid1(n), 256, 0, (cudaStream_t)stream>>>((const float*)x, (bf16*)out, n, 1.f / (float)hc);
  GRM_LAUNCH_RET();
}
GRM_API int grm_hc_mix_finish(const void* u, const void* normed, void* out_b, void* out_f, int rows, int H, int hc, void* stream) {
  if (rows < 1 || H < 1 || hc < 1) return -2;
  hc_mix_finish_kernel<<<grid1((long)rows * H), 256, 0, (cudaStream_t)stream>>>((const float*)u, (const float*)normed, (bf16*)out_b, (float*)out_f,
                                                                               rows, H, hc);
  GRM_LAUNCH_RET();
}
GRM_API int grm_hc_combine(void* hyper, const void* block, const void* inj, int ld_inj, int rows, int H, int hc, void* stream) {
  if (rows < 1 || H < 1 || hc < 1) return -2;
  hc_combine_kernel<<<grid1((long)rows * hc * H), 256, 0, (cudaStream_t)stream>>>((float*)hyper, (const float*)block, (const float*)inj, ld_inj,
                                                                                 rows, H, hc);
  GRM_LAUNCH_RET();
}
GRM_API int grm_qsa_index_logits(const void* q, const void* keys, const void* visible, void* logits, int rows, int heads, int d, int blocks,
                                 void* stream) {
  if (rows < 1 || heads < 1 || d < 1 || blocks < 1) return -2;
  const long warps = (long)rows * blocks;
  qsa_index_logits_kernel<<<(unsigned)((warps * 32 + 127) / 128), 128, 0, (cudaStream_t)stream>>>((const bf16*)q, (const bf16*)keys, (const int*)visible,
                                                                                                   (float*)logits, rows, heads, d, blocks);
  GRM_LAUNCH_RET();
}
GRM_API int grm_qsa_expand(const void* blk, int block_topk, int ratio, int token_topk, const void* seq_len, const void* query_pos, void* out,
                           int rows, void* stream) {
  if (rows < 1 || block_topk < 1 || ratio < 1 || token_topk < 1) return -2;
  qsa_expand_kernel<<<grid1((long)rows * (token_topk + ratio - 1)), 256, 0, (cudaStream_t)stream>>>((const int*)blk, block_topk, ratio, token_topk,
                                                                                                   (const int*)seq_len, (const int*)query_pos,
                                                                                                   (int*)out, rows);
  GRM_LAUNCH_RET();
}
GRM_API int grm_qsa_gather_attn(const void* q, const void* k, const void* v, const void* idx, void* out, int rows, int heads, int kv_heads, int d,
                                int cap, int n_idx, float scale, void* stream) {
  if (rows < 1 || heads < 1 || kv_heads < 1 || heads % kv_heads || (d & 31) || d > 256 || n_idx < 1) return -2;
  qsa_gather_attn_kernel<<<dim3(rows, heads), 128, 0, (cudaStream_t)stream>>>((const bf16*)q, (const bf16*)k, (const bf16*)v, (const int*)idx,
                                                                             (bf16*)out, heads, kv_heads, d, cap, n_idx, scale);
  GRM_LAUNCH_RET();
}
GRM_API int grm_ple_gate(const void* key, const void* value, const void* query, const void* nk, const void* nq, const void* ncw, void* gated,
                         void* conv_in, int rows, int H, int hc, float eps, void* stream) {
  if (rows < 1 || H < 1 || hc < 1) return -2;
  ple_gate_kernel<<<dim3(rows, hc), 256, 0, (cudaStream_t)stream>>>((const float*)key, (const float*)value, (const float*)query, (const float*)nk,
                                                                    (const float*)nq, (const float*)ncw, (float*)gated, (float*)conv_in, H, hc, eps);
  GRM_LAUNCH_RET();
}
GRM_API int grm_ple_conv(const void* conv_in, const void* gated, const void* hidden, const void* w, void* out, int T, int t0, int C, int Kn, int dil,
                         void* stream) {
  if (T < 1 || t0 < 0 || C < 1 || Kn < 1 || dil < 1) return -2;
  ple_conv_kernel<<<grid1((long)T * C), 256, 0, (cudaStream_t)stream>>>((const float*)conv_in, (const float*)gated, (const float*)hidden,
                                                                       (const float*)w, (float*)out, T, t0, C, Kn, dil);
  GRM_LAUNCH_RET();
}
