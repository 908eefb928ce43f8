// paged_decode_attn_i8kv: attention of M independent query rows over the pooled int8 KV cache.
// A row is (sequence, position): one decode token of some conversation, or one row of a
// speculative verify block (row r of a block sees keys 0..pos_r, which is the causal rule inside
// the block).  Covers the reference's launch_flash_decode* / _rows / _batched + launch_flash_merge*
// (src/attention.cpp:109-1547) and the verify-attention entry point (src/attn_verify.hpp:40-69).
//
// Design (bandwidth-bound, int8 K and V with one fp32 scale per token and kv head):
//   grid = (splits, kv heads, rows); the G = Hq/Hkv query heads of a group share every K/V byte;
//   a warp owns whole 16-token pages: QK with 2 lanes per token (D/2 dims each, 16-byte loads),
//   online softmax per warp, PV with lanes over D (coalesced 128-byte rows), probabilities passed
//   through warp-private shared memory with the V scale folded in;
//   the 4 warps merge in shared memory, split partials go to a scratch buffer and the last CTA to
//   arrive for a (row, kv head) merges the splits in split order (deterministic) and applies the
//   optional sigmoid output gate of gated attention.
#include "common.cuh"

namespace {

constexpr int kPage = 16;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxSplits = 64;

struct DecParams {
  const bf16* q; int ld_q;
  const int* row_seq; const int* row_pos;
  const int* block_table; int max_pages;
  const int8_t* k_pages; const int8_t* v_pages; const float* k_scale; const float* v_scale;
  const bf16* gate;           // [M][Hq*D] or null
  bf16* out; int ld_o;
  float* part_o;              // [M][Hkv][splits][G][D]
  float* part_ml;             // [M][Hkv][splits][G][2]
  unsigned int* counters;     // [M*Hkv]
  int M, Hq, Hkv, window;
  float scale;
};

template <int D, int G>
__global__ void __launch_bounds__(kThreads) decode_attn_kernel(const DecParams p) {
  constexpr int HD = D / 2;        // dims per lane in the QK phase
  constexpr int DPL = D / 32;      // dims per lane in the PV phase
  __shared__ float qs[G][D];
  __shared__ float ps[kWarps][G][kPage];
  __shared__ float sm_ml[kWarps][G][2];
  __shared__ float sm_o[kWarps][G][D];
  __shared__ int s_last;

  const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int nsplit = gridDim.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq = p.row_seq[row];
  const int len = p.row_pos[row] + 1;
  const int first = (p.window > 0 && len > p.window) ? (len - p.window) : 0;
  const int page_lo = first / kPage;
  const int page_hi = (len + kPage - 1) / kPage;       // exclusive
  const int npages = page_hi - page_lo;
  const int pps = (npages + nsplit - 1) / nsplit;
  const int pbeg = page_lo + split * pps;
  const int pend = min(pbeg + pps, page_hi);

  for (int i = tid; i < G * D; i += kThreads) {
    const int g = i / D, d = i % D;
    qs[g][d] = __bfloat162float(p.q[(size_t)row * p.ld_q + (size_t)(kvh * G + g) * D + d]) * p.scale;
  }
  __syncthreads();

  float m[G], l[G], o[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) o[g][d] = 0.f;
  }
  const int tok_in_page = lane >> 1, half = lane & 1;
  const int* bt = p.block_table + (size_t)seq * p.max_pages;

  // K of the first page is fetched before the loop; inside, the V rows of the current page and the K
  // rows of the next page are requested before the QK math so the loads overlap the arithmetic.
  uint4 kreg[HD / 16];
  float ksc = 0.f, vsc = 0.f;
  int pg = pbeg + warp;
  if (pg < pend) {
    const size_t pb = ((size_t)bt[pg] * p.Hkv + kvh) * kPage;
    const int8_t* kp = p.k_pages + (pb + tok_in_page) * D + half * HD;
#pragma unroll
    for (int c = 0; c < HD / 16; ++c) kreg[c] = *reinterpret_cast<const uint4*>(kp + c * 16);
    ksc = p.k_scale[pb + tok_in_page];
    vsc = p.v_scale[pb + tok_in_page];
  }
  for (; pg < pend; pg += kWarps) {
    const size_t pbase = ((size_t)bt[pg] * p.Hkv + kvh) * kPage;
    const int tok = pg * kPage + tok_in_page;
    const bool valid = tok < len && tok >= first;
    // V rows of this page (lane = 4 dims of every token row)
    const int8_t* vp = p.v_pages + pbase * D + lane * DPL;
    uint32_t vraw[kPage][(DPL + 3) / 4];
#pragma unroll
    for (int j = 0; j < kPage; ++j) {
      if (DPL == 4) vraw[j][0] = *reinterpret_cast<const uint32_t*>(vp + j * D);
      else if (DPL == 8) { const uint2 w8 = *reinterpret_cast<const uint2*>(vp + j * D); vraw[j][0] = w8.x; vraw[j][(DPL + 3) / 4 - 1] = w8.y; }
      else vraw[j][0] = *reinterpret_cast<const unsigned short*>(vp + j * D);
    }
    uint4 kcur[HD / 16];
#pragma unroll
    for (int c = 0; c < HD / 16; ++c) kcur[c] = kreg[c];
    const float ksc_c = ksc, vsc_c = vsc;
    if (pg + kWarps < pend) {
      const size_t pb = ((size_t)bt[pg + kWarps] * p.Hkv + kvh) * kPage;
      const int8_t* kp = p.k_pages + (pb + tok_in_page) * D + half * HD;
#pragma unroll
      for (int c = 0; c < HD / 16; ++c) kreg[c] = *reinterpret_cast<const uint4*>(kp + c * 16);
      ksc = p.k_scale[pb + tok_in_page];
      vsc = p.v_scale[pb + tok_in_page];
    }
    // ---- QK ----
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
#pragma unroll
    for (int c = 0; c < HD / 16; ++c) {
      const uint32_t wds[4] = {kcur[c].x, kcur[c].y, kcur[c].z, kcur[c].w};
#pragma unroll
      for (int wv = 0; wv < 4; ++wv) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const float kf = (float)(int8_t)((wds[wv] >> (8 * b)) & 0xff);
          const int d = half * HD + c * 16 + wv * 4 + b;
#pragma unroll
          for (int g = 0; g < G; ++g) s[g] = fmaf(kf, qs[g][d], s[g]);
        }
      }
    }
    float alpha[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sg = s[g] + __shfl_xor_sync(0xffffffffu, s[g], 1);
      sg = valid ? sg * ksc_c : -INFINITY;
      float mx = sg;
#pragma unroll
      for (int off = 2; off < 32; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float mnew = fmaxf(m[g], mx);
      alpha[g] = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mnew);
      const float pr = (sg == -INFINITY) ? 0.f : __expf(sg - mnew);
      m[g] = mnew;
      l[g] = l[g] * alpha[g] + (half == 0 ? pr : 0.f);
      if (half == 0) ps[warp][g][tok_in_page] = valid ? pr * vsc_c : 0.f;
    }
    __syncwarp();
    // ---- PV ----
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int d = 0; d < DPL; ++d) o[g][d] *= alpha[g];
#pragma unroll
    for (int j = 0; j < kPage; ++j) {
      float vf[DPL];
#pragma unroll
      for (int d = 0; d < DPL; ++d) vf[d] = (float)(int8_t)((vraw[j][d >> 2] >> (8 * (d & 3))) & 0xff);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pj = ps[warp][g][j];
#pragma unroll
        for (int d = 0; d < DPL; ++d) o[g][d] = fmaf(pj, vf[d], o[g][d]);
      }
    }
    __syncwarp();
  }

  // ---- merge the 4 warps ----
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const float lg = warp_sum(l[g]);
    if (lane == 0) { sm_ml[warp][g][0] = m[g]; sm_ml[warp][g][1] = lg; }
#pragma unroll
    for (int d = 0; d < DPL; ++d) sm_o[warp][g][lane * DPL + d] = o[g][d];
  }
  __syncthreads();

  const size_t pidx = ((size_t)row * p.Hkv + kvh) * nsplit + split;
  for (int i = tid; i < G * D; i += kThreads) {
    const int g = i / D, d = i % D;
    float M_ = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M_ = fmaxf(M_, sm_ml[w][g][0]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = sm_ml[w][g][0];
      const float f = (mw == -INFINITY) ? 0.f : __expf(mw - M_);
      L += sm_ml[w][g][1] * f;
      O += sm_o[w][g][d] * f;
    }
    if (nsplit == 1) {
      float r = L > 0.f ? O / L : 0.f;
      const size_t oi = (size_t)row * p.ld_o + (size_t)(kvh * G + g) * D + d;
      if (p.gate) r *= sigmoid_f(__bfloat162float(p.gate[oi]));
      p.out[oi] = __float2bfloat16(r);
    } else {
      p.part_o[(pidx * G + g) * D + d] = O;
      if (d == 0) { p.part_ml[(pidx * G + g) * 2] = M_; p.part_ml[(pidx * G + g) * 2 + 1] = L; }
    }
  }
  if (nsplit == 1) return;

  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int prev = atomicAdd(&p.counters[row * p.Hkv + kvh], 1u);
    s_last = (prev == (unsigned int)nsplit - 1u);
    if (s_last) p.counters[row * p.Hkv + kvh] = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Last CTA of this (row, kv head): merge the splits in split order.  The per-split (max, sum) pairs
  // are staged in shared memory first so the long loop only carries independent loads.
  const size_t base = ((size_t)row * p.Hkv + kvh) * nsplit;
  float* wts = &sm_o[0][0][0];            // reuse: [G][kMaxSplits] weights
  for (int i = tid; i < G * nsplit; i += kThreads) {
    const int g = i / nsplit, sp = i % nsplit;
    wts[g * kMaxSplits + sp] = __ldcg(&p.part_ml[((base + sp) * G + g) * 2]);
  }
  __syncthreads();
  if (tid < G) {
    float M_ = -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) M_ = fmaxf(M_, wts[tid * kMaxSplits + sp]);
    float L = 0.f;
    for (int sp = 0; sp < nsplit; ++sp) {
      const float ms = wts[tid * kMaxSplits + sp];
      const float f = (ms == -INFINITY) ? 0.f : __expf(ms - M_);
      wts[tid * kMaxSplits + sp] = f;
      L += __ldcg(&p.part_ml[((base + sp) * G + tid) * 2 + 1]) * f;
    }
    sm_ml[0][tid][0] = L;
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += kThreads) {
    const int g = i / D, d = i % D;
    float O = 0.f;
#pragma unroll 8
    for (int sp = 0; sp < nsplit; ++sp) O = fmaf(__ldcg(&p.part_o[((base + sp) * G + g) * D + d]), wts[g * kMaxSplits + sp], O);
    const float L = sm_ml[0][g][0];
    float r = L > 0.f ? O / L : 0.f;
    const size_t oi = (size_t)row * p.ld_o + (size_t)(kvh * G + g) * D + d;
    if (p.gate) r *= sigmoid_f(__bfloat162float(p.gate[oi]));
    p.out[oi] = __float2bfloat16(r);
  }
}

template <int D, int G>
int launch(const DecParams& p, int splits, cudaStream_t st) {
  dim3 grid(splits, p.Hkv, p.M);
  decode_attn_kernel<D, G><<<grid, kThreads, 0, st>>>(p);
  GRM_LAUNCH_RET();
}

template <int D>
int launch_g(const DecParams& p, int G, int splits, cudaStream_t st) {
  switch (G) {
    case 1: return launch<D, 1>(p, splits, st);
    case 2: return launch<D, 2>(p, splits, st);
    case 4: return launch<D, 4>(p, splits, st);
    case 5: return launch<D, 5>(p, splits, st);
    case 6: return launch<D, 6>(p, splits, st);
    case 8: return launch<D, 8>(p, splits, st);
    default: return -2;
  }
}

}  // namespace

// part_o: fp32 M*Hq*splits*D, part_ml: fp32 M*Hq*splits*2, counters: M*Hkv zeroed uints (only read
// when splits > 1).  window <= 0 disables the sliding window.
GRM_API int grm_paged_decode_attn(const void* q, int ld_q, const void* row_seq, const void* row_pos, const void* block_table,
                                  int max_pages, const void* k_pages, const void* v_pages, const void* k_scale,
                                  const void* v_scale, const void* gate, void* out, int ld_o, void* part_o, void* part_ml,
                                  void* counters, int M, int Hq, int Hkv, int D, int splits, int window, float scale,
                                  void* stream) {
  if (M < 1 || Hkv < 1 || Hq % Hkv || splits < 1 || splits > kMaxSplits) return -2;
  if (splits > 1 && (!part_o || !part_ml || !counters)) return -2;
  DecParams p;
  p.q = (const bf16*)q; p.ld_q = ld_q; p.row_seq = (const int*)row_seq; p.row_pos = (const int*)row_pos;
  p.block_table = (const int*)block_table; p.max_pages = max_pages;
  p.k_pages = (const int8_t*)k_pages; p.v_pages = (const int8_t*)v_pages; p.k_scale = (const float*)k_scale; p.v_scale = (const float*)v_scale;
  p.gate = (const bf16*)gate; p.out = (bf16*)out; p.ld_o = ld_o; p.part_o = (float*)part_o; p.part_ml = (float*)part_ml;
  p.counters = (unsigned int*)counters; p.M = M; p.Hq = Hq; p.Hkv = Hkv; p.window = window; p.scale = scale;
  cudaStream_t st = (cudaStream_t)stream;
  const int G = Hq / Hkv;
  switch (D) {
    case 64: return launch_g<64>(p, G, splits, st);
    case 128: return launch_g<128>(p, G, splits, st);
    case 256: return launch_g<256>(p, G, splits, st);
    default: return -2;
  }
}
