// gemv_w4: Y[1][N] = X[1][K] . W[N][K]^T for int4 (group 64/128/256, fp16 scale, integer zero) weights in the tiled
// execution layout of formats/w4_tile_layout.py -- the single-row decode step, the reference's gemv_impl int4 row
// (src/gemv_decode.cpp:77-347).
//
// One batch row leaves 7/8 of an m16n8k16 MMA empty and the fragment dequantisation of the tensor-core kernel
// (smallm_w4.cu) costs ~5 instructions per weight, so a single row runs on the CUDA cores instead, at ~2 instructions
// per weight: a lane's 16-byte word group holds rows g and g + 8 of a 16-row tile for 16 consecutive k; one
// logic op per nibble pair builds the fp16 pair {1024 + q, 1024 + q'} (or {1024 + 16 q, ...} for the odd nibbles),
// one fp16x2 subtract / fma removes the bias and the zero point exactly, and one fp16x2 fma multiplies with the
// activations (converted to fp16 once per CTA into shared memory).  The fp16 partial sums of one quantisation group
// (16 or 32 products per accumulator half) are scaled and added into fp32.  A CTA owns one 16-row tile (SwiGLU: the
// gate tile and its up tile); its 8 warps split K and reduce through shared memory in a fixed order, so there is no
// cross-CTA reduction, no scratch and no atomics, and results are bit-reproducible.
//
// Overflow: a half accumulates up to 16 products of |q - zero| <= 16 per group, so the staged activations carry a fixed
// factor 2^-4 and saturate at +-240 (|x| = 3840; activations down to 1e-3 keep full fp16 precision): the fp16 sums
// stay below 16 * 16 * 240 < 65504 for every input, at no cost in the prologue (a data-dependent scale needs a pass over x before the staging; measured, that extra round
// trip costs every CTA about a microsecond, 10-15 % of these kernels).  The factor is undone in fp32.
// Also measured and not kept: a per-warp cp.async ring four groups deep instead of the register double buffer (more
// bytes in flight, 15 % slower), K split over two CTAs per tile for the narrow projections (no gain), nibbles read as
// fp16 subnormals with the zero point folded in per group (9 instead of 13 instructions per word, no faster, and the
// uncentred sums cost a digit of precision).
#include "common.cuh"

namespace {

constexpr int kGvWarps = 8;
constexpr float kGvXScale = 0.0625f;        // 2^-4 on the staged activations
constexpr float kGvXInv = 16.f;
constexpr float kGvXClamp = 240.f;          // saturation of the staged values

struct GemvW4Params {
  const uint4* w;         // tiles [N/32][K/64][2][32] x 16 bytes
  const uint32_t* sz;     // [N/16][G][16]: fp16 scale | bf16(128 + zero) << 16
  const bf16* x;          // [K]
  void* out;              // bf16 or fp32 [N] (SwiGLU: bf16 [N/2])
  int N, K, g64;
  // fused RMSNorm prologue (h != null): x = bf16(h * rsqrt(mean(h^2) + eps) * (offset + nw)) is computed by every CTA
  // from the fp32 residual row instead of being read
  const float* h;         // [K]
  const float* nw;        // [K]
  float eps, offset;
  // fused tensor-parallel all-reduce (EPI 4): out (fp32) += sum over ranks of the partial products.  Receive region
  // of a rank: {value, epoch} pairs [2 parity][world][tiles][16]; one epoch counter per tile (shared with smallm_w4.cu).
  float* ar_recv[8];
  unsigned int* ar_flags[8];
  unsigned int* ar_epochs;
  unsigned int* status;
  int ar_world, ar_rank;
  unsigned int ar_spin;
};

// One-shot all-reduce of a tile's 16 partial sums by warp 0, without fences: every partial sum travels as one 8-byte
// {value, epoch} store into the slot (parity, source rank, tile, row) of each peer's receive region; an aligned 8-byte
// store lands as a whole, so the receiver polls the slot itself until its epoch word is this launch's and then holds the
// value (the low-latency protocol of collective libraries).  The cost is one one-way NVLink latency instead of two
// system-scope fences plus a flag.  Partials are added in rank order, so every rank holds the same bits.  A peer can be at
// most one launch ahead (its next launch needs this rank's next push), hence the two parities.  out (fp32) += the sum.
template <typename P>
__device__ __forceinline__ void gemv_allreduce_tile(const P& p, float mine, int tile, int lane, float* out) {
  const int W = p.ar_world;
  const unsigned int e = p.ar_epochs[tile] + 1u;
  const size_t tiles = gridDim.x, par = e & 1u;
  bool ok = true;
  if (lane < 16) {
    const size_t slot = ((par * W + p.ar_rank) * tiles + tile) * 16 + lane;
    for (int r = 0; r < W; ++r) {
      if (r == p.ar_rank) continue;
      uint2* dst = reinterpret_cast<uint2*>(p.ar_recv[r]) + slot;
      asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(mine)), "r"(e) : "memory");
    }
    float s = 0.f;
    const uint2* base = reinterpret_cast<const uint2*>(p.ar_recv[p.ar_rank]);
    for (int r = 0; r < W; ++r) {
      if (r == p.ar_rank) { s += mine; continue; }
      const uint2* src = base + ((par * W + r) * tiles + tile) * 16 + lane;
      uint32_t vx = 0u, vy = 0u;
      bool got = false;
      for (unsigned int i = 0; i < p.ar_spin; ++i) {
        asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(vx), "=r"(vy) : "l"(src) : "memory");
        if (vy == e) { got = true; break; }
        if (i > 64) __nanosleep(20);
      }
      if (!got) { ok = false; grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x20000u | (r << 12) | (tile & 0xfff)); break; }
      s += __uint_as_float(vx);
    }
    if (ok) out[(size_t)tile * 16 + lane] += s;
  }
  __syncwarp();
  if (lane == 0) p.ar_epochs[tile] = e;   // advance even after a timeout so later launches stay aligned
}

__device__ __forceinline__ uint32_t lop3_or_and(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));   // (a & mask) | orv
  return r;
}
__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }

// 8 weights of one 32-bit word (rows g and g + 8, four consecutive k) times their activations
__device__ __forceinline__ void word_fma(uint32_t w, __half2 x01, __half2 x23, __half2 c_lo, __half2 c_hi, __half2& a0, __half2& a1) {
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  const uint32_t w2 = w >> 8;
  const __half2 l0 = as_h2(lop3_or_and(w, 0x000f000fu, 0x64006400u)), h0 = as_h2(lop3_or_and(w, 0x00f000f0u, 0x64006400u));
  const __half2 l1 = as_h2(lop3_or_and(w2, 0x000f000fu, 0x64006400u)), h1 = as_h2(lop3_or_and(w2, 0x00f000f0u, 0x64006400u));
  a0 = __hfma2(__hsub2(l0, c_lo), x01, a0);                    // row g,     k = 4j, 4j + 1
  a1 = __hfma2(__hfma2(h0, sixteenth, c_hi), x01, a1);         // row g + 8
  a0 = __hfma2(__hsub2(l1, c_lo), x23, a0);                    // row g,     k = 4j + 2, 4j + 3
  a1 = __hfma2(__hfma2(h1, sixteenth, c_hi), x23, a1);
}

// EPI: 0 bf16, 1 f32, 2 add_f32, 3 swiglu, 4 add_f32 after an all-reduce over ranks.  G64: k tiles per quantisation group.
template <int EPI, int G64>
__global__ void __launch_bounds__(kGvWarps * 32) gemv_w4_kernel(const GemvW4Params p) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  __half* xs = reinterpret_cast<__half*>(gv_smem);                       // [K] fp16 activations
  __shared__ float red[kGvWarps][16];
  constexpr bool SW = EPI == 3;
  constexpr int TILES = SW ? 2 : 1;               // 16-row tiles per CTA
  constexpr int SLICES = kGvWarps / TILES;        // K slices per tile
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int KT = p.K >> 6, G = KT / G64;
  const int tile = blockIdx.x * TILES + (SW ? warp / SLICES : 0);   // 16-row tile of this warp
  const int slice = SW ? warp % SLICES : warp;
  const int per = (G + SLICES - 1) / SLICES;
  const int gbeg = slice * per, gend = min(gbeg + per, G);
  const uint4* wp = p.w + ((size_t)(tile >> 1) * KT * 2 + (tile & 1)) * 32 + lane;   // + kt * 64
  const uint32_t* szp = p.sz + (size_t)tile * G * 16 + g;

  // first weights in flight before the activations are staged -- and, under a programmatic dependent launch, before the
  // kernel that produces the activations has finished: everything above and these loads touch only the weights
  grm_pdl_trigger();
  uint4 cur[G64];
  if (gbeg < gend) {
#pragma unroll
    for (int u = 0; u < G64; ++u) cur[u] = ldg_stream_v4(wp + (size_t)(gbeg * G64 + u) * 64);
  }
  grm_pdl_wait();
  // activations -> fp16 in shared memory.  Without SwiGLU every K slice belongs to one warp, which stages just its
  // own columns and needs no CTA barrier; the gate and up warps of a SwiGLU CTA share slices and stage together.
  float rnorm = 0.f;
  if (p.h != nullptr) {
    float ss = 0.f;
    for (int i = tid * 4; i < p.K; i += kGvWarps * 32 * 4) {
      const float4 a = *reinterpret_cast<const float4*>(p.h + i);
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp][0] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < kGvWarps; ++k) ss += red[k][0];
    rnorm = rsqrtf(ss / (float)p.K + p.eps);
    __syncthreads();                       // red is reused by the K-slice reduction below
  }
  const int xbeg = SW ? tid * 8 : gbeg * G64 * 64 + lane * 8;
  const int xend = SW ? p.K : min(gend * G64 * 64, p.K);
  const int xstep = SW ? kGvWarps * 32 * 8 : 256;
  for (int i = xbeg; i < xend; i += xstep) {
    uint32_t s[4];
    if (p.h != nullptr) {
      const float4 a = *reinterpret_cast<const float4*>(p.h + i), b = *reinterpret_cast<const float4*>(p.h + i + 4);
      const float4 wa = *reinterpret_cast<const float4*>(p.nw + i), wb = *reinterpret_cast<const float4*>(p.nw + i + 4);
      s[0] = pack_bf16x2(a.x * rnorm * (p.offset + wa.x), a.y * rnorm * (p.offset + wa.y));
      s[1] = pack_bf16x2(a.z * rnorm * (p.offset + wa.z), a.w * rnorm * (p.offset + wa.w));
      s[2] = pack_bf16x2(b.x * rnorm * (p.offset + wb.x), b.y * rnorm * (p.offset + wb.y));
      s[3] = pack_bf16x2(b.z * rnorm * (p.offset + wb.z), b.w * rnorm * (p.offset + wb.w));
    } else {
      const uint4 v = *reinterpret_cast<const uint4*>(p.x + i);
      s[0] = v.x; s[1] = v.y; s[2] = v.z; s[3] = v.w;
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 h = __floats2half2_rn(fminf(fmaxf(bf16lo_to_f(s[j]) * kGvXScale, -kGvXClamp), kGvXClamp),
                                          fminf(fmaxf(bf16hi_to_f(s[j]) * kGvXScale, -kGvXClamp), kGvXClamp));
      o[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(xs + i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (SW) __syncthreads();
  else __syncwarp();

  float f0 = 0.f, f1 = 0.f;
  for (int grp = gbeg; grp < gend; ++grp) {
    uint4 nxt[G64];
    if (grp + 1 < gend) {
#pragma unroll
      for (int u = 0; u < G64; ++u) nxt[u] = ldg_stream_v4(wp + (size_t)((grp + 1) * G64 + u) * 64);
    }
    const uint32_t s0 = __ldg(szp + (size_t)grp * 16), s1 = __ldg(szp + (size_t)grp * 16 + 8);
    const float z0 = bf16hi_to_f(s0) - 128.f, z1 = bf16hi_to_f(s1) - 128.f;
    const __half2 c_lo = __float2half2_rn(1024.f + z0), c_hi = __float2half2_rn(-(64.f + z1));
    __half2 a0 = __float2half2_rn(0.f), a1 = a0, b0 = a0, b1 = a0;
#pragma unroll
    for (int u = 0; u < G64; ++u) {
      const uint4* xp = reinterpret_cast<const uint4*>(xs + ((size_t)(grp * G64 + u) * 64 + t * 16));
      const uint4 xa = xp[0], xb = xp[1];
      word_fma(cur[u].x, as_h2(xa.x), as_h2(xa.y), c_lo, c_hi, a0, a1);
      word_fma(cur[u].y, as_h2(xa.z), as_h2(xa.w), c_lo, c_hi, b0, b1);
      word_fma(cur[u].z, as_h2(xb.x), as_h2(xb.y), c_lo, c_hi, a0, a1);
      word_fma(cur[u].w, as_h2(xb.z), as_h2(xb.w), c_lo, c_hi, b0, b1);
    }
    const float2 r0 = __half22float2(__hadd2(a0, b0)), r1 = __half22float2(__hadd2(a1, b1));
    f0 += __half2float(__ushort_as_half((unsigned short)(s0 & 0xffffu))) * (r0.x + r0.y);
    f1 += __half2float(__ushort_as_half((unsigned short)(s1 & 0xffffu))) * (r1.x + r1.y);
#pragma unroll
    for (int u = 0; u < G64; ++u) cur[u] = nxt[u];
  }
  // the four lanes of a row group hold disjoint k subsets
  f0 += __shfl_xor_sync(0xffffffffu, f0, 1); f0 += __shfl_xor_sync(0xffffffffu, f0, 2);
  f1 += __shfl_xor_sync(0xffffffffu, f1, 1); f1 += __shfl_xor_sync(0xffffffffu, f1, 2);
  if (t == 0) { red[warp][g] = f0 * kGvXInv; red[warp][g + 8] = f1 * kGvXInv; }
  __syncthreads();
  if (EPI == 4) {
    if (warp != 0) return;
    float mine = 0.f;
    if (lane < 16) {
#pragma unroll
      for (int k = 0; k < SLICES; ++k) mine += red[k][lane];
    }
    gemv_allreduce_tile(p, mine, tile, lane, reinterpret_cast<float*>(p.out));
    return;
  }
  if (tid < 16) {
    float s = 0.f, u = 0.f;
#pragma unroll
    for (int k = 0; k < SLICES; ++k) s += red[k][tid];
    if (SW) {
#pragma unroll
      for (int k = 0; k < SLICES; ++k) u += red[SLICES + k][tid];
    }
    const size_t col = (size_t)blockIdx.x * 16 + tid;
    if (EPI == 0) reinterpret_cast<bf16*>(p.out)[col] = __float2bfloat16(s);
    else if (EPI == 1) reinterpret_cast<float*>(p.out)[col] = s;
    else if (EPI == 2) reinterpret_cast<float*>(p.out)[col] += s;
    else reinterpret_cast<bf16*>(p.out)[col] = __float2bfloat16(silu_f(s) * u);
  }
}

// ---- MXFP4 (tile_mx layout: byte b = 2 hi + r8 of a lane's word j holds row g + 8 r8, columns 16 j + 2 t + 8 hi, +1;
// e8m0 scale bytes [N/16][K/32][16]) -------------------------------------------------------------------------------
__device__ __forceinline__ __half2 gv_e2m1x2(uint32_t byte) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b0;\n\t}" : "=r"(r) : "r"(byte));
  return as_h2(r);
}

struct GemvMxParams {
  const uint4* w;
  const uint8_t* sz;
  const bf16* x;
  void* out;
  int N, K;
  const float* h;
  const float* nw;
  float eps, offset;
  // EPI 4: fused tensor-parallel all-reduce, see gemv_allreduce_tile
  float* ar_recv[8];
  unsigned int* ar_epochs;
  unsigned int* status;
  int ar_world, ar_rank;
  unsigned int ar_spin;
};

template <int EPI>
__global__ void __launch_bounds__(256) gemv_mx_kernel(const GemvMxParams p) {
  extern __shared__ __align__(16) uint8_t gv_smem[];
  __half* xs = reinterpret_cast<__half*>(gv_smem);
  __shared__ float red[8][16];
  constexpr bool SW = EPI == 3;
  constexpr int TILES = SW ? 2 : 1;
  constexpr int SLICES = 8 / TILES;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int KT = p.K >> 6;
  const int tile = blockIdx.x * TILES + (SW ? warp / SLICES : 0);
  const int slice = SW ? warp % SLICES : warp;
  const int per = (KT + SLICES - 1) / SLICES;
  const int kbeg = slice * per, kend = min(kbeg + per, KT);
  const uint4* wp = p.w + ((size_t)(tile >> 1) * KT * 2 + (tile & 1)) * 32 + lane;   // + kt * 64
  const uint8_t* szp = p.sz + (size_t)tile * (KT * 2) * 16 + g;                        // + block * 16 (+ 8)

  uint4 cur = make_uint4(0u, 0u, 0u, 0u), nxt = cur;
  if (kbeg < kend) cur = ldg_stream_v4(wp + (size_t)kbeg * 64);
  if (kbeg + 1 < kend) nxt = ldg_stream_v4(wp + (size_t)(kbeg + 1) * 64);

  float rnorm = 0.f;
  if (p.h != nullptr) {
    float ss = 0.f;
    for (int i = tid * 4; i < p.K; i += 256 * 4) {
      const float4 a = *reinterpret_cast<const float4*>(p.h + i);
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
    ss = warp_sum(ss);
    if (lane == 0) red[warp][0] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += red[k][0];
    rnorm = rsqrtf(ss / (float)p.K + p.eps);
    __syncthreads();
  }
  const int xbeg = SW ? tid * 8 : kbeg * 64 + lane * 8;
  const int xend = SW ? p.K : min(kend * 64, p.K);
  const int xstep = SW ? 256 * 8 : 256;
  for (int i = xbeg; i < xend; i += xstep) {
    uint32_t s[4];
    if (p.h != nullptr) {
      const float4 a = *reinterpret_cast<const float4*>(p.h + i), b = *reinterpret_cast<const float4*>(p.h + i + 4);
      const float4 wa = *reinterpret_cast<const float4*>(p.nw + i), wb = *reinterpret_cast<const float4*>(p.nw + i + 4);
      s[0] = pack_bf16x2(a.x * rnorm * (p.offset + wa.x), a.y * rnorm * (p.offset + wa.y));
      s[1] = pack_bf16x2(a.z * rnorm * (p.offset + wa.z), a.w * rnorm * (p.offset + wa.w));
      s[2] = pack_bf16x2(b.x * rnorm * (p.offset + wb.x), b.y * rnorm * (p.offset + wb.y));
      s[3] = pack_bf16x2(b.z * rnorm * (p.offset + wb.z), b.w * rnorm * (p.offset + wb.w));
    } else {
      const uint4 v = *reinterpret_cast<const uint4*>(p.x + i);
      s[0] = v.x; s[1] = v.y; s[2] = v.z; s[3] = v.w;
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 hh = __floats2half2_rn(bf16lo_to_f(s[j]), bf16hi_to_f(s[j]));
      o[j] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    *reinterpret_cast<uint4*>(xs + i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  if (SW) __syncthreads();
  else __syncwarp();

  float f0 = 0.f, f1 = 0.f;
  for (int kt = kbeg; kt < kend; ++kt) {
    uint4 nx2 = make_uint4(0u, 0u, 0u, 0u);
    if (kt + 2 < kend) nx2 = ldg_stream_v4(wp + (size_t)(kt + 2) * 64);
    const uint32_t wv[4] = {cur.x, cur.y, cur.z, cur.w};
    const __half2* xk = reinterpret_cast<const __half2*>(xs + (size_t)kt * 64) + t;    // half2 index: (16 j + 2 t) / 2 = 8 j + t
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const int j = blk * 2 + jj;
        const uint32_t u = wv[j];
        const __half2 xlo = xk[8 * j], xhi = xk[8 * j + 4];
        a0 = __hfma2(gv_e2m1x2(u), xlo, a0);
        a1 = __hfma2(gv_e2m1x2(u >> 8), xlo, a1);
        a0 = __hfma2(gv_e2m1x2(u >> 16), xhi, a0);
        a1 = __hfma2(gv_e2m1x2(u >> 24), xhi, a1);
      }
      const uint8_t* sb = szp + (size_t)(kt * 2 + blk) * 16;
      const float s0 = __uint_as_float((uint32_t)__ldg(sb) << 23), s1 = __uint_as_float((uint32_t)__ldg(sb + 8) << 23);
      const float2 r0 = __half22float2(a0), r1 = __half22float2(a1);
      f0 += s0 * (r0.x + r0.y);
      f1 += s1 * (r1.x + r1.y);
    }
    cur = nxt; nxt = nx2;
  }
  f0 += __shfl_xor_sync(0xffffffffu, f0, 1); f0 += __shfl_xor_sync(0xffffffffu, f0, 2);
  f1 += __shfl_xor_sync(0xffffffffu, f1, 1); f1 += __shfl_xor_sync(0xffffffffu, f1, 2);
  if (t == 0) { red[warp][g] = f0; red[warp][g + 8] = f1; }
  __syncthreads();
  if (EPI == 4) {
    if (warp != 0) return;
    float mine = 0.f;
    if (lane < 16) {
#pragma unroll
      for (int k = 0; k < SLICES; ++k) mine += red[k][lane];
    }
    gemv_allreduce_tile(p, mine, (int)blockIdx.x, lane, reinterpret_cast<float*>(p.out));
    return;
  }
  if (tid < 16) {
    float s = 0.f, u = 0.f;
#pragma unroll
    for (int k = 0; k < SLICES; ++k) s += red[k][tid];
    if (SW) {
#pragma unroll
      for (int k = 0; k < SLICES; ++k) u += red[SLICES + k][tid];
    }
    const size_t col = (size_t)blockIdx.x * 16 + tid;
    if (EPI == 0) reinterpret_cast<bf16*>(p.out)[col] = __float2bfloat16(s);
    else if (EPI == 1) reinterpret_cast<float*>(p.out)[col] = s;
    else if (EPI == 2) reinterpret_cast<float*>(p.out)[col] += s;
    else reinterpret_cast<bf16*>(p.out)[col] = __float2bfloat16(silu_f(s) * u);
  }
}

template <int EPI>
int launch_epi(const GemvW4Params& p, cudaStream_t st) {
  const int tiles = p.N / 16;
  const unsigned grid = (unsigned)(EPI == 3 ? tiles / 2 : tiles);
  const size_t smem = (size_t)p.K * 2;
  if (EPI == 4) {
    // CTAs of different ranks wait for one another's pushes: the whole grid must be resident at once
    int per_sm = 0, dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t oe = cudaErrorInvalidValue;
    if (p.g64 == 1) oe = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_w4_kernel<EPI, 1>, kGvWarps * 32, smem);
    else if (p.g64 == 2) oe = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_w4_kernel<EPI, 2>, kGvWarps * 32, smem);
    else if (p.g64 == 4) oe = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_w4_kernel<EPI, 4>, kGvWarps * 32, smem);
    if (oe != cudaSuccess || (long)per_sm * sms < (long)grid) return -2;
  }
  cudaError_t e;
  switch (p.g64) {
    case 1: e = grm_launch_pdl(GRM_PDL_GEMV, gemv_w4_kernel<EPI, 1>, dim3(grid), dim3(kGvWarps * 32), smem, st, p); break;
    case 2: e = grm_launch_pdl(GRM_PDL_GEMV, gemv_w4_kernel<EPI, 2>, dim3(grid), dim3(kGvWarps * 32), smem, st, p); break;
    case 4: e = grm_launch_pdl(GRM_PDL_GEMV, gemv_w4_kernel<EPI, 4>, dim3(grid), dim3(kGvWarps * 32), smem, st, p); break;
    default: return -2;
  }
  if (e != cudaSuccess) return (int)e;
  GRM_LAUNCH_RET();
}

}  // namespace

// One activation row.  w / sz: the tiled int4 layout (N % 32 == 0, K % 64 == 0, K % group == 0, K <= 20480 so that the
// fp16 activations fit the default shared-memory window).  epi: 0 bf16, 1 f32, 2 add_f32, 3 swiglu (gate / up row tiles
// interleaved, out has N / 2 columns).  h != null: x is ignored and the activations are RMSNorm(h) with weight nw
// (fp32 [K] both), computed in the prologue.  Returns -2 on an unsupported shape.
GRM_API int grm_gemv_w4_norm(const void* w, const void* sz, const void* x, const void* h, const void* nw, float eps, float offset,
                             void* out, int N, int K, int group, int epi, void* stream) {
  if ((N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || K > 20480 || epi < 0 || epi > 3 ||
      (!h && ((uintptr_t)x & 15)) || (h && (!nw || ((uintptr_t)h & 15) || ((uintptr_t)nw & 15))))
    return -2;
  GemvW4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = (const bf16*)x; p.out = out;
  p.N = N; p.K = K; p.g64 = group / 64;
  p.h = (const float*)h; p.nw = (const float*)nw; p.eps = eps; p.offset = offset;
  for (int i = 0; i < 8; ++i) { p.ar_recv[i] = nullptr; p.ar_flags[i] = nullptr; }
  p.ar_epochs = nullptr; p.status = nullptr; p.ar_world = 1; p.ar_rank = 0; p.ar_spin = 0;
  cudaStream_t st = (cudaStream_t)stream;
  switch (epi) {
    case 0: return launch_epi<0>(p, st);
    case 1: return launch_epi<1>(p, st);
    case 2: return launch_epi<2>(p, st);
    default: return launch_epi<3>(p, st);
  }
}

GRM_API int grm_gemv_w4(const void* w, const void* sz, const void* x, void* out, int N, int K, int group, int epi, void* stream) {
  return grm_gemv_w4_norm(w, sz, x, nullptr, nullptr, 0.f, 0.f, out, N, K, group, epi, stream);
}

// Row-parallel projection of one activation row fused with the tensor-parallel all-reduce: h[N] (fp32) += sum over
// ranks of x_r . W_r^T.  recv / epochs: the exchange buffers of grm_smallm_w4_allreduce; this kernel uses the
// 2 * world * (N / 16) * 16 {value, epoch} pairs (8 bytes each) that start recv_off floats (a multiple of 2) into each
// rank's receive region, zero before first use -- a range the small-M kernel never touches, because a peer that is one
// launch ahead may already be writing the next launch's region while this rank still reads its own (epochs: N / 16
// uints, shared; flags are not used by this kernel).  Every rank issues the
// same sequence of fused calls.  spin = poll limit of the arrival wait (0 = default, ~0.1 s).  Returns -2 when the
// shape is unsupported or the grid could not be resident at once.
GRM_API int grm_gemv_w4_allreduce(const void* w, const void* sz, const void* x, void* h, int N, int K, int group,
                                  const void* const* recv, long recv_off, const void* const* flags, void* epochs, int world,
                                  int rank, unsigned int spin, void* stream) {
  if ((N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || K > 20480 || ((uintptr_t)x & 15))
    return -2;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !recv || !epochs || (recv_off & 1)) return -2;
  GemvW4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = (const bf16*)x; p.out = h;
  p.N = N; p.K = K; p.g64 = group / 64;
  p.h = nullptr; p.nw = nullptr; p.eps = 0.f; p.offset = 0.f;
  for (int i = 0; i < 8; ++i) {
    p.ar_recv[i] = i < world ? (float*)const_cast<void*>(recv[i]) + recv_off : nullptr;
    p.ar_flags[i] = (i < world && flags) ? (unsigned int*)const_cast<void*>(flags[i]) : nullptr;
  }
  p.ar_epochs = (unsigned int*)epochs; p.status = grm_status_ptr(); p.ar_world = world; p.ar_rank = rank;
  p.ar_spin = spin ? spin : 2000000u;
  return launch_epi<4>(p, (cudaStream_t)stream);
}

// MXFP4 weights in the tile_mx layout (formats/w4_tile_layout.py), one activation row; same epilogues and optional
// RMSNorm prologue as grm_gemv_w4_norm.  N % 32 == 0, K % 64 == 0, K <= 20480.
GRM_API int grm_gemv_mx(const void* w, const void* sz, const void* x, const void* h, const void* nw, float eps, float offset, void* out,
                        int N, int K, int epi, void* stream) {
  if ((N % 32) || (K % 64) || K > 20480 || epi < 0 || epi > 3 || (!h && ((uintptr_t)x & 15)) ||
      (h && (!nw || ((uintptr_t)h & 15) || ((uintptr_t)nw & 15))))
    return -2;
  GemvMxParams p;
  p.w = (const uint4*)w; p.sz = (const uint8_t*)sz; p.x = (const bf16*)x; p.out = out; p.N = N; p.K = K;
  p.h = (const float*)h; p.nw = (const float*)nw; p.eps = eps; p.offset = offset;
  cudaStream_t st = (cudaStream_t)stream;
  const int tiles = N / 16;
  const size_t smem = (size_t)K * 2;
  switch (epi) {
    case 0: gemv_mx_kernel<0><<<tiles, 256, smem, st>>>(p); break;
    case 1: gemv_mx_kernel<1><<<tiles, 256, smem, st>>>(p); break;
    case 2: gemv_mx_kernel<2><<<tiles, 256, smem, st>>>(p); break;
    default: gemv_mx_kernel<3><<<tiles / 2, 256, smem, st>>>(p); break;
  }
  GRM_LAUNCH_RET();
}

// Row-parallel MXFP4 projection of one activation row with the all-reduce over the tensor-parallel ranks in its epilogue:
// h (fp32 [N], replicated) += sum over ranks of x_rank . W_rank^T -- the MXFP4 counterpart of grm_gemv_w4_allreduce (same
// receive region layout and epoch counters, which the two kernels may share: launches are ordered on the stream).
GRM_API int grm_gemv_mx_allreduce(const void* w, const void* sz, const void* x, void* h, int N, int K, const void* const* recv,
                                  long recv_off, void* epochs, int world, int rank, unsigned int spin, void* stream) {
  if ((N % 32) || (K % 64) || K > 20480 || ((uintptr_t)x & 15)) return -2;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !recv || !epochs || (recv_off & 1)) return -2;
  GemvMxParams p;
  p.w = (const uint4*)w; p.sz = (const uint8_t*)sz; p.x = (const bf16*)x; p.out = h; p.N = N; p.K = K;
  p.h = nullptr; p.nw = nullptr; p.eps = 0.f; p.offset = 0.f;
  for (int i = 0; i < 8; ++i) p.ar_recv[i] = i < world ? (float*)const_cast<void*>(recv[i]) + recv_off : nullptr;
  p.ar_epochs = (unsigned int*)epochs; p.status = grm_status_ptr(); p.ar_world = world; p.ar_rank = rank;
  p.ar_spin = spin ? spin : 2000000u;
  const int tiles = N / 16;
  const size_t smem = (size_t)K * 2;
  // CTAs of different ranks wait for one another's pushes: the whole grid must be resident at once
  int per_sm = 0, dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemv_mx_kernel<4>, 256, smem) != cudaSuccess || (long)per_sm * sms < (long)tiles)
    return -2;
  gemv_mx_kernel<4><<<tiles, 256, smem, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}
