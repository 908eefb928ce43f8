// smallm_mx: y[M][N] = x[M][K] . W^T for 1..8 rows with MXFP4 weights (OCP MX: e2m1 elements in blocks
// of 32 along K sharing one e8m0 scale), the decode / verify-rows projection of the MXFP4 model.
// Covers the reference's MXFP4 decode GEMV family (launch_gemv_mxfp4*, src/kernels.hpp:163-169 quotes
// 345 GB/s = 57 % of its card's bandwidth for it).
//
// Weights stay in the checkpoint's natural layout ([N][K/2] bytes, even k in the low nibble, scales
// [N][K/32]); nothing is re-tiled at load.  A warp owns 16 weight rows (for SwiGLU: 16 gate rows and
// the matching 16 up rows) and a K slice; rows of the batch sit in the MMA N dimension, so one to
// eight rows cost one pass over the weights:
//   * every lane of a quad loads the same 16-byte block of its weight row (one MX block, a broadcast
//     load), picks the two bytes its A fragment needs with a byte permute and expands them with the
//     hardware e2m1x2 -> f16x2 conversion;
//   * the activations are pre-converted to f16 once per call (x16) and read as B fragments;
//   * the two m16n8k16 MMAs of a block accumulate into a scratch fragment that is folded into the
//     fp32 accumulator with the block's e8m0 scale, so the scale never touches f16 range;
//   * the K slices of a CTA's warps are summed in shared memory in warp order (deterministic).
#include "common.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
enum { MX_BF16 = 0, MX_F32 = 1, MX_ADD_F32 = 2, MX_SWIGLU = 3 };

struct MxParams {
  const uint8_t* w;      // [N][K/2]
  const uint8_t* s;      // [N][K/32] e8m0
  const __half* x16;     // [M][ldx] f16
  void* out; int ldo;
  int M, N, K, ldx, epi;
  int rt, ks;            // row tiles per CTA, K slices per CTA (rt * ks == kWarps)
};

__device__ __forceinline__ uint32_t cvt_e2m1x2(uint32_t byte) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b0;\n\t}" : "=r"(r) : "r"(byte));
  return r;
}
__device__ __forceinline__ uint32_t prmt_(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float e8m0_f(uint32_t e) { return e == 0u ? 5.877471754111438e-39f : __uint_as_float(e << 23); }

template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads) smallm_mx_kernel(const MxParams p) {
  constexpr int NB = SWIGLU ? 2 : 1;
  __shared__ float red[kWarps][NB][4][32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int wr = warp / p.ks, wk = warp - wr * p.ks;            // row tile and K slice of this warp
  const int NO = SWIGLU ? p.N / 2 : p.N;                        // output columns
  const int row0 = (blockIdx.x * p.rt + wr) * 16;               // first output column (= weight row) of the tile
  const int nblk = p.K / 32;
  const int b_lo = (int)(((long long)nblk * wk) / p.ks), b_hi = (int)(((long long)nblk * (wk + 1)) / p.ks);
  const bool live = row0 < NO;
  float acc[NB][4];
#pragma unroll
  for (int b = 0; b < NB; ++b) { acc[b][0] = 0.f; acc[b][1] = 0.f; acc[b][2] = 0.f; acc[b][3] = 0.f; }
  if (live) {
    // byte t and byte 4+t of each 8-byte half block feed the k slots (2t, 2t+1) and (2t+8, 2t+9)
    const uint32_t sel = (uint32_t)t | ((uint32_t)(4 + t) << 4);
    const uint8_t* wrow[NB][2];
    const uint8_t* srow[NB][2];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      // SwiGLU weights are stored gate/up interleaved per 16 rows: output tile i = rows [32i, 32i+16) gate, [32i+16, 32i+32) up
      const int ra = SWIGLU ? 2 * row0 + 16 * b + g : min(row0 + g, NO - 1);
      const int rb = SWIGLU ? ra + 8 : min(row0 + g + 8, NO - 1);
      wrow[b][0] = p.w + (size_t)ra * (p.K / 2); wrow[b][1] = p.w + (size_t)rb * (p.K / 2);
      srow[b][0] = p.s + (size_t)ra * nblk;      srow[b][1] = p.s + (size_t)rb * nblk;
    }
    const __half* xr = p.x16 + (size_t)min(g, p.M - 1) * p.ldx;
    const bool has_x = g < p.M;
#pragma unroll 4
    for (int blk = b_lo; blk < b_hi; ++blk) {
      uint4 wv[NB][2];
      uint32_t sc[NB][2];
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          wv[b][h] = ldg_stream_v4(wrow[b][h] + (size_t)blk * 16);
          sc[b][h] = srow[b][h][blk];
        }
      uint32_t xb[2][2] = {{0u, 0u}, {0u, 0u}};
      if (has_x) {
        const uint32_t* xp = reinterpret_cast<const uint32_t*>(xr + (size_t)blk * 32);
        xb[0][0] = xp[t]; xb[0][1] = xp[4 + t]; xb[1][0] = xp[8 + t]; xb[1][1] = xp[12 + t];
      }
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        float part[4] = {0.f, 0.f, 0.f, 0.f};
        // step 0: k 0..15 of the block = words x, y; step 1: k 16..31 = words z, w
        {
          const uint32_t pa = prmt_(wv[b][0].x, wv[b][0].y, sel), pb = prmt_(wv[b][1].x, wv[b][1].y, sel);
          mma_f16(part, cvt_e2m1x2(pa), cvt_e2m1x2(pb), cvt_e2m1x2(pa >> 8), cvt_e2m1x2(pb >> 8), xb[0][0], xb[0][1]);
        }
        {
          const uint32_t pa = prmt_(wv[b][0].z, wv[b][0].w, sel), pb = prmt_(wv[b][1].z, wv[b][1].w, sel);
          mma_f16(part, cvt_e2m1x2(pa), cvt_e2m1x2(pb), cvt_e2m1x2(pa >> 8), cvt_e2m1x2(pb >> 8), xb[1][0], xb[1][1]);
        }
        const float s0 = e8m0_f(sc[b][0]), s1 = e8m0_f(sc[b][1]);
        acc[b][0] = fmaf(s0, part[0], acc[b][0]); acc[b][1] = fmaf(s0, part[1], acc[b][1]);
        acc[b][2] = fmaf(s1, part[2], acc[b][2]); acc[b][3] = fmaf(s1, part[3], acc[b][3]);
      }
    }
  }
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int c = 0; c < 4; ++c) red[warp][b][c][lane] = acc[b][c];
  __syncthreads();
  if (wk != 0 || !live) return;
  float r[NB][4];
#pragma unroll
  for (int b = 0; b < NB; ++b)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float v = 0.f;
      for (int k = 0; k < p.ks; ++k) v += red[wr * p.ks + k][b][c][lane];
      r[b][c] = v;
    }
  // c0: (weight row g, token 2t)  c1: (g, 2t+1)  c2: (g+8, 2t)  c3: (g+8, 2t+1)
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int n = row0 + g + 8 * (c >> 1), m = 2 * t + (c & 1);
    if (n >= NO || m >= p.M) continue;
    const size_t o = (size_t)m * p.ldo + n;
    if (SWIGLU) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(silu_f(r[0][c]) * r[NB - 1][c]);
    else if (p.epi == MX_BF16) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(r[0][c]);
    else if (p.epi == MX_F32) reinterpret_cast<float*>(p.out)[o] = r[0][c];
    else reinterpret_cast<float*>(p.out)[o] += r[0][c];
  }
}

__global__ void bf16_to_f16_kernel(const bf16* __restrict__ x, int ldx, __half* __restrict__ y, int ldy, int M, int K) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * (K / 2)) return;
  const int m = i / (K / 2), c = (i - m * (K / 2)) * 2;
  const uint32_t v = *reinterpret_cast<const uint32_t*>(x + (size_t)m * ldx + c);
  *reinterpret_cast<__half2*>(y + (size_t)m * ldy + c) = __floats2half2_rn(bf16lo_to_f(v), bf16hi_to_f(v));
}

// bf16 rows -> f16 rows in the lane order of the tiled MXFP4 kernel: inside every 64-column k tile, position
// 16 t + 4 j + c holds column 16 j + (2t, 2t+1, 2t+8, 2t+9)[c], so lane t of a quad reads its B fragments of the
// four k16 steps as 32 contiguous bytes.
__global__ void x16_lane_order_kernel(const bf16* __restrict__ x, int ldx, __half* __restrict__ y, int ldy, int M, int K) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * K) return;
  const int m = i / K, pos = i - m * K;
  const int kt = pos >> 6, r = pos & 63;
  const int t = r >> 4, j = (r >> 2) & 3, c = r & 3;
  const int col = (kt << 6) + 16 * j + 2 * t + (c & 1) + ((c >> 1) << 3);
  y[(size_t)m * ldy + pos] = __float2half_rn(__bfloat162float(x[(size_t)m * ldx + col]));
}

// dequantise a whole MXFP4 matrix to bf16 [N][K] (prefill: dequantise once, then the tcgen05 GEMM)
__global__ void __launch_bounds__(256) dequant_mx_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ s, bf16* __restrict__ out,
                                                         long nblocks) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;      // one MX block (32 values) per thread
  if (i >= nblocks) return;
  const uint4 v = *reinterpret_cast<const uint4*>(w + i * 16);
  const float sc = e8m0_f(s[i]);
  const uint32_t words[4] = {v.x, v.y, v.z, v.w};
  uint4* o = reinterpret_cast<uint4*>(out + i * 32);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t r[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t h2 = cvt_e2m1x2(words[q] >> (8 * b));
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
      r[b] = pack_bf16x2(f.x * sc, f.y * sc);
    }
    o[q] = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

}  // namespace

// x16: f16 scratch [M][ldx16] owned by the caller (filled here from the bf16 x).  epi: 0 bf16, 1 fp32, 2 fp32 +=,
// 3 SwiGLU (weight rows interleaved per 16: [32i, 32i+16) gate, [32i+16, 32i+32) up of output tile i; out bf16
// [M][N/2]).  Requires K % 32 == 0, M in 1..8, N % 32 == 0 for SwiGLU.
GRM_API int grm_smallm_mx(const void* w, const void* scales, const void* x, int ldx, void* x16, int ldx16, void* out, int ldo, int M,
                          int N, int K, int epi, void* stream) {
  if (M < 1 || M > 8 || (K % 32) || (ldx & 1) || (ldx16 & 7) || epi < 0 || epi > 3 || (epi == MX_SWIGLU && (N & 31))) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  const int nconv = M * (K / 2);
  bf16_to_f16_kernel<<<(nconv + 255) / 256, 256, 0, st>>>((const bf16*)x, ldx, (__half*)x16, ldx16, M, K);
  MxParams p;
  p.w = (const uint8_t*)w; p.s = (const uint8_t*)scales; p.x16 = (const __half*)x16; p.out = out; p.ldo = ldo;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx16; p.epi = epi;
  const int NO = epi == MX_SWIGLU ? N / 2 : N;
  const int tiles = (NO + 15) / 16;
  // enough CTAs for 148 SMs: split K inside the CTA as long as the tile count alone would not fill the part
  int ks = 8;
  while (ks > 1 && (tiles / (kWarps / ks)) >= 4 * 148 && (K / 32) / ks >= 1) ks >>= 1;
  while (ks > 1 && (K / 32) < ks) ks >>= 1;
  p.ks = ks; p.rt = kWarps / ks;
  const int grid = (tiles + p.rt - 1) / p.rt;
  if (epi == MX_SWIGLU) smallm_mx_kernel<true><<<grid, kThreads, 0, st>>>(p);
  else smallm_mx_kernel<false><<<grid, kThreads, 0, st>>>(p);
  GRM_LAUNCH_RET();
}

GRM_API int grm_dequant_mxfp4(const void* w, const void* scales, void* out, int N, int K, void* stream) {
  if (K % 32) return -2;
  const long nblocks = (long)N * (K / 32);
  dequant_mx_kernel<<<(unsigned)((nblocks + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)w, (const uint8_t*)scales, (bf16*)out,
                                                                                          nblocks);
  GRM_LAUNCH_RET();
}

GRM_API int grm_x16_lane_order(const void* x, int ldx, void* y, int ldy, int M, int K, void* stream) {
  if (M < 1 || (K % 64) || (ldy & 7)) return -2;
  const int n = M * K;
  x16_lane_order_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, ldx, (__half*)y, ldy, M, K);
  GRM_LAUNCH_RET();
}
