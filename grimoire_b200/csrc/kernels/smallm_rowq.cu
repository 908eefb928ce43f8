// smallm_rowq: Y[M<=8][N] = X[M][K] . W[N][K]^T for the 8- and 16-bit weight formats of --proj
// {bf16, int8, fp8_e4m3, fp8_e5m2, mxfp8}: one byte (or one bf16) per weight, a fp32 scale per output row
// (int8 / fp8) or an e8m0 scale per 32 weights (mxfp8).  Reference: the int8 / fp8 / mxfp8 rows of gemv_impl
// (src/gemv_decode.cpp:77-347) and their small-M forms (src/gemm_fast.cpp).
//
// The kernel is a weight stream: a warp owns one output column (two weight rows with the SwiGLU epilogue: gate and
// up rows are interleaved per 16, the order of interleave_gate_up in formats/w4_tile_layout.py).  Every lane reads
// 16 weights per step with one 16-byte load (two for bf16), converts them in registers (hardware fp8x2 -> f16x2
// conversions, sign-extending shifts for int8) and multiplies them with the bf16 activations of up to 8 batch rows,
// which stay in L1.
// More rows dequantise to bf16 (grm_dequant_rowq) and run the tcgen05 GEMM.
#include "common.cuh"
#include <cuda_fp8.h>

namespace {

enum RowQKind : int { RQ_BF16 = 0, RQ_INT8 = 1, RQ_E4M3 = 2, RQ_E5M2 = 3, RQ_MXFP8 = 4 };

__device__ __forceinline__ float2 fp8x2_to_f2(uint32_t v16, bool e5m2) {
  uint32_t h2;
  const unsigned short s = (unsigned short)v16;
  if (e5m2) asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(h2) : "h"(s));
  else asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(s));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

// 16 weights of one lane -> fp32
template <int KIND>
__device__ __forceinline__ void load16(const uint8_t* wrow, int k, float (&wf)[16]) {
  if constexpr (KIND == RQ_BF16) {
    const uint4 a = ldg_stream_v4(wrow + (size_t)k * 2), b = ldg_stream_v4(wrow + (size_t)k * 2 + 16);
    const uint32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) { wf[2 * i] = bf16lo_to_f(v[i]); wf[2 * i + 1] = bf16hi_to_f(v[i]); }
  } else {
    const uint4 a = ldg_stream_v4(wrow + k);
    const uint32_t v[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (KIND == RQ_INT8) {
#pragma unroll
        for (int b = 0; b < 4; ++b) wf[4 * i + b] = (float)(int)(int8_t)((v[i] >> (8 * b)) & 0xffu);
      } else {
        const float2 lo = fp8x2_to_f2(v[i] & 0xffffu, KIND == RQ_E5M2), hi = fp8x2_to_f2(v[i] >> 16, KIND == RQ_E5M2);
        wf[4 * i] = lo.x; wf[4 * i + 1] = lo.y; wf[4 * i + 2] = hi.x; wf[4 * i + 3] = hi.y;
      }
    }
  }
}

__device__ __forceinline__ float dot16(const float (&wf)[16], const bf16* xr) {
  const uint4 a = *reinterpret_cast<const uint4*>(xr), b = *reinterpret_cast<const uint4*>(xr + 8);
  const uint32_t v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += wf[2 * i] * bf16lo_to_f(v[i]) + wf[2 * i + 1] * bf16hi_to_f(v[i]);
  return s;
}

struct RowQParams {
  const uint8_t* w;       // [N][ldw bytes]
  const float* scale;     // [N] (int8 / fp8), null for bf16
  const uint8_t* e8;      // [N][K/32] (mxfp8)
  const bf16* x;          // [M][ldx]
  void* out;              // [M][ldo]: bf16 (epi 0, 3) or fp32 (epi 1, 2)
  int M, N, K, ldx, ldo, epi;
  long ldw;
};

// epi: 0 bf16, 1 f32, 2 add_f32, 3 swiglu (N = 2 I rows, gate / up interleaved per 16; out bf16 [M][I])
template <int KIND, int MB, bool SWIGLU>
__global__ void __launch_bounds__(256) smallm_rowq_kernel(const RowQParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int NO = SWIGLU ? p.N / 2 : p.N;
  if (warp >= NO) return;
  constexpr int NR = SWIGLU ? 2 : 1;
  const uint8_t* wr[NR];
  int rows[NR];
  rows[0] = SWIGLU ? 32 * (warp >> 4) + (warp & 15) : warp;
  if (SWIGLU) rows[NR - 1] = rows[0] + 16;
#pragma unroll
  for (int r = 0; r < NR; ++r) wr[r] = p.w + (size_t)rows[r] * p.ldw;
  float acc[NR][MB];
#pragma unroll
  for (int r = 0; r < NR; ++r)
#pragma unroll
    for (int m = 0; m < MB; ++m) acc[r][m] = 0.f;
  const int KB = p.K >> 5;
  for (int k = lane * 16; k < p.K; k += 512) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      float wf[16];
      load16<KIND>(wr[r], k, wf);
      float bs = 1.f;
      if constexpr (KIND == RQ_MXFP8) {
        bs = __uint_as_float((uint32_t)p.e8[(size_t)rows[r] * KB + (k >> 5)] << 23);
      }
#pragma unroll
      for (int m = 0; m < MB; ++m)
        if (m < p.M) acc[r][m] += bs * dot16(wf, p.x + (size_t)m * p.ldx + k);
    }
  }
  float rs[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) rs[r] = (p.scale != nullptr) ? p.scale[rows[r]] : 1.f;
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    float s[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) s[r] = warp_sum(acc[r][m]) * rs[r];
    if (lane == 0 && m < p.M) {
      const size_t o = (size_t)m * p.ldo + warp;
      if (SWIGLU) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(silu_f(s[0]) * s[NR - 1]);
      else if (p.epi == 0) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(s[0]);
      else if (p.epi == 1) reinterpret_cast<float*>(p.out)[o] = s[0];
      else reinterpret_cast<float*>(p.out)[o] += s[0];
    }
  }
}

template <int KIND, int MB>
int launch_mb(const RowQParams& p, cudaStream_t st) {
  const int NO = p.epi == 3 ? p.N / 2 : p.N;
  const int threads = 256;
  const long blocks = ((long)NO * 32 + threads - 1) / threads;
  if (p.epi == 3) smallm_rowq_kernel<KIND, MB, true><<<(unsigned)blocks, threads, 0, st>>>(p);
  else smallm_rowq_kernel<KIND, MB, false><<<(unsigned)blocks, threads, 0, st>>>(p);
  GRM_LAUNCH_RET();
}

template <int KIND>
int launch_kind(const RowQParams& p, cudaStream_t st) {
  if (p.M <= 1) return launch_mb<KIND, 1>(p, st);
  if (p.M <= 2) return launch_mb<KIND, 2>(p, st);
  if (p.M <= 4) return launch_mb<KIND, 4>(p, st);
  return launch_mb<KIND, 8>(p, st);
}

template <int KIND>
__global__ void __launch_bounds__(256) dequant_rowq_kernel(const uint8_t* __restrict__ w, const float* __restrict__ scale,
                                                           const uint8_t* __restrict__ e8, bf16* __restrict__ out, int N, int K,
                                                           long ldw, int ldo) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;   // one 16-weight group per thread
  const int per = K >> 4;
  if (idx >= (long)N * per) return;
  const int n = (int)(idx / per), k = (int)(idx % per) * 16;
  float wf[16];
  load16<KIND>(w + (size_t)n * ldw, k, wf);
  float s = scale ? scale[n] : 1.f;
  if constexpr (KIND == RQ_MXFP8) s = __uint_as_float((uint32_t)e8[(size_t)n * (K >> 5) + (k >> 5)] << 23);
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = pack_bf16x2(wf[2 * i] * s, wf[2 * i + 1] * s);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)n * ldo + k);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

}  // namespace

// kind: 0 bf16, 1 int8, 2 fp8 e4m3, 3 fp8 e5m2 (fp32 scale per row, may be null = 1), 4 mxfp8 (e4m3 payload, e8m0 per 32
// weights along K).  ldw in bytes.  epi: 0 bf16, 1 f32, 2 add_f32, 3 swiglu.  Returns -2 on an unsupported shape.
GRM_API int grm_smallm_rowq(const void* w, const void* scale, const void* e8, const void* x, void* out, int kind, int M, int N, int K,
                            long ldw, int ldx, int ldo, int epi, void* stream) {
  if (M < 1 || M > 8 || (K & 31) || (ldx & 7) || (ldw & 15) || ((uintptr_t)w & 15) || ((uintptr_t)x & 15) || epi < 0 || epi > 3 ||
      (epi == 3 && (N & 31)) || (kind == RQ_MXFP8 && !e8))
    return -2;
  RowQParams p;
  p.w = (const uint8_t*)w; p.scale = (const float*)scale; p.e8 = (const uint8_t*)e8; p.x = (const bf16*)x; p.out = out;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldo = ldo; p.epi = epi; p.ldw = ldw;
  cudaStream_t st = (cudaStream_t)stream;
  switch (kind) {
    case RQ_BF16: return launch_kind<RQ_BF16>(p, st);
    case RQ_INT8: return launch_kind<RQ_INT8>(p, st);
    case RQ_E4M3: return launch_kind<RQ_E4M3>(p, st);
    case RQ_E5M2: return launch_kind<RQ_E5M2>(p, st);
    case RQ_MXFP8: return launch_kind<RQ_MXFP8>(p, st);
  }
  return -2;
}

// W -> bf16 [N][ldo] (scales applied), for the tcgen05 GEMM on tall inputs.
GRM_API int grm_dequant_rowq(const void* w, const void* scale, const void* e8, void* out, int kind, int N, int K, long ldw, int ldo,
                             void* stream) {
  if ((K & 31) || (ldo & 7) || (ldw & 15) || ((uintptr_t)out & 15) || (kind == RQ_MXFP8 && !e8)) return -2;
  const long groups = (long)N * (K >> 4);
  const int threads = 256;
  const unsigned blocks = (unsigned)((groups + threads - 1) / threads);
  cudaStream_t st = (cudaStream_t)stream;
  const uint8_t* wp = (const uint8_t*)w;
  const float* sp = (const float*)scale;
  const uint8_t* ep = (const uint8_t*)e8;
  switch (kind) {
    case RQ_BF16: dequant_rowq_kernel<RQ_BF16><<<blocks, threads, 0, st>>>(wp, sp, ep, (bf16*)out, N, K, ldw, ldo); break;
    case RQ_INT8: dequant_rowq_kernel<RQ_INT8><<<blocks, threads, 0, st>>>(wp, sp, ep, (bf16*)out, N, K, ldw, ldo); break;
    case RQ_E4M3: dequant_rowq_kernel<RQ_E4M3><<<blocks, threads, 0, st>>>(wp, sp, ep, (bf16*)out, N, K, ldw, ldo); break;
    case RQ_E5M2: dequant_rowq_kernel<RQ_E5M2><<<blocks, threads, 0, st>>>(wp, sp, ep, (bf16*)out, N, K, ldw, ldo); break;
    case RQ_MXFP8: dequant_rowq_kernel<RQ_MXFP8><<<blocks, threads, 0, st>>>(wp, sp, ep, (bf16*)out, N, K, ldw, ldo); break;
    default: return -2;
  }
  GRM_LAUNCH_RET();
}
