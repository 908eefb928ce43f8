// gemv_gguf: projections straight over raw GGUF blocks -- decode steps of a model that keeps its checkpoint's ggml
// quantisation (``--proj native`` on a .gguf file) read the stored bytes as they are instead of a re-quantised copy.
// Reference: gemv_native_qk (src/gemv_decode.cpp:1216-1274) with the per-type block readers of
// include/b70/native_qk_*.hpp.  Types served: Q4_0 (2), Q8_0 (8), Q4_K (12), Q5_K (13), Q6_K (14), IQ4_NL (20), IQ4_XS (23);
// the block layouts are
// ggml's (the host decoder csrc/host/gguf.cpp is the oracle the tests compare with).
//
// One warp per output row, 8 rows per CTA.  A lane takes 32-weight pieces -- a whole block of the 32-weight types, one of
// the eight sub-blocks of a 256-weight K-quant super-block -- at indices lane, lane + 32, ...: it decodes the piece's 32
// weights in registers and multiplies them with up to 8 activation rows held as bf16 in shared memory, so 1..8 rows cost
// one pass over the weights.  fp32 accumulation, shuffle reduction, bf16 / fp32 / accumulate epilogues.  Block sizes of
// 18, 34 and 210 bytes leave the blocks 2-byte aligned only, so weights are fetched with 16-bit loads: this path is about
// keeping the checkpoint's exact numbers and a quarter of the memory of a bf16 expansion, not about the last GB/s.
// Taller inputs expand the rows to bf16 (grm_dequant_gguf) for the tcgen05 GEMM.
#include "common.cuh"

namespace {

constexpr int kRowsPerCta = 8;
constexpr int kMaxM = 8;

__device__ __forceinline__ float h2f_dev(const uint8_t* p) {
  const unsigned short v = *reinterpret_cast<const unsigned short*>(p);
  return __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ uint32_t ld16(const uint8_t* p) { return *reinterpret_cast<const unsigned short*>(p); }

// 6-bit scale / min pair j of a Q4_K / Q5_K super-block (12 packed bytes)
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& sc, int& m) {
  if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
  else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
}

// bytes per block, weights per block
__host__ __device__ inline int blk_bytes(int type) {
  return type == 2 ? 18 : type == 8 ? 34 : type == 12 ? 144 : type == 13 ? 176 : type == 14 ? 210 : type == 20 ? 18 : type == 23 ? 136 : 0;
}
__host__ __device__ inline int blk_weights(int type) { return (type == 2 || type == 8 || type == 20) ? 32 : 256; }

// the 16 levels of ggml's non-linear 4-bit code (IQ4_NL / IQ4_XS), four per word, read with a byte extract
__device__ __forceinline__ float iq4_level(int q) {
  constexpr uint32_t t0 = 0xBFAD9881u, t1 = 0xF6EADDCFu, t2 = 0x26190D01u, t3 = 0x71594535u;   // -127 -104 -83 -65 | -49 -35 -22 -10 | 1 13 25 38 | 53 69 89 113
  const uint32_t word = (q & 8) ? ((q & 4) ? t3 : t2) : ((q & 4) ? t1 : t0);
  return (float)(int8_t)((word >> (8 * (q & 3))) & 0xFF);
}

// Decode piece ``piece`` (32 weights: columns 32 * piece .. 32 * piece + 31) of a row stored at ``row`` into w[32].
template <int TYPE>
__device__ __forceinline__ void decode_piece(const uint8_t* row, int piece, float (&w)[32]) {
  if (TYPE == 2) {          // Q4_0: d, 16 bytes; weight j = low nibble of byte j, weight j + 16 = high nibble
    const uint8_t* b = row + (size_t)piece * 18;
    const float d = h2f_dev(b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t v = ld16(b + 2 + 2 * j);
      w[2 * j] = (float)((int)(v & 0xF) - 8) * d;
      w[2 * j + 1] = (float)((int)((v >> 8) & 0xF) - 8) * d;
      w[2 * j + 16] = (float)((int)((v >> 4) & 0xF) - 8) * d;
      w[2 * j + 17] = (float)((int)((v >> 12) & 0xF) - 8) * d;
    }
  } else if (TYPE == 20 || TYPE == 23) {   // IQ4_NL: d, 16 bytes | IQ4_XS: d, 16 high scale bits, 4 low scale bytes, 8 x 16 bytes
    const uint8_t* b;
    const uint8_t* q;
    float d;
    if (TYPE == 20) {
      b = row + (size_t)piece * 18;
      q = b + 2;
      d = h2f_dev(b);
    } else {
      b = row + (size_t)(piece >> 3) * 136;
      const int ib = piece & 7;
      const uint32_t sh = ld16(b + 2);
      const int ls = (int)((b[4 + (ib >> 1)] >> (4 * (ib & 1))) & 0xF) | (int)(((sh >> (2 * ib)) & 3) << 4);
      q = b + 8 + 16 * ib;
      d = h2f_dev(b) * (float)(ls - 32);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t v = ld16(q + 2 * j);
      w[2 * j] = iq4_level((int)(v & 0xF)) * d;
      w[2 * j + 1] = iq4_level((int)((v >> 8) & 0xF)) * d;
      w[2 * j + 16] = iq4_level((int)((v >> 4) & 0xF)) * d;
      w[2 * j + 17] = iq4_level((int)((v >> 12) & 0xF)) * d;
    }
  } else if (TYPE == 8) {   // Q8_0: d, 32 int8
    const uint8_t* b = row + (size_t)piece * 34;
    const float d = h2f_dev(b);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t v = ld16(b + 2 + 2 * j);
      w[2 * j] = (float)(int8_t)(v & 0xFF) * d;
      w[2 * j + 1] = (float)(int8_t)(v >> 8) * d;
    }
  } else if (TYPE == 12 || TYPE == 13) {   // Q4_K / Q5_K: d, dmin, 12 scale bytes, [32 high-bit bytes,] 128 nibble bytes
    const uint8_t* b = row + (size_t)(piece >> 3) * (TYPE == 12 ? 144 : 176);
    const int sb = piece & 7, chunk = sb >> 1, hi = sb & 1;
    int sc, m;
    scale_min_k4(sb, b + 4, sc, m);
    const float d = h2f_dev(b) * (float)sc, mn = h2f_dev(b + 2) * (float)m;
    const uint8_t* q = b + (TYPE == 12 ? 16 : 48) + 32 * chunk;
    const uint8_t* qh = b + 16;           // Q5_K only: bit (2 chunk + hi) of byte l is the fifth bit of weight l
#pragma unroll
    for (int l = 0; l < 32; l += 2) {
      const uint32_t v = ld16(q + l);
      int q0 = hi ? (int)((v >> 4) & 0xF) : (int)(v & 0xF), q1 = hi ? (int)((v >> 12) & 0xF) : (int)((v >> 8) & 0xF);
      if (TYPE == 13) {
        const uint32_t hb = ld16(qh + l);
        q0 += ((hb >> sb) & 1) ? 16 : 0;
        q1 += ((hb >> (8 + sb)) & 1) ? 16 : 0;
      }
      w[l] = d * (float)q0 - mn;
      w[l + 1] = d * (float)q1 - mn;
    }
  } else {                  // Q6_K: 128 low-nibble bytes, 64 high-2-bit bytes, 16 int8 scales, d
    const uint8_t* b = row + (size_t)(piece >> 3) * 210;
    const int sb = piece & 7, n = sb >> 2, qd = sb & 3;
    const uint8_t* ql = b + 64 * n + ((qd & 1) ? 32 : 0);
    const uint8_t* qh = b + 128 + 32 * n;
    const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192) + 8 * n + 2 * qd;
    const float d = h2f_dev(b + 208);
    const float d0 = d * (float)sc[0], d1 = d * (float)sc[1];
#pragma unroll
    for (int l = 0; l < 32; l += 2) {
      const uint32_t lo = ld16(ql + l), hb = ld16(qh + l);
      const int n0 = (qd >= 2) ? (int)((lo >> 4) & 0xF) : (int)(lo & 0xF), n1 = (qd >= 2) ? (int)((lo >> 12) & 0xF) : (int)((lo >> 8) & 0xF);
      const int h0 = (int)((hb >> (2 * qd)) & 3), h1 = (int)((hb >> (8 + 2 * qd)) & 3);
      w[l] = (l < 16 ? d0 : d1) * (float)((n0 | (h0 << 4)) - 32);
      w[l + 1] = (l < 16 ? d0 : d1) * (float)((n1 | (h1 << 4)) - 32);
    }
  }
}

struct GgufParams {
  const uint8_t* w; long row_bytes;
  const bf16* x; int ldx;
  void* out; int ldo;
  int M, N, K, epi;            // epi: 0 bf16, 1 f32, 2 add_f32
};

template <int TYPE>
__global__ void __launch_bounds__(kRowsPerCta * 32) gemv_gguf_kernel(const GgufParams p) {
  extern __shared__ __align__(16) uint8_t gg_smem[];
  bf16* xs = reinterpret_cast<bf16*>(gg_smem);                 // [M][K]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid * 8; i < p.M * p.K; i += kRowsPerCta * 32 * 8) {
    const int m = i / p.K, k = i - m * p.K;
    *reinterpret_cast<uint4*>(xs + i) = *reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx + k);
  }
  __syncthreads();
  const int n = blockIdx.x * kRowsPerCta + warp;
  if (n >= p.N) return;
  const uint8_t* row = p.w + (size_t)n * p.row_bytes;
  float acc[kMaxM];
#pragma unroll
  for (int m = 0; m < kMaxM; ++m) acc[m] = 0.f;
  const int pieces = p.K / 32;
  for (int pc = lane; pc < pieces; pc += 32) {
    float w[32];
    decode_piece<TYPE>(row, pc, w);
#pragma unroll
    for (int m = 0; m < kMaxM; ++m) {
      if (m < p.M) {
        const uint4* xv = reinterpret_cast<const uint4*>(xs + (size_t)m * p.K + 32 * pc);
        float s = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 v = xv[c];
          s += w[8 * c] * bf16lo_to_f(v.x) + w[8 * c + 1] * bf16hi_to_f(v.x) + w[8 * c + 2] * bf16lo_to_f(v.y) + w[8 * c + 3] * bf16hi_to_f(v.y)
             + w[8 * c + 4] * bf16lo_to_f(v.z) + w[8 * c + 5] * bf16hi_to_f(v.z) + w[8 * c + 6] * bf16lo_to_f(v.w) + w[8 * c + 7] * bf16hi_to_f(v.w);
        }
        acc[m] += s;
      }
    }
  }
#pragma unroll
  for (int m = 0; m < kMaxM; ++m) {
    if (m < p.M) {
      const float s = warp_sum(acc[m]);
      if (lane == 0) {
        const size_t o = (size_t)m * p.ldo + n;
        if (p.epi == 0) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(s);
        else if (p.epi == 1) reinterpret_cast<float*>(p.out)[o] = s;
        else reinterpret_cast<float*>(p.out)[o] += s;
      }
    }
  }
}

template <int TYPE>
__global__ void __launch_bounds__(256) dequant_gguf_kernel(const uint8_t* w, long row_bytes, bf16* out, long ldo, int N, int K) {
  const int pieces = K / 32;
  const long total = (long)N * pieces;
  for (long i = blockIdx.x * 256L + threadIdx.x; i < total; i += (long)gridDim.x * 256) {
    const int n = (int)(i / pieces), pc = (int)(i - (long)n * pieces);
    float v[32];
    decode_piece<TYPE>(w + (size_t)n * row_bytes, pc, v);
    uint32_t pk[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)n * ldo + 32 * pc);
#pragma unroll
    for (int c = 0; c < 4; ++c) dst[c] = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
  }
}

__global__ void __launch_bounds__(256) swiglu_mul_kernel(const float* g, const float* u, bf16* out, int M, int I, int ldg, int ldo) {
  const long total = (long)M * I;
  for (long i = blockIdx.x * 256L + threadIdx.x; i < total; i += (long)gridDim.x * 256) {
    const int m = (int)(i / I), c = (int)(i - (long)m * I);
    out[(size_t)m * ldo + c] = __float2bfloat16(silu_f(g[(size_t)m * ldg + c]) * u[(size_t)m * ldg + c]);
  }
}

template <int TYPE>
int launch_gemv(const GgufParams& p, cudaStream_t st) {
  const size_t smem = (size_t)p.M * p.K * 2;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemv_gguf_kernel<TYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  gemv_gguf_kernel<TYPE><<<(p.N + kRowsPerCta - 1) / kRowsPerCta, kRowsPerCta * 32, smem, st>>>(p);
  GRM_LAUNCH_RET();
}

}  // namespace

// 1 when the raw-block kernels serve this ggml type id.
GRM_API int grm_gguf_native_type(int type) { return blk_bytes(type) != 0 ? 1 : 0; }

// out[M][N] (epi 0 bf16 / 1 f32 / 2 fp32 accumulate) = x[M][K] (bf16) . W^T with W's N rows stored as raw ggml blocks of
// ``type``, row n at w + n * row_bytes.  M <= 8, M * K * 2 bytes of shared memory <= 200 KB, K a multiple of the type's block
// size and of 32, x rows 16-byte aligned.  Returns -2 on anything else.
GRM_API int grm_gemv_gguf(int type, const void* w, long row_bytes, const void* x, int ldx, void* out, int ldo, int M, int N, int K, int epi,
                          void* stream) {
  if (!blk_bytes(type) || M < 1 || M > kMaxM || N < 1 || (K % blk_weights(type)) || (K & 31) || epi < 0 || epi > 2 || (ldx & 7) ||
      ((uintptr_t)x & 15) || ((uintptr_t)w & 1) || (row_bytes & 1) || (size_t)M * K * 2 > 200 * 1024)
    return -2;
  GgufParams p;
  p.w = (const uint8_t*)w; p.row_bytes = row_bytes; p.x = (const bf16*)x; p.ldx = ldx; p.out = out; p.ldo = ldo;
  p.M = M; p.N = N; p.K = K; p.epi = epi;
  cudaStream_t st = (cudaStream_t)stream;
  switch (type) {
    case 2: return launch_gemv<2>(p, st);
    case 8: return launch_gemv<8>(p, st);
    case 12: return launch_gemv<12>(p, st);
    case 13: return launch_gemv<13>(p, st);
    case 14: return launch_gemv<14>(p, st);
    case 20: return launch_gemv<20>(p, st);
    case 23: return launch_gemv<23>(p, st);
    default: return -2;
  }
}

// Expand N raw rows to bf16 [N][ldo] (for the tcgen05 GEMM of taller inputs).
GRM_API int grm_dequant_gguf(int type, const void* w, long row_bytes, void* out, long ldo, int N, int K, void* stream) {
  if (!blk_bytes(type) || N < 1 || (K % blk_weights(type)) || (K & 31) || (ldo & 7) || ((uintptr_t)out & 15) || ((uintptr_t)w & 1) || (row_bytes & 1))
    return -2;
  const long total = (long)N * (K / 32);
  const int grid = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  cudaStream_t st = (cudaStream_t)stream;
  switch (type) {
    case 2: dequant_gguf_kernel<2><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, (bf16*)out, ldo, N, K); break;
    case 8: dequant_gguf_kernel<8><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, (bf16*)out, ldo, N, K); break;
    case 12: dequant_gguf_kernel<12><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, (bf16*)out, ldo, N, K); break;
    case 13: dequant_gguf_kernel<13><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, (bf16*)out, ldo, N, K); break;
    case 14: dequant_gguf_kernel<14><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, (bf16*)out, ldo, N, K); break;
    case 20: dequant_gguf_kernel<20><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, (bf16*)out, ldo, N, K); break;
    case 23: dequant_gguf_kernel<23><<<grid, 256, 0, st>>>((const uint8_t*)w, row_bytes, (bf16*)out, ldo, N, K); break;
    default: return -2;
  }
  GRM_LAUNCH_RET();
}

// out (bf16 [M][I]) = silu(g) * u for fp32 g, u [M][ldg] (the gate / up halves of an MLP whose two projections keep
// different block types and therefore cannot share one fused-epilogue launch).
GRM_API int grm_swiglu_mul(const void* g, const void* u, void* out, int M, int I, int ldg, int ldo, void* stream) {
  if (M < 1 || I < 1) return -2;
  const long total = (long)M * I;
  const int grid = (int)((total + 255) / 256 < 148 * 4 ? (total + 255) / 256 : 148 * 4);
  swiglu_mul_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const float*)g, (const float*)u, (bf16*)out, M, I, ldg, ldo);
  GRM_LAUNCH_RET();
}
