// Load-time / per-call format conversion kernels.
//   dequant_w4_tiled : tiled int4 (see smallm_w4.cu) -> bf16 [N][K] row-major, the B operand of the
//                      tcgen05 prefill GEMM.  Same policy as the reference's large-M path, which
//                      dequantizes a weight once per call into a bf16 scratch before the matrix-unit
//                      GEMM (dequant_* + gemm_bf16_vnni, src/gemm_fast.cpp:138-560); the values are
//                      bf16(scale * (q - zero)) computed in fp32.
// A CTA converts 32 rows x 512 k through shared memory so global stores are 1 KiB row segments.
#include "common.cuh"

namespace {

constexpr int kRows = 32;
constexpr int kKT = 8;            // k tiles (of 64) per CTA
constexpr int kCols = kKT * 64;   // 512

__global__ void __launch_bounds__(256) dequant_w4_kernel(const uint4* __restrict__ w, const uint32_t* __restrict__ sz,
                                                         bf16* __restrict__ out, int N, int K, int g64, int ldo) {
  __shared__ __align__(16) bf16 tile[kRows][kCols + 8];
  const int ns = blockIdx.x, ktb = blockIdx.y * kKT;
  const int KT = K >> 6, G = KT / g64;
  const int tid = threadIdx.x;
  // 8 k tiles x 2 halves x 32 lanes = 512 uint4 -> 2 per thread
  for (int i = tid; i < kKT * 64; i += 256) {
    const int ktl = i >> 6, rem = i & 63, half = rem >> 5, lane = rem & 31;
    const int kt = ktb + ktl;
    if (kt >= KT) continue;
    const uint4 v = w[((size_t)ns * KT + kt) * 64 + rem];
    const int g = lane >> 2, t = lane & 3;
    const int nt = ns * 2 + half;
    const int gi = kt / g64;
    const uint32_t s0 = sz[((size_t)nt * G + gi) * 16 + g], s1 = sz[((size_t)nt * G + gi) * 16 + g + 8];
    const float sc[2] = {__half2float(__ushort_as_half((unsigned short)(s0 & 0xffff))),
                         __half2float(__ushort_as_half((unsigned short)(s1 & 0xffff)))};
    const float zc[2] = {bf16hi_to_f(s0) - 128.f, bf16hi_to_f(s1) - 128.f};
    const uint32_t wj[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
      for (int r = 0; r < 4; ++r) {   // register r: row g + 8*(r&1), k = 16t + 4j + 2*(r>>1) + {0,1}
        const int lo = (wj[j] >> (4 * r)) & 0xf, hi = (wj[j] >> (4 * r + 16)) & 0xf;
        const int rr = r & 1;
        const int row = half * 16 + g + 8 * rr;
        const int col = ktl * 64 + 16 * t + 4 * j + 2 * (r >> 1);
        const uint32_t o = pack_bf16x2(((float)lo - zc[rr]) * sc[rr], ((float)hi - zc[rr]) * sc[rr]);
        *reinterpret_cast<uint32_t*>(&tile[row][col]) = o;
      }
    }
  }
  __syncthreads();
  // 32 rows x 512 cols -> 16-byte stores, a row segment (1 KiB) per 64 threads
  for (int i = tid; i < kRows * (kCols / 8); i += 256) {
    const int row = i / (kCols / 8), c8 = i % (kCols / 8);
    const int n = ns * 32 + row, k = ktb * 64 + c8 * 8;
    if (n < N && k < K) *reinterpret_cast<uint4*>(out + (size_t)n * ldo + k) = *reinterpret_cast<const uint4*>(&tile[row][c8 * 8]);
  }
}

}  // namespace

GRM_API int grm_dequant_w4(const void* w, const void* sz, void* out, int N, int K, int group, int ldo, void* stream) {
  if ((N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (ldo & 7)) return -2;
  dim3 grid(N / 32, ((K >> 6) + kKT - 1) / kKT);
  dequant_w4_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)w, (const uint32_t*)sz, (bf16*)out, N, K, group / 64, ldo);
  GRM_LAUNCH_RET();
}
