// Warp-MMA helpers shared by the paged attention kernels over the int8 KV cache (attn_decode.cu, attn_verify.cu).
#pragma once
#include "common.cuh"

namespace attn_mma {

// int8 x int8 -> int32 tensor-core MMA (K rows are int8 already; q is split in two int8 levels)
__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Rotation of the float4 chunks of lane (g, t)'s window in the per-warp output staging (see the store in the kernel).
template <int D>
__device__ __forceinline__ int so_rot(int g, int t) {
  return D == 64 ? ((t >> 1) + 2 * g) : (2 * t + g);
}
// Position of dim d of head g inside sm_o[warp][g][]: the inverse of that rotation.
template <int D>
__device__ __forceinline__ int so_index(int g, int d) {
  constexpr int W = D / 4;                       // dims per lane window
  const int t = d / W, m = d % W;
  const int chunk = ((m >> 2) + so_rot<D>(g, t)) & (D / 16 - 1);
  return t * W + 4 * chunk + (m & 3);
}

}  // namespace attn_mma
