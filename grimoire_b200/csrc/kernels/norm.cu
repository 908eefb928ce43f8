// RMSNorm family over the fp32 residual stream.
//   rmsnorm      : x = rms(h) * (offset + w)                       -> bf16 (feeds the next GEMM)
//   add_rmsnorm  : h += r (fp32 or bf16 delta); x = rms(h)*(offset+w)
//   rmsnorm_heads: per-head RMSNorm over head_dim (q/k norm, GDN gated output norm with silu(z))
// offset = 1 selects the zero-centred (1+w) convention of the Qwen3.5 family, 0 the plain one
// (reference: set_norm_convention, src/kernels.hpp:760-771; launch_rmsnorm_residual*, src/ops.cpp:205-313).
// One CTA per row, 128-bit loads, fp32 math, one pass (the row stays in registers).
#include "common.cuh"

namespace {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 8;  // float4 per thread: H <= 256*4*8 = 8192

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) sh[0] = t;
  }
  __syncthreads();
  t = sh[0];
  __syncthreads();
  return t;
}

// DT: 0 = no delta, 1 = fp32 delta, 2 = bf16 delta
template <int DT>
__global__ void __launch_bounds__(kNormThreads) add_rmsnorm_kernel(float* __restrict__ h, const void* __restrict__ delta,
                                                                   const float* __restrict__ w, bf16* __restrict__ x,
                                                                   float* __restrict__ x32, int H, int ldh, int ldd,
                                                                   int ldx, float eps, float offset) {
  __shared__ float sh[32];
  const int row = blockIdx.x;
  float* hr = h + (size_t)row * ldh;
  const int nvec = H >> 2;
  float4 v[kMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) {
      float4 a = reinterpret_cast<const float4*>(hr)[c];
      if (DT == 1) {
        const float4 d = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(delta) + (size_t)row * ldd)[c];
        a.x += d.x; a.y += d.y; a.z += d.z; a.w += d.w;
      } else if (DT == 2) {
        const uint2 d = reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(delta) + (size_t)row * ldd)[c];
        a.x += bf16lo_to_f(d.x); a.y += bf16hi_to_f(d.x); a.z += bf16lo_to_f(d.y); a.w += bf16hi_to_f(d.y);
      }
      if (DT != 0) reinterpret_cast<float4*>(hr)[c] = a;
      v[i] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = block_sum(ss, sh);
  const float r = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) {
      const float4 g = reinterpret_cast<const float4*>(w)[c];
      const float o0 = v[i].x * r * (offset + g.x), o1 = v[i].y * r * (offset + g.y);
      const float o2 = v[i].z * r * (offset + g.z), o3 = v[i].w * r * (offset + g.w);
      if (x) {
        uint2 o; o.x = pack_bf16x2(o0, o1); o.y = pack_bf16x2(o2, o3);
        reinterpret_cast<uint2*>(x + (size_t)row * ldx)[c] = o;
      }
      if (x32) reinterpret_cast<float4*>(x32 + (size_t)row * ldx)[c] = make_float4(o0, o1, o2, o3);
    }
  }
}

// Per-head norm over D (<= 256, multiple of 32): one warp per (row, head).
//   out = rms(in) * (offset + w)  [* silu(z) when z != null]   (GDN gated output norm:
//   rms_norm(o) * silu(z), not rms_norm(o * silu(z)); src/ops.cpp:770-869)
__global__ void rmsnorm_heads_kernel(const float* __restrict__ in, const bf16* __restrict__ z, const float* __restrict__ w,
                                     bf16* __restrict__ out, int rows, int heads, int D, int ld_in, int ld_z, int ld_out,
                                     float eps, float offset) {
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (wid >= rows * heads) return;
  const int row = wid / heads, hd = wid % heads;
  const float* p = in + (size_t)row * ld_in + hd * D;
  float v[8];
  float ss = 0.f;
  const int per = D >> 5;
  for (int i = 0; i < per; ++i) { v[i] = p[lane + 32 * i]; ss += v[i] * v[i]; }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)D + eps);
  for (int i = 0; i < per; ++i) {
    const int d = lane + 32 * i;
    float o = v[i] * r * (offset + w[d]);
    if (z) o *= silu_f(__bfloat162float(z[(size_t)row * ld_z + hd * D + d]));
    out[(size_t)row * ld_out + hd * D + d] = __float2bfloat16(o);
  }
}

}  // namespace

// h: fp32 [M][ldh] (updated in place when delta != null); delta_dtype 0 none / 1 fp32 / 2 bf16;
// x: bf16 out [M][ldx] (may be null); x32: fp32 out (may be null).  H % 4 == 0, H <= 8192.
GRM_API int grm_add_rmsnorm(void* h, const void* delta, int delta_dtype, const void* w, void* x, void* x32, int M, int H,
                            int ldh, int ldd, int ldx, float eps, float offset, void* stream) {
  if ((H & 3) || H > kNormThreads * 4 * kMaxVec || M < 1) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  if (!delta || delta_dtype == 0)
    add_rmsnorm_kernel<0><<<M, kNormThreads, 0, st>>>((float*)h, nullptr, (const float*)w, (bf16*)x, (float*)x32, H, ldh, ldd, ldx, eps, offset);
  else if (delta_dtype == 1)
    add_rmsnorm_kernel<1><<<M, kNormThreads, 0, st>>>((float*)h, delta, (const float*)w, (bf16*)x, (float*)x32, H, ldh, ldd, ldx, eps, offset);
  else
    add_rmsnorm_kernel<2><<<M, kNormThreads, 0, st>>>((float*)h, delta, (const float*)w, (bf16*)x, (float*)x32, H, ldh, ldd, ldx, eps, offset);
  GRM_LAUNCH_RET();
}

GRM_API int grm_rmsnorm_heads(const void* in, const void* z, const void* w, void* out, int rows, int heads, int D, int ld_in,
                              int ld_z, int ld_out, float eps, float offset, void* stream) {
  if ((D & 31) || D > 256) return -2;
  const int warps = rows * heads;
  const int threads = 256;
  const int blocks = (warps * 32 + threads - 1) / threads;
  rmsnorm_heads_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((const float*)in, (const bf16*)z, (const float*)w, (bf16*)out,
                                                                   rows, heads, D, ld_in, ld_z, ld_out, eps, offset);
  GRM_LAUNCH_RET();
}
