// Small bandwidth-trivial kernels: embedding lookup, arg-max over the vocabulary, sampling glue,
// element-wise helpers and the debug probe.
//   embed_lookup   (reference: launch_embed*, src/ops.cpp:684-731)
//   argmax_rows    (reference: two-stage launch_argmax, src/ops.cpp:611; here one CTA per row)
//   probe_stats    (reference: launch_probe, src/ops.cpp:1688: rms / max / nan / inf of a buffer)
#include "common.cuh"

namespace {

// table bf16 [V][H] -> h fp32 [M][H]; ids < 0 or >= V give a zero row and record GRM_ERR_BOUNDS (detail = row) in the
// status block: the access is skipped, never made.
__global__ void embed_kernel(const int* __restrict__ ids, const bf16* __restrict__ table, float* __restrict__ h, int H, int V,
                             int ldh, float scale, unsigned int* status) {
  grm_pdl_trigger();
  grm_pdl_wait();      // the ids may come from the previous step's token pick
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool ok = id >= 0 && id < V;
  if (!ok && threadIdx.x == 0) grm_set_error(status, GRM_ERR_BOUNDS, 0x10000u | (unsigned int)(row & 0xffff));
  const uint2* src = reinterpret_cast<const uint2*>(table + (size_t)(ok ? id : 0) * H);
  float4* dst = reinterpret_cast<float4*>(h + (size_t)row * ldh);
  for (int c = threadIdx.x; c < (H >> 2); c += blockDim.x) {
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    if (ok) {
      const uint2 v = src[c];
      o = make_float4(bf16lo_to_f(v.x) * scale, bf16hi_to_f(v.x) * scale, bf16lo_to_f(v.y) * scale, bf16hi_to_f(v.y) * scale);
    }
    dst[c] = o;
  }
}

// ties resolve to the lowest index (greedy decoding must be reproducible across batchings).
__device__ __forceinline__ void amax_combine(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
}

constexpr int kArgChunks = 64;

// Stage 1: grid (kArgChunks, M), each CTA scans a slice of the vocabulary with coalesced loads;
// the last CTA to arrive for a row folds the kArgChunks partial (value, index) pairs.
__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, int* __restrict__ out_id,
                                                     float* __restrict__ out_val, float* __restrict__ part_val,
                                                     int* __restrict__ part_idx, unsigned int* __restrict__ counters, int V,
                                                     int ld) {
  grm_pdl_trigger();
  grm_pdl_wait();      // the logits come from the launch before this one
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ int s_last;
  const int row = blockIdx.y, chunk = blockIdx.x;
  const int per = (V + kArgChunks - 1) / kArgChunks;
  const int lo = chunk * per, hi = min(V, lo + per);
  const float* p = logits + (size_t)row * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += 256) amax_combine(best, bi, p[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax_combine(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) amax_combine(best, bi, sv[w], si[w]);
    part_val[row * kArgChunks + chunk] = best;
    part_idx[row * kArgChunks + chunk] = bi;
    __threadfence();
    const unsigned int prev = atomicAdd(&counters[row], 1u);
    s_last = (prev == kArgChunks - 1);
    if (s_last) counters[row] = 0u;
  }
  __syncthreads();
  if (!s_last || warp != 0) return;
  __threadfence();
  best = -INFINITY; bi = 0x7fffffff;
  for (int c = lane; c < kArgChunks; c += 32) amax_combine(best, bi, __ldcg(&part_val[row * kArgChunks + c]), __ldcg(&part_idx[row * kArgChunks + c]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax_combine(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane == 0) { out_id[row] = bi; if (out_val) out_val[row] = best; }
}

// out[0]=sum of squares, [1]=max abs, [2]=#nan, [3]=#inf  (fp32 input)
__global__ void probe_kernel(const float* __restrict__ x, long n, float* __restrict__ out) {
  float ss = 0.f, mx = 0.f, nn = 0.f, ni = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float v = x[i];
    if (isnan(v)) nn += 1.f;
    else if (isinf(v)) ni += 1.f;
    else { ss += v * v; mx = fmaxf(mx, fabsf(v)); }
  }
  ss = warp_sum(ss); mx = warp_max(mx); nn = warp_sum(nn); ni = warp_sum(ni);
  if ((threadIdx.x & 31) == 0) {
    atomicAdd(out + 0, ss);
    atomicMax(reinterpret_cast<int*>(out + 1), __float_as_int(mx));
    atomicAdd(out + 2, nn);
    atomicAdd(out + 3, ni);
  }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(in[i]);
}

// bumps the per-row positions / sequence lengths that live on the device so a captured decode
// graph can be replayed (reference: launch_incr_pos2, src/ops.cpp).
__global__ void incr_pos_kernel(int* __restrict__ pos, int n, int by) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) pos[i] += by;
}

}  // namespace

GRM_API int grm_embed(const void* ids, const void* table, void* h, int M, int H, int V, int ldh, float scale, void* stream) {
  if (H & 3) return -2;
  cudaError_t e = grm_launch_pdl(GRM_PDL_MISC, embed_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, (const int*)ids, (const bf16*)table, (float*)h, H,
                                 V, ldh, scale, grm_status_ptr());
  if (e != cudaSuccess) return (int)e;
  GRM_LAUNCH_RET();
}

// part_val / part_idx: M*64 floats / ints of scratch; counters: M zeroed uints (left at zero).
GRM_API int grm_argmax(const void* logits, void* out_id, void* out_val, void* part_val, void* part_idx, void* counters, int M,
                       int V, int ld, void* stream) {
  if (!part_val || !part_idx || !counters || M < 1) return -2;
  dim3 grid(kArgChunks, M);
  cudaError_t e = grm_launch_pdl(GRM_PDL_MISC, argmax_kernel, grid, dim3(256), 0, (cudaStream_t)stream, (const float*)logits, (int*)out_id, (float*)out_val,
                                 (float*)part_val, (int*)part_idx, (unsigned int*)counters, V, ld);
  if (e != cudaSuccess) return (int)e;
  GRM_LAUNCH_RET();
}

GRM_API int grm_probe(const void* x, long n, void* out4, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  cudaMemsetAsync(out4, 0, 4 * sizeof(float), st);
  probe_kernel<<<148, 256, 0, st>>>((const float*)x, n, (float*)out4);
  GRM_LAUNCH_RET();
}

GRM_API int grm_f32_to_bf16(const void* in, void* out, long n, void* stream) {
  f32_to_bf16_kernel<<<148 * 4, 256, 0, (cudaStream_t)stream>>>((const float*)in, (bf16*)out, n);
  GRM_LAUNCH_RET();
}

GRM_API int grm_incr_pos(void* pos, int n, int by, void* stream) {
  incr_pos_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>((int*)pos, n, by);
  GRM_LAUNCH_RET();
}
