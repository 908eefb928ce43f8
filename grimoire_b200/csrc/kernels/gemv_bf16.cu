// gemv_bf16: Y[M<=8][N] = X[M][K] . W[N][K]^T for unquantized bf16 weights (tied lm_head, MoE
// router, DeltaNet a/b gate projections, MTP fc).  Reference: bf16_smallm_impl
// (src/gemm_fast.cpp:4220) and the bf16 row of gemv_impl (src/gemv_decode.cpp:77-347).
// Bandwidth-bound: one warp per output row, 16-byte weight loads (512 B per warp request),
// activations re-read from L1/L2, fp32 accumulate, warp-shuffle reduce.  Larger M goes to the
// tcgen05 GEMM.
#include "common.cuh"

namespace {

template <int MB>
__global__ void __launch_bounds__(256) gemv_bf16_kernel(const bf16* __restrict__ w, const bf16* __restrict__ x, void* __restrict__ out,
                                                        int M, int N, int K, int ldw, int ldx, int ldo, int out_f32,
                                                        int accumulate) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= N) return;
  const bf16* wr = w + (size_t)warp * ldw;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 wv = ldg_stream_v4(wr + k);
    const float wf[8] = {bf16lo_to_f(wv.x), bf16hi_to_f(wv.x), bf16lo_to_f(wv.y), bf16hi_to_f(wv.y),
                         bf16lo_to_f(wv.z), bf16hi_to_f(wv.z), bf16lo_to_f(wv.w), bf16hi_to_f(wv.w)};
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (m < M) {
        const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k);
        acc[m] += wf[0] * bf16lo_to_f(xv.x) + wf[1] * bf16hi_to_f(xv.x) + wf[2] * bf16lo_to_f(xv.y) + wf[3] * bf16hi_to_f(xv.y) +
                  wf[4] * bf16lo_to_f(xv.z) + wf[5] * bf16hi_to_f(xv.z) + wf[6] * bf16lo_to_f(xv.w) + wf[7] * bf16hi_to_f(xv.w);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    const float s = warp_sum(acc[m]);
    if (lane == 0 && m < M) {
      const size_t o = (size_t)m * ldo + warp;
      if (out_f32) {
        float* p = reinterpret_cast<float*>(out) + o;
        *p = accumulate ? *p + s : s;
      } else {
        reinterpret_cast<bf16*>(out)[o] = __float2bfloat16(s);
      }
    }
  }
}

// Few rows (a router, the a | b gate projection of a DeltaNet layer): one CTA per output row, the 8 warps split K, so a
// row's weights are fetched by 256 threads at once instead of by one warp in 20 dependent rounds.
template <int MB>
__global__ void __launch_bounds__(256) gemv_bf16_rowcta_kernel(const bf16* __restrict__ w, const bf16* __restrict__ x, void* __restrict__ out,
                                                               int M, int N, int K, int ldw, int ldx, int ldo, int out_f32,
                                                               int accumulate) {
  __shared__ float part[8][MB];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bf16* wr = w + (size_t)row * ldw;
  float acc[MB];
#pragma unroll
  for (int m = 0; m < MB; ++m) acc[m] = 0.f;
#pragma unroll 4
  for (int k = tid * 8; k < K; k += 2048) {
    const uint4 wv = ldg_stream_v4(wr + k);
    const float wf[8] = {bf16lo_to_f(wv.x), bf16hi_to_f(wv.x), bf16lo_to_f(wv.y), bf16hi_to_f(wv.y),
                         bf16lo_to_f(wv.z), bf16hi_to_f(wv.z), bf16lo_to_f(wv.w), bf16hi_to_f(wv.w)};
#pragma unroll
    for (int m = 0; m < MB; ++m) {
      if (m < M) {
        const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k);
        acc[m] += wf[0] * bf16lo_to_f(xv.x) + wf[1] * bf16hi_to_f(xv.x) + wf[2] * bf16lo_to_f(xv.y) + wf[3] * bf16hi_to_f(xv.y) +
                  wf[4] * bf16lo_to_f(xv.z) + wf[5] * bf16hi_to_f(xv.z) + wf[6] * bf16lo_to_f(xv.w) + wf[7] * bf16hi_to_f(xv.w);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MB; ++m) {
    const float s = warp_sum(acc[m]);
    if (lane == 0) part[warp][m] = s;
  }
  __syncthreads();
  if (tid < MB && tid < M) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += part[i][tid];           // fixed order: the result does not depend on timing
    const size_t o = (size_t)tid * ldo + row;
    if (out_f32) {
      float* p = reinterpret_cast<float*>(out) + o;
      *p = accumulate ? *p + s : s;
    } else {
      reinterpret_cast<bf16*>(out)[o] = __float2bfloat16(s);
    }
  }
}

}  // namespace

GRM_API int grm_gemv_bf16(const void* w, const void* x, void* out, int M, int N, int K, int ldw, int ldx, int ldo, int out_f32,
                          int accumulate, void* stream) {
  if (M < 1 || M > 8 || (K & 7) || (ldw & 7) || (ldx & 7)) return -2;
  const int threads = 256;
  const long blocks = ((long)N * 32 + threads - 1) / threads;
  cudaStream_t st = (cudaStream_t)stream;
  if (N <= 1024 && K >= 2048) {
    if (M <= 1)
      gemv_bf16_rowcta_kernel<1><<<N, 256, 0, st>>>((const bf16*)w, (const bf16*)x, out, M, N, K, ldw, ldx, ldo, out_f32, accumulate);
    else if (M <= 4)
      gemv_bf16_rowcta_kernel<4><<<N, 256, 0, st>>>((const bf16*)w, (const bf16*)x, out, M, N, K, ldw, ldx, ldo, out_f32, accumulate);
    else
      gemv_bf16_rowcta_kernel<8><<<N, 256, 0, st>>>((const bf16*)w, (const bf16*)x, out, M, N, K, ldw, ldx, ldo, out_f32, accumulate);
    GRM_LAUNCH_RET();
  }
  if (M <= 1)
    gemv_bf16_kernel<1><<<(unsigned)blocks, threads, 0, st>>>((const bf16*)w, (const bf16*)x, out, M, N, K, ldw, ldx, ldo, out_f32, accumulate);
  else if (M <= 4)
    gemv_bf16_kernel<4><<<(unsigned)blocks, threads, 0, st>>>((const bf16*)w, (const bf16*)x, out, M, N, K, ldw, ldx, ldo, out_f32, accumulate);
  else
    gemv_bf16_kernel<8><<<(unsigned)blocks, threads, 0, st>>>((const bf16*)w, (const bf16*)x, out, M, N, K, ldw, ldx, ldo, out_f32, accumulate);
  GRM_LAUNCH_RET();
}
