// Gated DeltaNet on sm_100a: causal conv (kernel 4) + SiLU over the packed q|k|v channels, and the
// gated delta-rule recurrence with its fused gates, q/k L2 norm and gated output RMSNorm.
//
// Reference kernels: launch_causal_conv1d* (src/deltanet.cpp:629-700, src/prefill.cpp:1049-1260),
// dn_step_sg / launch_deltanet_step(_rows) (src/deltanet.cpp:67-355), the chunked prefill scans
// dn_xmx_* / dn_chunk_* (src/gemm_fast.cpp:2690-3362), launch_deltanet_gates, launch_l2norm_heads,
// launch_rmsnorm_gate_silu (src/ops.cpp:548-869).  Recurrence per value head (q/k head = v head /
// (Hv/Hk)):  w = S k;  S = a S + beta (v - a w) k^T;  o = (S q) / sqrt(Dk).
//
// One kernel serves decode rows, verify blocks and prompt chunks: the rows of a call are grouped
// into "runs" (consecutive positions of one conversation slot); a CTA owns (run, value head), keeps
// the whole 128 x 128 fp32 state of that head in registers (64 values per thread), walks the run's
// rows in order and writes the state back once.  Everything that used to be a separate launch in
// the reference (gates, L2 norms, gated output norm) happens on the row while it is in shared memory.
// This is the sequential-in-time form; the chunk-64 tensor-core form is future work.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------
// causal conv (k = 4) + SiLU.  x [M][C] bf16, w [C][4] fp32 (w[3] multiplies the current token),
// ring_in / ring_out [slots][C][3] fp32 (older tokens, oldest first; double-buffered by the caller).
// Rows of one slot are contiguous and at consecutive positions.  grid (C/256, ceil(M/kConvRows)).
// ---------------------------------------------------------------------------------------------
constexpr int kConvRows = 32;

__global__ void __launch_bounds__(256) conv4_silu_kernel(const bf16* __restrict__ x, const float* __restrict__ w,
                                                         const float* __restrict__ ring_in, float* __restrict__ ring_out,
                                                         const int* __restrict__ row_seq, const int* __restrict__ row_pos,
                                                         bf16* __restrict__ y, int M, int C, int ldx, int ldy) {
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  const int m0 = blockIdx.y * kConvRows, m1 = min(M, m0 + kConvRows);
  const float w0 = w[c * 4 + 0], w1 = w[c * 4 + 1], w2 = w[c * 4 + 2], w3 = w[c * 4 + 3];
  for (int m = m0; m < m1; ++m) {
    const int slot = row_seq[m], pos = row_pos[m];
    float hist[3];   // tokens t-3, t-2, t-1
#pragma unroll
    for (int j = 1; j <= 3; ++j) {
      const int pm = m - j;
      if (pm >= 0 && row_seq[pm] == slot && row_pos[pm] == pos - j) {
        hist[3 - j] = __bfloat162float(x[(size_t)pm * ldx + c]);
      } else {
        // row m-j is not in this call: take it from the ring.  The ring holds the 3 tokens before the
        // first row of this slot in this call; count how many in-call rows precede row m.
        int have = 0;
        while (have < 3 && m - 1 - have >= 0 && row_seq[m - 1 - have] == slot && row_pos[m - 1 - have] == pos - 1 - have) ++have;
        const int back = j - have;           // 1 = newest ring entry
        hist[3 - j] = (back >= 1 && back <= 3) ? ring_in[((size_t)slot * C + c) * 3 + (3 - back)] : 0.f;
      }
    }
    const float cur = __bfloat162float(x[(size_t)m * ldx + c]);
    const float v = hist[0] * w0 + hist[1] * w1 + hist[2] * w2 + cur * w3;
    y[(size_t)m * ldy + c] = __float2bfloat16(silu_f(v));
    const bool tail = (m + 1 >= M) || row_seq[m + 1] != slot;
    if (tail) {
      float* ro = ring_out + ((size_t)slot * C + c) * 3;
      ro[0] = hist[1]; ro[1] = hist[2]; ro[2] = cur;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// gated delta rule over runs of rows
// ---------------------------------------------------------------------------------------------
struct GdnParams {
  const bf16* qkv;        // [M][ld_qkv]: conv+SiLU output, channels [q: Hk*Dk | k: Hk*Dk | v: Hv*Dv]
  int ld_qkv;
  const float* ab;        // [M][2*Hv] fp32: a_raw | b_raw (outputs of the in_proj_a / in_proj_b projections)
  int ld_ab;
  const bf16* z;          // [M][Hv*Dv] gate input of the output norm
  int ld_z;
  const float* A_log;     // [Hv]
  const float* dt_bias;   // [Hv]
  const float* norm_w;    // [Dv]
  float norm_eps;
  float* state;           // [slots][Hv][Dv][Dk] fp32
  const int* run_slot;    // [runs]
  const int* run_start;   // [runs] first row of the run
  const int* run_len;     // [runs]
  bf16* out;              // [M][Hv*Dv]
  int ld_out;
  int Hk, Hv;
};

constexpr int D = 128;          // Dk = Dv = 128
constexpr int kGdnThreads = 256;

__global__ void __launch_bounds__(kGdnThreads) gdn_runs_kernel(const GdnParams p) {
  __shared__ float sq[D], sk[D], sv[D], so[D];
  __shared__ float sred[16];
  __shared__ float sgate[2];
  const int run = blockIdx.x, vh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int slot = p.run_slot[run], r0 = p.run_start[run], n = p.run_len[run];
  const int kh = vh / (p.Hv / p.Hk);
  const int dv = tid >> 1, part = tid & 1;          // thread owns S[dv][part*64 .. part*64+63]
  float S[64];
  float* sp = p.state + (((size_t)slot * p.Hv + vh) * D + dv) * D + part * 64;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float4 t4 = reinterpret_cast<const float4*>(sp)[i];
    S[4 * i] = t4.x; S[4 * i + 1] = t4.y; S[4 * i + 2] = t4.z; S[4 * i + 3] = t4.w;
  }
  const float neg_expA = -__expf(p.A_log[vh]);
  const float dtb = p.dt_bias[vh];
  const float inv_sqrt_d = rsqrtf((float)D);
  const int qoff = kh * D, koff = p.Hk * D + kh * D, voff = 2 * p.Hk * D + vh * D;

  for (int i = 0; i < n; ++i) {
    const int row = r0 + i;
    const bf16* xr = p.qkv + (size_t)row * p.ld_qkv;
    // ---- stage q, k, v; L2-normalise q and k; gates ----
    float val = 0.f, ssq = 0.f;
    if (tid < D) { val = __bfloat162float(xr[qoff + tid]); ssq = val * val; }
    else { val = __bfloat162float(xr[koff + tid - D]); ssq = val * val; }
    ssq = warp_sum(ssq);
    if (lane == 0) sred[warp] = ssq;                 // warps 0-3: q, 4-7: k
    if (tid < D) sv[tid] = __bfloat162float(xr[voff + tid]);
    if (tid == 0) {
      const float a_raw = p.ab[(size_t)row * p.ld_ab + vh], b_raw = p.ab[(size_t)row * p.ld_ab + p.Hv + vh];
      const float xs = a_raw + dtb;
      const float sp_ = xs > 20.f ? xs : log1pf(__expf(xs));      // softplus
      sgate[0] = __expf(neg_expA * sp_);                          // a
      sgate[1] = sigmoid_f(b_raw);                                // beta
    }
    __syncthreads();
    {
      const float tot = (tid < D) ? (sred[0] + sred[1] + sred[2] + sred[3]) : (sred[4] + sred[5] + sred[6] + sred[7]);
      const float nv = val * rsqrtf(tot + 1e-6f);
      if (tid < D) sq[tid] = nv; else sk[tid - D] = nv;
    }
    __syncthreads();
    const float a = sgate[0], beta = sgate[1];
    // ---- w = S k ----
    float w = 0.f;
#pragma unroll
    for (int j = 0; j < 64; ++j) w = fmaf(S[j], sk[part * 64 + j], w);
    w += __shfl_xor_sync(0xffffffffu, w, 1);
    const float upd = beta * (sv[dv] - a * w);
    // ---- S = a S + upd k^T ; o = S q ----
    float o = 0.f;
#pragma unroll
    for (int j = 0; j < 64; ++j) {
      S[j] = fmaf(a, S[j], upd * sk[part * 64 + j]);
      o = fmaf(S[j], sq[part * 64 + j], o);
    }
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o *= inv_sqrt_d;
    // ---- gated output norm: rms(o) * w * silu(z) ----
    float oss = (part == 0) ? o * o : 0.f;
    oss = warp_sum(oss);
    if (lane == 0) sred[8 + warp] = oss;
    if (part == 0) so[dv] = o;
    __syncthreads();
    if (tid < D) {
      float tot = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < 8; ++w8) tot += sred[8 + w8];
      const float r = rsqrtf(tot / (float)D + p.norm_eps);
      const float zz = __bfloat162float(p.z[(size_t)row * p.ld_z + vh * D + tid]);
      p.out[(size_t)row * p.ld_out + vh * D + tid] = __float2bfloat16(so[tid] * r * p.norm_w[tid] * silu_f(zz));
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 16; ++i)
    reinterpret_cast<float4*>(sp)[i] = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
}

}  // namespace

GRM_API int grm_conv4_silu(const void* x, const void* w, const void* ring_in, void* ring_out, const void* row_seq,
                           const void* row_pos, void* y, int M, int C, int ldx, int ldy, void* stream) {
  if (M < 1 || C < 1) return -2;
  dim3 grid((C + 255) / 256, (M + kConvRows - 1) / kConvRows);
  conv4_silu_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const float*)w, (const float*)ring_in, (float*)ring_out,
                                                            (const int*)row_seq, (const int*)row_pos, (bf16*)y, M, C, ldx, ldy);
  GRM_LAUNCH_RET();
}

// head dims are fixed at Dk = Dv = 128.  runs: rows grouped by conversation slot (consecutive positions).
GRM_API int grm_gdn_runs(const void* qkv, int ld_qkv, const void* ab, int ld_ab, const void* z, int ld_z, const void* A_log,
                         const void* dt_bias, const void* norm_w, float norm_eps, void* state, const void* run_slot,
                         const void* run_start, const void* run_len, int n_runs, void* out, int ld_out, int Hk, int Hv,
                         int Dk, int Dv, void* stream) {
  if (Dk != D || Dv != D || n_runs < 1 || Hv % Hk) return -2;
  GdnParams p;
  p.qkv = (const bf16*)qkv; p.ld_qkv = ld_qkv; p.ab = (const float*)ab; p.ld_ab = ld_ab; p.z = (const bf16*)z; p.ld_z = ld_z;
  p.A_log = (const float*)A_log; p.dt_bias = (const float*)dt_bias; p.norm_w = (const float*)norm_w; p.norm_eps = norm_eps;
  p.state = (float*)state; p.run_slot = (const int*)run_slot; p.run_start = (const int*)run_start; p.run_len = (const int*)run_len;
  p.out = (bf16*)out; p.ld_out = ld_out; p.Hk = Hk; p.Hv = Hv;
  dim3 grid(n_runs, Hv);
  gdn_runs_kernel<<<grid, kGdnThreads, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}
