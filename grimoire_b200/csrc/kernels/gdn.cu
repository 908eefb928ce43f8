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


// ---------------------------------------------------------------------------------------------
// Chunked form of the same recurrence for prompt chunks (64 tokens per chunk).
//
// With u_t = beta_t (v_t - a_t S_{t-1} k_t) the step is S_t = a_t S_{t-1} + u_t k_t^T, so inside a chunk
// (gamma_t = prod_{j<=t} a_j, S_0 the state at the chunk start)
//     (I + L) U = diag(beta) (V - diag(gamma) K S_0^T),   L_tj = beta_t (gamma_t/gamma_j) (k_t.k_j), j < t
//     O = (diag(gamma) Q S_0^T + M U) / sqrt(Dk),          M_tj = (gamma_t/gamma_j) (q_t.k_j),       j <= t
//     S_C = gamma_C S_0 + U^T diag(gamma_C/gamma) K
// (the WY / UT-transform form of the gated delta rule; every ratio gamma_t/gamma_j is <= 1).  All
// products are fp32.  A CTA owns (run, v head, a quarter of Dv): thread = (dv, quarter of Dk) keeps its 32
// state values in registers across the whole run, the chunk's K / Q rows and the two C x C matrices sit
// in shared memory, the triangular system is solved by forward substitution with the 64 unknowns of a
// dv column spread over the 4 threads of its quad.  The output norm needs all of Dv, so the raw outputs
// go to an fp32 scratch and gdn_gated_norm_kernel finishes them.
// ---------------------------------------------------------------------------------------------
constexpr int CH = 64;             // chunk length
constexpr int DVL = 32;            // Dv rows per CTA
constexpr int kChThreads = 128;
constexpr int LDK = D + 4;         // padded row pitch of the K / Q tiles
constexpr int UP = DVL + 8;        // row pitch of the [token][dv] tiles: the four j-phases of a quad hit different banks

struct GdnChunkParams {
  const bf16* qkv; int ld_qkv;
  const float* ab; int ld_ab;
  const float* A_log; const float* dt_bias;
  float* state;
  const int* run_slot; const int* run_start; const int* run_len;
  float* o_raw; int ld_o;          // fp32 [M][Hv*Dv], un-normalised outputs
  int Hk, Hv;
  long long* tl;                   // debug: clock64 stamps of CTA (0, 0, 0), 8 per chunk (null: off)
};

static_assert(2 * CH * (CH + 1) <= CH * LDK, "L and M must fit in the Q tile");

__global__ void __launch_bounds__(kChThreads, 2) gdn_chunked_kernel(const GdnChunkParams p) {
  extern __shared__ __align__(16) float smc[];
  float* Ks = smc;                          // [CH][LDK]
  float* Qs = Ks + CH * LDK;                // [CH][LDK]
  float* Vs = Qs + CH * LDK;                // [CH][DVL]
  // the two C x C matrices live where the Q tile was: Q is last read (K S_0^T / Q S_0^T and q.k below) before they are
  // written, which keeps a CTA under half of an SM's shared memory so that two CTAs share an SM
  float* Lm = Qs;                           // [CH][CH + 1]
  float* Mm = Lm + CH * (CH + 1);           // [CH][CH + 1]
  float* Us = Vs + CH * DVL;                // [CH][DVL + 1]
  float* Ps = Us + CH * UP;          // [CH][DVL + 1]  (K S_0^T) for this CTA's dv rows
  float* Rs = Ps + CH * UP;          // [CH][DVL + 1]  (Q S_0^T)
  float* Gs = Rs + CH * UP;          // [CH] cumulative log decay
  float* Bs = Gs + CH;                      // [CH] beta
  const int run = blockIdx.x, vh = blockIdx.y, dvs = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int dvl = tid >> 2, part = tid & 3;             // thread = (dv row, quarter of Dk)
  const int slot = p.run_slot[run], r0 = p.run_start[run], n = p.run_len[run];
  const int kh = vh / (p.Hv / p.Hk);
  const int dv = dvs * DVL + dvl;
  float S[32];
  // thread `part` owns the k columns 16 i + 4 part + (0..3), i = 0..7: the four threads of a quad read four
  // consecutive 16-byte words of a K / Q row, which keeps the shared-memory reads free of bank conflicts
  float* sp = p.state + (((size_t)slot * p.Hv + vh) * D + dv) * D + part * 4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 t4 = reinterpret_cast<const float4*>(sp)[4 * i];
    S[4 * i] = t4.x; S[4 * i + 1] = t4.y; S[4 * i + 2] = t4.z; S[4 * i + 3] = t4.w;
  }
  const float neg_expA = -__expf(p.A_log[vh]);
  const float dtb = p.dt_bias[vh];
  const float inv_sqrt_d = rsqrtf((float)D);
  const int qoff = kh * D, koff = p.Hk * D + kh * D, voff = 2 * p.Hk * D + vh * D + dvs * DVL;

  for (int c0 = 0; c0 < n; c0 += CH) {
    const int nc = min(CH, n - c0);
    __syncthreads();
    // ---- stage the chunk: L2-normalised q / k rows (a warp per token), the v slice, gates ----
    // a warp owns 16 tokens (t = warp + 4 i); the global loads of 8 tokens are issued before any reduction
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint2 qa[8], ka[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int t = warp + 4 * (half * 8 + i);
        qa[i] = ka[i] = make_uint2(0u, 0u);
        if (t < nc) {
          const bf16* xr = p.qkv + (size_t)(r0 + c0 + t) * p.ld_qkv;
          qa[i] = *reinterpret_cast<const uint2*>(xr + qoff + lane * 4);
          ka[i] = *reinterpret_cast<const uint2*>(xr + koff + lane * 4);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int t = warp + 4 * (half * 8 + i);
        const float4 qv = make_float4(bf16lo_to_f(qa[i].x), bf16hi_to_f(qa[i].x), bf16lo_to_f(qa[i].y), bf16hi_to_f(qa[i].y));
        const float4 kv = make_float4(bf16lo_to_f(ka[i].x), bf16hi_to_f(ka[i].x), bf16lo_to_f(ka[i].y), bf16hi_to_f(ka[i].y));
        const float qs = warp_sum(qv.x * qv.x + qv.y * qv.y + qv.z * qv.z + qv.w * qv.w);
        const float ks = warp_sum(kv.x * kv.x + kv.y * kv.y + kv.z * kv.z + kv.w * kv.w);
        const float qr = t < nc ? rsqrtf(qs + 1e-6f) : 0.f, kr = t < nc ? rsqrtf(ks + 1e-6f) : 0.f;
        *reinterpret_cast<float4*>(Qs + t * LDK + lane * 4) = make_float4(qv.x * qr, qv.y * qr, qv.z * qr, qv.w * qr);
        *reinterpret_cast<float4*>(Ks + t * LDK + lane * 4) = make_float4(kv.x * kr, kv.y * kr, kv.z * kr, kv.w * kr);
      }
    }
    for (int i = tid; i < CH * DVL; i += kChThreads) {
      const int t = i / DVL, d = i - t * DVL;
      Vs[i] = t < nc ? __bfloat162float(p.qkv[(size_t)(r0 + c0 + t) * p.ld_qkv + voff + d]) : 0.f;
    }
    if (tid < CH) {
      float la = 0.f, be = 0.f;
      if (tid < nc) {
        const size_t row = (size_t)(r0 + c0 + tid);
        const float xs = p.ab[row * p.ld_ab + vh] + dtb;
        const float spl = xs > 20.f ? xs : log1pf(__expf(xs));
        la = neg_expA * spl;                              // log a_t  (<= 0)
        be = sigmoid_f(p.ab[row * p.ld_ab + p.Hv + vh]);
      }
      Gs[tid] = la; Bs[tid] = be;
    }
    __syncthreads();
    if (tid == 0) {
      float acc = 0.f;
      for (int t = 0; t < CH; ++t) { acc += Gs[t]; Gs[t] = acc; }
    }
    // ---- p_t = (K S_0^T)[t][dv], r_t = (Q S_0^T)[t][dv]: partial over this thread's 32 k, quad-reduced; thread
    //      `part` keeps the values of its 16 tokens ----
    // (results go to shared memory so the token loops below stay rolled: the code of a chunk fits the
    //  instruction cache)
#pragma unroll 2
    for (int t = 0; t < CH; ++t) {
      float a1 = 0.f, a2 = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 kx = *reinterpret_cast<const float4*>(Ks + t * LDK + i * 16 + part * 4);
        const float4 qx = *reinterpret_cast<const float4*>(Qs + t * LDK + i * 16 + part * 4);
        a1 = fmaf(S[4 * i], kx.x, fmaf(S[4 * i + 1], kx.y, fmaf(S[4 * i + 2], kx.z, fmaf(S[4 * i + 3], kx.w, a1))));
        a2 = fmaf(S[4 * i], qx.x, fmaf(S[4 * i + 1], qx.y, fmaf(S[4 * i + 2], qx.z, fmaf(S[4 * i + 3], qx.w, a2))));
      }
      a1 += __shfl_xor_sync(0xffffffffu, a1, 1); a1 += __shfl_xor_sync(0xffffffffu, a1, 2);
      a2 += __shfl_xor_sync(0xffffffffu, a2, 1); a2 += __shfl_xor_sync(0xffffffffu, a2, 2);
      if (part == 0) { Ps[t * UP + dvl] = a1; Rs[t * UP + dvl] = a2; }
    }
    // ---- k_t.k_j and q_t.k_j: thread = (row t, half of the j range) ----
    {
      const int t = tid >> 1, jh = (tid & 1) * 32;
      float akk[32], aqk[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) { akk[j] = 0.f; aqk[j] = 0.f; }
      for (int kb = 0; kb < D / 4; ++kb) {
        const float4 kt = *reinterpret_cast<const float4*>(Ks + t * LDK + kb * 4);
        const float4 qt = *reinterpret_cast<const float4*>(Qs + t * LDK + kb * 4);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float4 kj = *reinterpret_cast<const float4*>(Ks + (jh + j) * LDK + kb * 4);
          akk[j] = fmaf(kt.x, kj.x, fmaf(kt.y, kj.y, fmaf(kt.z, kj.z, fmaf(kt.w, kj.w, akk[j]))));
          aqk[j] = fmaf(qt.x, kj.x, fmaf(qt.y, kj.y, fmaf(qt.z, kj.z, fmaf(qt.w, kj.w, aqk[j]))));
        }
      }
      __syncthreads();                                     // Gs is complete; nobody reads the Q tile any more
      const float gt = Gs[t], bt = Bs[t];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int jj = jh + j;
        const float ratio = jj <= t ? __expf(gt - Gs[jj]) : 0.f;
        Lm[t * (CH + 1) + jj] = jj < t ? bt * ratio * akk[j] : 0.f;
        Mm[t * (CH + 1) + jj] = ratio * aqk[j];
      }
    }
    __syncthreads();                                       // Lm / Mm / Ps / Rs are complete
    // ---- forward substitution for this dv column of U (in Us); the four threads of a quad split the sum over j ----
#pragma unroll 1
    for (int t = 0; t < CH; ++t) {
      float sacc = 0.f;
      for (int j = part; j < t; j += 4) sacc = fmaf(Lm[t * (CH + 1) + j], Us[j * UP + dvl], sacc);
      sacc += __shfl_xor_sync(0xffffffffu, sacc, 1); sacc += __shfl_xor_sync(0xffffffffu, sacc, 2);
      if (part == 0) Us[t * UP + dvl] = Bs[t] * (Vs[t * DVL + dvl] - __expf(Gs[t]) * Ps[t * UP + dvl]) - sacc;
      __syncwarp();
    }
    // ---- outputs ----
#pragma unroll 1
    for (int t = 0; t < nc; ++t) {
      float oacc = 0.f;
      for (int j = part; j <= t; j += 4) oacc = fmaf(Mm[t * (CH + 1) + j], Us[j * UP + dvl], oacc);
      oacc += __shfl_xor_sync(0xffffffffu, oacc, 1); oacc += __shfl_xor_sync(0xffffffffu, oacc, 2);
      if (part == 0) p.o_raw[(size_t)(r0 + c0 + t) * p.ld_o + vh * D + dv] = (__expf(Gs[t]) * Rs[t * UP + dvl] + oacc) * inv_sqrt_d;
    }
    // ---- state: S = gamma_C S + sum_j (gamma_C / gamma_j) u_j k_j^T over this thread's 32 k ----
    const float gC = Gs[CH - 1];
    const float gamC = __expf(gC);
#pragma unroll
    for (int i = 0; i < 32; ++i) S[i] *= gamC;
    for (int j = 0; j < CH; ++j) {
      const float cu = __expf(gC - Gs[j]) * Us[j * UP + dvl];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 kx = *reinterpret_cast<const float4*>(Ks + j * LDK + i * 16 + part * 4);
        S[4 * i] = fmaf(cu, kx.x, S[4 * i]); S[4 * i + 1] = fmaf(cu, kx.y, S[4 * i + 1]);
        S[4 * i + 2] = fmaf(cu, kx.z, S[4 * i + 2]); S[4 * i + 3] = fmaf(cu, kx.w, S[4 * i + 3]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i)
    reinterpret_cast<float4*>(sp)[4 * i] = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
}

// ---------------------------------------------------------------------------------------------
// The chunked form with its matrix products on the tensor cores (mma.sync m16n8k8, tf32 operands, fp32 accumulation): the
// default.  Same algebra, same CTA = (run, v head, 32 Dv rows), 4 warps.  Per 64-token chunk
//   P = K S_0^T, R = Q S_0^T      [t][dv]  warp w owns token rows 16 w .. 16 w + 15; S_0 is read from a shared-memory copy
//   K K^T, Q K^T                  [t][j]   same rows, only the 8-column tiles at or below the diagonal; shares the K / Q
//                                          fragments of the first product (one pass over k)
//   forward substitution for U    (scalar, a quad per dv column, as in the fp32 kernel)
//   O^T = U^T M^T                 [dv][t]  warp w owns token tiles w and 7 - w (balanced under the causal cut)
//   S = gamma_C S_0 + (E U)^T K   [dv][k]  the state lives in the accumulator registers of this product across the run:
//                                          warp w owns k in [32 w, 32 w + 32)
// Shared memory: K and Q tiles (tf32-rounded at staging), L and M where Q was, the S_0 copy where V and U are staged
// afterwards -- 106 KB, two CTAs per SM.  Operand rounding is tf32 (10-bit mantissa; the reference's chunk kernel uses
// bf16 operands, src/gemm_fast.cpp:3021-3362); the state and every accumulation stay fp32.
// ---------------------------------------------------------------------------------------------
constexpr int PL = CH + 4;         // row pitch of L and of M: both are read as MMA operands (8 rows x 4 columns hit 32 banks)
constexpr int PM = CH + 4;
constexpr int QREG = (CH * PL + CH * PM > CH * LDK) ? (CH * PL + CH * PM) : (CH * LDK);      // the Q tile, then L and M
static_assert(DVL * LDK <= CH * DVL + CH * UP, "the S_0 copy must fit where V and U are staged");

__device__ __forceinline__ uint32_t tf32r(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float tf32f(float x) { return __uint_as_float(tf32r(x)); }
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(kChThreads, 2) gdn_chunked_mma_kernel(const GdnChunkParams p) {
  extern __shared__ __align__(16) float smc[];
  float* Ks = smc;                          // [CH][LDK]  tf32-rounded, L2-normalised k rows
  float* Qs = Ks + CH * LDK;                // [CH][LDK]  same for q; dead after the first pass over k
  float* Lm = Qs;                           // [CH][PL]
  float* Mm = Lm + CH * PL;                 // [CH][PM]
  float* Vs = Qs + QREG;                    // [CH][DVL]
  float* Us = Vs + CH * DVL;                // [CH][UP]
  float* Ss = Vs;                           // [DVL][LDK] copy of S_0 for the first pass (V and U are staged after it)
  float* Ps = Us + CH * UP;                 // [CH][UP]  K S_0^T
  float* Rs = Ps + CH * UP;                 // [CH][UP]  Q S_0^T
  float* Gs = Rs + CH * UP;                 // [CH] cumulative log decay
  float* Bs = Gs + CH;                      // [CH] beta
  float* Es = Bs + CH;                      // [CH] gamma_C / gamma_j
  bf16* Vh = reinterpret_cast<bf16*>(Es + CH);   // [CH][DVL] this CTA's v slice as loaded (read once, by the substitution's right side)
  const int run = blockIdx.x, vh = blockIdx.y, dvs = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;               // MMA fragment coordinates
  const int dvl = tid >> 2, part = tid & 3;             // substitution: thread = (dv column, quarter of the j range)
  const int slot = p.run_slot[run], r0 = p.run_start[run], n = p.run_len[run];
  const int kh = vh / (p.Hv / p.Hk);
  // state tile (m = dv tile mt, n = k tile 4 warp + ntl) in accumulator layout: [0],[1] = (dv 16 mt + g, k 8 nt + 2 t4 (+1)),
  // [2],[3] = the same columns of row dv + 8
  float Sr[2][4][4];
  float* sbase = p.state + (((size_t)slot * p.Hv + vh) * D + (size_t)dvs * DVL) * D;
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int ntl = 0; ntl < 4; ++ntl) {
      const int k = 8 * (4 * warp + ntl) + 2 * t4;
      const float2 lo = *reinterpret_cast<const float2*>(sbase + (size_t)(16 * mt + g) * D + k);
      const float2 hi = *reinterpret_cast<const float2*>(sbase + (size_t)(16 * mt + g + 8) * D + k);
      Sr[mt][ntl][0] = lo.x; Sr[mt][ntl][1] = lo.y; Sr[mt][ntl][2] = hi.x; Sr[mt][ntl][3] = hi.y;
    }
  const float neg_expA = -__expf(p.A_log[vh]);
  const float dtb = p.dt_bias[vh];
  const float inv_sqrt_d = rsqrtf((float)D);
  const int qoff = kh * D, koff = p.Hk * D + kh * D, voff = 2 * p.Hk * D + vh * D + dvs * DVL;

  const bool stamp = p.tl != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid == 32;
  for (int c0 = 0; c0 < n; c0 += CH) {
    const int nc = min(CH, n - c0);
    long long* tlc = p.tl + (c0 / CH) * 8;
    __syncthreads();
    if (stamp) tlc[0] = clock64();
    // ---- stage: every global load of the chunk is issued before the first use (v slice, q / k rows); then the
    //      L2-normalised q / k rows (a thread per row), gates, and the S_0 copy ----
    {
      uint2 vv[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int t = (tid >> 3) + 16 * r;
        vv[r] = make_uint2(0u, 0u);
        if (t < nc) vv[r] = *reinterpret_cast<const uint2*>(p.qkv + (size_t)(r0 + c0 + t) * p.ld_qkv + voff + (tid & 7) * 4);
      }
      // q / k rows: a thread owns one whole row (threads 0-63: q of token tid, 64-127: k of token tid - 64), so the sum of
      // squares needs no shuffles and the 16-byte stores of eight neighbouring tokens fall into 32 different banks
      uint4 rw[16];
      const int tok = tid & 63;
      {
        const bf16* xr = p.qkv + (size_t)(r0 + c0 + tok) * p.ld_qkv + (tid < 64 ? qoff : koff);
#pragma unroll
        for (int i = 0; i < 16; ++i) rw[i] = tok < nc ? *reinterpret_cast<const uint4*>(xr + 8 * i) : make_uint4(0u, 0u, 0u, 0u);
      }
      // the next chunk's rows are asked into L2 now, a whole chunk of compute ahead of their use
      if (c0 + CH < n) {
        const int nn = min(CH, n - c0 - CH);
        if (lane < 4) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int t = warp + 4 * i;
            if (t < nn) {
              const bf16* xr = p.qkv + (size_t)(r0 + c0 + CH + t) * p.ld_qkv + ((lane & 2) ? koff : qoff) + (lane & 1) * 64;
              asm volatile("prefetch.global.L2 [%0];" ::"l"(xr));
            }
          }
        }
        if (tid < nn) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.qkv + (size_t)(r0 + c0 + CH + tid) * p.ld_qkv + voff));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.ab + (size_t)(r0 + c0 + CH + tid) * p.ld_ab + vh));
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) *reinterpret_cast<uint2*>(Vh + ((tid >> 3) + 16 * r) * DVL + (tid & 7) * 4) = vv[r];
      {
        float ss0 = 0.f, ss1 = 0.f, ss2 = 0.f, ss3 = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float x0 = bf16lo_to_f(rw[i].x), x1 = bf16hi_to_f(rw[i].x), x2 = bf16lo_to_f(rw[i].y), x3 = bf16hi_to_f(rw[i].y);
          const float x4 = bf16lo_to_f(rw[i].z), x5 = bf16hi_to_f(rw[i].z), x6 = bf16lo_to_f(rw[i].w), x7 = bf16hi_to_f(rw[i].w);
          ss0 = fmaf(x0, x0, fmaf(x4, x4, ss0)); ss1 = fmaf(x1, x1, fmaf(x5, x5, ss1));
          ss2 = fmaf(x2, x2, fmaf(x6, x6, ss2)); ss3 = fmaf(x3, x3, fmaf(x7, x7, ss3));
        }
        const float rn = tok < nc ? rsqrtf((ss0 + ss1) + (ss2 + ss3) + 1e-6f) : 0.f;
        float* dst = (tid < 64 ? Qs : Ks) + tok * LDK;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          *reinterpret_cast<float4*>(dst + 8 * i) = make_float4(tf32f(bf16lo_to_f(rw[i].x) * rn), tf32f(bf16hi_to_f(rw[i].x) * rn),
                                                                tf32f(bf16lo_to_f(rw[i].y) * rn), tf32f(bf16hi_to_f(rw[i].y) * rn));
          *reinterpret_cast<float4*>(dst + 8 * i + 4) = make_float4(tf32f(bf16lo_to_f(rw[i].z) * rn), tf32f(bf16hi_to_f(rw[i].z) * rn),
                                                                    tf32f(bf16lo_to_f(rw[i].w) * rn), tf32f(bf16hi_to_f(rw[i].w) * rn));
        }
      }
    }
    if (tid < CH) {
      float la = 0.f, be = 0.f;
      if (tid < nc) {
        const size_t row = (size_t)(r0 + c0 + tid);
        const float xs = p.ab[row * p.ld_ab + vh] + dtb;
        const float spl = xs > 20.f ? xs : log1pf(__expf(xs));
        la = neg_expA * spl;
        be = sigmoid_f(p.ab[row * p.ld_ab + p.Hv + vh]);
      }
      Gs[tid] = la; Bs[tid] = be;
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int ntl = 0; ntl < 4; ++ntl) {
        const int k = 8 * (4 * warp + ntl) + 2 * t4;
        *reinterpret_cast<float2*>(Ss + (16 * mt + g) * LDK + k) = make_float2(tf32f(Sr[mt][ntl][0]), tf32f(Sr[mt][ntl][1]));
        *reinterpret_cast<float2*>(Ss + (16 * mt + g + 8) * LDK + k) = make_float2(tf32f(Sr[mt][ntl][2]), tf32f(Sr[mt][ntl][3]));
      }
    __syncthreads();
    if (stamp) tlc[1] = clock64();
    if (tid == 0) {
      float acc = 0.f;
      for (int t = 0; t < CH; ++t) { acc += Gs[t]; Gs[t] = acc; }
    }
    // ---- one pass over k: P, R (against S_0) and K K^T, Q K^T (tiles at or below the diagonal) for token rows 16 warp .. ----
    float accP[4][4], accR[4][4], akk[8][4], aqk[8][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { accP[i][j] = 0.f; accR[i][j] = 0.f; }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) { akk[i][j] = 0.f; aqk[i][j] = 0.f; }
    const int nt_hi = 2 * warp + 1;                       // last 8-column tile this warp's rows can see
    {
      const float* ka0 = Ks + (16 * warp + g) * LDK + t4;
      const float* qa0 = Qs + (16 * warp + g) * LDK + t4;
#pragma unroll 2
      for (int ks = 0; ks < D / 8; ++ks) {
        const int k0 = 8 * ks;
        uint32_t aK[4], aQ[4];
        aK[0] = __float_as_uint(ka0[k0]); aK[1] = __float_as_uint(ka0[8 * LDK + k0]);
        aK[2] = __float_as_uint(ka0[k0 + 4]); aK[3] = __float_as_uint(ka0[8 * LDK + k0 + 4]);
        aQ[0] = __float_as_uint(qa0[k0]); aQ[1] = __float_as_uint(qa0[8 * LDK + k0]);
        aQ[2] = __float_as_uint(qa0[k0 + 4]); aQ[3] = __float_as_uint(qa0[8 * LDK + k0 + 4]);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const float* sb = Ss + (8 * nt + g) * LDK + k0 + t4;
          const uint32_t b0 = __float_as_uint(sb[0]), b1 = __float_as_uint(sb[4]);
          mma_tf32(accP[nt], aK, b0, b1);
          mma_tf32(accR[nt], aQ, b0, b1);
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          if (nt <= nt_hi) {
            const float* kb = Ks + (8 * nt + g) * LDK + k0 + t4;
            const uint32_t b0 = __float_as_uint(kb[0]), b1 = __float_as_uint(kb[4]);
            mma_tf32(akk[nt], aK, b0, b1);
            mma_tf32(aqk[nt], aQ, b0, b1);
          }
        }
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int ra = 16 * warp + g, dc = 8 * nt + 2 * t4;
      *reinterpret_cast<float2*>(Ps + ra * UP + dc) = make_float2(accP[nt][0], accP[nt][1]);
      *reinterpret_cast<float2*>(Ps + (ra + 8) * UP + dc) = make_float2(accP[nt][2], accP[nt][3]);
      *reinterpret_cast<float2*>(Rs + ra * UP + dc) = make_float2(accR[nt][0], accR[nt][1]);
      *reinterpret_cast<float2*>(Rs + (ra + 8) * UP + dc) = make_float2(accR[nt][2], accR[nt][3]);
    }
    if (stamp) tlc[2] = clock64();
    __syncthreads();                                       // Gs complete; Q tile and the S_0 copy are dead
    if (stamp) tlc[3] = clock64();
    // ---- L, M into the Q tile; gamma_C / gamma_j ----
    {
      const int ra = 16 * warp + g, rb = ra + 8;
      const float ga = Gs[ra], gb = Gs[rb], ba = Bs[ra], bb = Bs[rb];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (nt <= nt_hi) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int col = 8 * nt + 2 * t4 + e;
            const float gc = Gs[col];
            const float rta = col <= ra ? __expf(ga - gc) : 0.f, rtb = col <= rb ? __expf(gb - gc) : 0.f;
            Lm[ra * PL + col] = col < ra ? ba * rta * akk[nt][e] : 0.f;
            Lm[rb * PL + col] = col < rb ? bb * rtb * akk[nt][2 + e] : 0.f;
            Mm[ra * PM + col] = tf32f(rta * aqk[nt][e]);
            Mm[rb * PM + col] = tf32f(rtb * aqk[nt][2 + e]);
          }
        }
      }
    }
    const float gC = Gs[CH - 1];
    if (tid < CH) Es[tid] = __expf(gC - Gs[tid]);
    __syncthreads();
    if (stamp) tlc[4] = clock64();
    // ---- (I + L) U = rhs, in place in Us, in four blocks of 16 rows.
    //      (a) every warp inverts one 16 x 16 diagonal block exactly (fp32 forward substitution on the matrix: a lane owns
    //          a column of the inverse in registers, the L entries are shared-memory broadcasts, no shuffles) and writes
    //          the inverse over the block; the right side rhs_t = beta_t (v_t - gamma_t p_t) goes into Us meanwhile;
    //      (b) a warp then solves its own 8 dv columns block by block with two small tensor-core products per block,
    //          rhs_b - L_b,<b U_<b and T_bb times that, each as three tf32 products of split operands (fp32 accuracy).
    //      The 64 dependent steps of a plain substitution become 16 + 4. ----
    for (int t = part; t < CH; t += 4) Us[t * UP + dvl] = Bs[t] * (__bfloat162float(Vh[t * DVL + dvl]) - __expf(Gs[t]) * Ps[t * UP + dvl]);
    {
      const int col = lane & 15;
      const float* lb = Lm + (16 * warp) * PL + 16 * warp;
      float Tc[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float a0 = (i == col) ? 1.f : 0.f, a1 = 0.f;
#pragma unroll
        for (int j = 0; j < i; ++j) {
          if (j & 1) a1 = fmaf(-lb[i * PL + j], Tc[j], a1);
          else a0 = fmaf(-lb[i * PL + j], Tc[j], a0);
        }
        Tc[i] = a0 + a1;
      }
      __syncwarp();                                        // every lane has read the block before it is overwritten
      if (lane < 16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) Lm[(16 * warp + i) * PL + 16 * warp + col] = Tc[i];
      }
    }
    __syncthreads();                                       // the four inverses and the right sides are in place
#pragma unroll 1
    for (int blk = 0; blk < CH / 16; ++blk) {
      float* ur = Us + (16 * blk + g) * UP + 8 * warp + 2 * t4;
      float c[4] = {ur[0], ur[1], ur[8 * UP], ur[8 * UP + 1]};
      const float* la = Lm + (16 * blk + g) * PL + t4;
      for (int ks = 0; ks < 2 * blk; ++ks) {               // c -= L[block rows][earlier rows] U[earlier rows]
        const int j0 = 8 * ks;
        const float av[4] = {-la[j0], -la[8 * PL + j0], -la[j0 + 4], -la[8 * PL + j0 + 4]};
        const float* ub = Us + (j0 + t4) * UP + 8 * warp + g;
        const float bv0 = ub[0], bv1 = ub[4 * UP];
        uint32_t ah[4], al[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) { ah[e] = tf32r(av[e]); al[e] = tf32r(av[e] - __uint_as_float(ah[e])); }
        const uint32_t bh0 = tf32r(bv0), bh1 = tf32r(bv1);
        const uint32_t bl0 = tf32r(bv0 - __uint_as_float(bh0)), bl1 = tf32r(bv1 - __uint_as_float(bh1));
        mma_tf32(c, al, bh0, bh1);
        mma_tf32(c, ah, bl0, bl1);
        mma_tf32(c, ah, bh0, bh1);
      }
      __syncwarp();
      ur[0] = c[0]; ur[1] = c[1]; ur[8 * UP] = c[2]; ur[8 * UP + 1] = c[3];
      __syncwarp();
      float u[4] = {0.f, 0.f, 0.f, 0.f};
      const float* ta = Lm + (16 * blk + g) * PL + 16 * blk + t4;
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {                     // U_b = T_bb (that)
        const int j0 = 8 * ks;
        const float av[4] = {ta[j0], ta[8 * PL + j0], ta[j0 + 4], ta[8 * PL + j0 + 4]};
        const float* ub = Us + (16 * blk + j0 + t4) * UP + 8 * warp + g;
        const float bv0 = ub[0], bv1 = ub[4 * UP];
        uint32_t ah[4], al[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) { ah[e] = tf32r(av[e]); al[e] = tf32r(av[e] - __uint_as_float(ah[e])); }
        const uint32_t bh0 = tf32r(bv0), bh1 = tf32r(bv1);
        const uint32_t bl0 = tf32r(bv0 - __uint_as_float(bh0)), bl1 = tf32r(bv1 - __uint_as_float(bh1));
        mma_tf32(u, al, bh0, bh1);
        mma_tf32(u, ah, bl0, bl1);
        mma_tf32(u, ah, bh0, bh1);
      }
      __syncwarp();                                        // every lane has read the block's right side
      ur[0] = u[0]; ur[1] = u[1]; ur[8 * UP] = u[2]; ur[8 * UP + 1] = u[3];
      __syncwarp();
    }
    if (stamp) tlc[5] = clock64();
    __syncthreads();                                       // every dv column of U is in place
    if (stamp) tlc[6] = clock64();
    // ---- outputs: O^T[dv][t] = sum_{j <= t} U[j][dv] M[t][j] for token tiles `warp` and 7 - warp ----
#pragma unroll
    for (int side = 0; side < 2; ++side) {
      const int nt = side ? 7 - warp : warp;
      float acc[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[mt][j] = 0.f;
      for (int ks = 0; ks <= nt; ++ks) {
        const int j0 = 8 * ks;
        const float* mb = Mm + (8 * nt + g) * PM + j0 + t4;
        const uint32_t b0 = __float_as_uint(mb[0]), b1 = __float_as_uint(mb[4]);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
          const float* ua = Us + (j0 + t4) * UP + 16 * mt + g;
          uint32_t a[4];
          a[0] = tf32r(ua[0]); a[1] = tf32r(ua[8]); a[2] = tf32r(ua[4 * UP]); a[3] = tf32r(ua[4 * UP + 8]);
          mma_tf32(acc[mt], a, b0, b1);
        }
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int dvr = 16 * mt + g + ((e & 2) ? 8 : 0), t = 8 * nt + 2 * t4 + (e & 1);
          if (t < nc)
            p.o_raw[(size_t)(r0 + c0 + t) * p.ld_o + vh * D + dvs * DVL + dvr] = (__expf(Gs[t]) * Rs[t * UP + dvr] + acc[mt][e]) * inv_sqrt_d;
        }
    }
    if (stamp) tlc[7] = clock64();
    // ---- state: S = gamma_C S + sum_j (gamma_C / gamma_j) u_j k_j^T for this warp's k range ----
    const float gamC = __expf(gC);
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int ntl = 0; ntl < 4; ++ntl)
#pragma unroll
        for (int e = 0; e < 4; ++e) Sr[mt][ntl][e] *= gamC;
#pragma unroll 2
    for (int ks = 0; ks < CH / 8; ++ks) {
      const int j0 = 8 * ks;
      const float e0 = Es[j0 + t4], e1 = Es[j0 + t4 + 4];
      uint32_t a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        const float* ua = Us + (j0 + t4) * UP + 16 * mt + g;
        a[mt][0] = tf32r(e0 * ua[0]); a[mt][1] = tf32r(e0 * ua[8]); a[mt][2] = tf32r(e1 * ua[4 * UP]); a[mt][3] = tf32r(e1 * ua[4 * UP + 8]);
      }
#pragma unroll
      for (int ntl = 0; ntl < 4; ++ntl) {
        const float* kb = Ks + (j0 + t4) * LDK + 8 * (4 * warp + ntl) + g;
        const uint32_t b0 = __float_as_uint(kb[0]), b1 = __float_as_uint(kb[4 * LDK]);
        mma_tf32(Sr[0][ntl], a[0], b0, b1);
        mma_tf32(Sr[1][ntl], a[1], b0, b1);
      }
    }
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int ntl = 0; ntl < 4; ++ntl) {
      const int k = 8 * (4 * warp + ntl) + 2 * t4;
      *reinterpret_cast<float2*>(sbase + (size_t)(16 * mt + g) * D + k) = make_float2(Sr[mt][ntl][0], Sr[mt][ntl][1]);
      *reinterpret_cast<float2*>(sbase + (size_t)(16 * mt + g + 8) * D + k) = make_float2(Sr[mt][ntl][2], Sr[mt][ntl][3]);
    }
}

// out = rms_norm(o_raw) * w * silu(z) per (row, v head)
__global__ void __launch_bounds__(128) gdn_gated_norm_kernel(const float* __restrict__ o_raw, int ld_o, const bf16* __restrict__ z, int ld_z,
                                                             const float* __restrict__ w, float eps, bf16* __restrict__ out, int ld_out) {
  __shared__ float red[4];
  const int row = blockIdx.x, vh = blockIdx.y, tid = threadIdx.x;
  const float o = o_raw[(size_t)row * ld_o + vh * D + tid];
  const float ss = warp_sum(o * o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  const float r = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)D + eps);
  const float zz = __bfloat162float(z[(size_t)row * ld_z + vh * D + tid]);
  out[(size_t)row * ld_out + vh * D + tid] = __float2bfloat16(o * r * w[tid] * silu_f(zz));
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

// Chunked (prompt) form: same contract as grm_gdn_runs plus an fp32 scratch o_raw [M][Hv*Dv]; M = total rows.
static long long* g_gdn_timeline = nullptr;
// Debug aid: while set, CTA (0, 0, 0) of the tensor-core chunk kernel writes 8 clock64 stamps per chunk (chunk start, after
// staging, after the pass over k, after its barrier, after L / M, after the substitution, after its barrier, after the
// outputs); the buffer must hold 8 words per chunk of the first run.  Null switches it off.
GRM_API void grm_gdn_set_timeline(void* buf) { g_gdn_timeline = (long long*)buf; }

GRM_API int grm_gdn_chunked(const void* qkv, int ld_qkv, const void* ab, int ld_ab, const void* z, int ld_z, const void* A_log,
                            const void* dt_bias, const void* norm_w, float norm_eps, void* state, const void* run_slot,
                            const void* run_start, const void* run_len, int n_runs, void* o_raw, void* out, int ld_out, int M,
                            int Hk, int Hv, int Dk, int Dv, void* stream) {
  if (Dk != D || Dv != D || n_runs < 1 || Hv % Hk || M < 1 || (ld_qkv & 3)) return -2;
  GdnChunkParams p;
  p.qkv = (const bf16*)qkv; p.ld_qkv = ld_qkv; p.ab = (const float*)ab; p.ld_ab = ld_ab;
  p.A_log = (const float*)A_log; p.dt_bias = (const float*)dt_bias; p.state = (float*)state;
  p.run_slot = (const int*)run_slot; p.run_start = (const int*)run_start; p.run_len = (const int*)run_len;
  p.o_raw = (float*)o_raw; p.ld_o = Hv * D; p.Hk = Hk; p.Hv = Hv; p.tl = g_gdn_timeline;
  size_t smem = sizeof(float) * (2 * CH * LDK + CH * DVL + 3 * CH * UP + 2 * CH);
  // GRIMOIRE_GDN_SOLO=1 asks for more than half of an SM's shared memory, so that every CTA gets an SM to itself
  // (measurement switch for the two-CTAs-per-SM layout)
  static int solo = -1;
  if (solo < 0) { const char* e = getenv("GRIMOIRE_GDN_SOLO"); solo = (e && e[0] == '1') ? 1 : 0; }
  if (solo) smem = 120 * 1024;
  static bool configured = false;
  cudaStream_t st = (cudaStream_t)stream;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  static int use_mma = -1;
  if (use_mma < 0) {
    const char* ev = getenv("GRIMOIRE_GDN_MMA");
    use_mma = (ev && ev[0] == '0') ? 0 : 1;
    if (use_mma && cudaFuncSetAttribute(gdn_chunked_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 120 * 1024) != cudaSuccess)
      use_mma = 0;
  }
  if (use_mma && !(ld_qkv & 7)) {
    const size_t smem_mma = solo ? smem : sizeof(float) * (CH * LDK + QREG + CH * DVL + 3 * CH * UP + 3 * CH) + sizeof(bf16) * CH * DVL;
    gdn_chunked_mma_kernel<<<dim3(n_runs, Hv, D / DVL), kChThreads, smem_mma, st>>>(p);
  } else {
    gdn_chunked_kernel<<<dim3(n_runs, Hv, D / DVL), kChThreads, smem, st>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  gdn_gated_norm_kernel<<<dim3(M, Hv), 128, 0, st>>>((const float*)o_raw, Hv * D, (const bf16*)z, ld_z, (const float*)norm_w, norm_eps,
                                                     (bf16*)out, ld_out);
  GRM_LAUNCH_RET();
}
