// Mixture-of-experts kernels: routing (softmax over all experts, top-k, renormalise), the grouped
// expert GEMM over block-scaled fp8 weights (e4m3 payload, one fp32 scale per 1x128 block along K)
// and the top-k weighted combine.
//
// Reference: launch_router_topk* (src/ops.cpp:1022-1490), moe_gate_up_impl_r / moe_down_impl_r and
// the grouped expert GEMMs (src/moe_kernels.cpp:83-1170, src/gemm_fast.cpp:1444-2560), dispatch /
// un-permute helpers (src/prefill.cpp:2644-2905).  One grouped kernel serves decode rows (one tile
// per (row, selected expert)) and prompt chunks (rows sorted by expert, 16-row tiles): every tile
// names its expert and its rows, weights are converted fp8 -> f16 in registers and multiplied with
// warp-level f16 MMAs (fp32 accumulate), the block scale is applied to the fp32 partial sum every
// 128 columns of K, the gate/up projection applies SwiGLU in the epilogue.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------------------------
// routing: one warp per row.  logits fp32 [M][ld] (E experts, optional extra column E = shared gate)
// ---------------------------------------------------------------------------------------------
constexpr int kMaxExpertsPerLane = 16;   // E <= 512

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int ld, int M, int E, int top_k, int renorm,
                                                        int* __restrict__ ids, int ld_ids, float* __restrict__ weights, int ld_w,
                                                        int* __restrict__ counts, int shared_gate) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (row >= M) return;
  const float* lg = logits + (size_t)row * ld;
  float v[kMaxExpertsPerLane];
  float mx = -INFINITY;
  const int per = (E + 31) / 32;
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) {
    const int e = lane + 32 * i;
    v[i] = (i < per && e < E) ? lg[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) { v[i] = (v[i] == -INFINITY) ? 0.f : __expf(v[i] - mx); sum += v[i]; }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float wsum = 0.f, mine_w = 0.f;
  int mine_id = 0;
  for (int k = 0; k < top_k; ++k) {
    float bv = -1.f; int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > bv || (v[i] == bv && e < bi)) { bv = v[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) v[bi >> 5] = -1.f;      // taken (all probabilities are >= 0)
    if (lane == k) { mine_id = bi; mine_w = bv * inv; }
    wsum += bv * inv;
  }
  if (lane < top_k) {
    ids[(size_t)row * ld_ids + lane] = mine_id;
    weights[(size_t)row * ld_w + lane] = renorm ? mine_w / wsum : mine_w;
    if (counts) atomicAdd(&counts[mine_id], 1);
  }
  // shared expert: its weight sigmoid(logits[E]) goes to slot top_k of the row (the caller's rows have top_k + 1 slots)
  if (shared_gate && lane == 0) weights[(size_t)row * ld_w + top_k] = sigmoid_f(lg[E]);
}

// ---------------------------------------------------------------------------------------------
// grouped GEMM: tile = up to 32 rows of one expert x 128 output columns.
// ---------------------------------------------------------------------------------------------
struct GroupedParams {
  const bf16* x; int ldx;           // activations [rows][K]
  const int* row_ids;               // [total_rows] source row of x for each grouped row (null: identity)
  const int* tile_expert;           // [tiles]
  const int* tile_row0;             // [tiles] first grouped row
  const int* tile_rows;             // [tiles] rows in the tile (1..16)
  const uint8_t* w;                 // [E][N][K] e4m3
  const float* scale;               // [E][N][K/128]
  void* out; int ldo;               // mode 0: bf16 [total_rows][N/2] (SwiGLU: rows [0,N/2) gate, [N/2,N) up)
                                    // mode 1: fp32 [total_rows][N]
  int N, K, mode;
  // expert-parallel extensions (null / unused on the single-GPU path)
  const int* n_tiles_dev;           // device-side tile count: CTAs of tiles beyond it exit (grid is an upper bound)
  const int* tile_src;              // [tiles] rank whose tokens the tile's rows belong to            (MODE 4)
  const int* row_dst;               // [total_rows] row of the source rank's return buffer            (MODE 4)
  float* peer_y[8];                 // return buffers of all ranks, fp32 [pairs][ldo]                 (MODE 4)
  unsigned int* peer_done[8];       // arrival counters of all ranks (one count per row and column block)
};

constexpr int kGThreads = 128;      // 4 warps, each 32 output columns (x2 for gate/up)

__device__ __forceinline__ void cvt_e4m3x4_to_f16x2x2(uint32_t v, uint32_t& lo, uint32_t& hi) {
  unsigned short a = (unsigned short)(v & 0xffffu), b = (unsigned short)(v >> 16);
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(lo) : "h"(a));
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(hi) : "h"(b));
}
__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MODE 0: gate|up + SwiGLU (each warp computes 32 gate and the matching 32 up columns); MODE 1: plain.
// MODE 4 (expert parallel combine): the fp32 result rows are stored straight into the return buffer of
// the rank that owns the token (peer stores over NVLink), then the tile raises that rank's arrival
// counter with a system-scope release, so the owner's weighted top-k sum can start as rows land.
constexpr int kTileRows = 32;       // rows of one tile: two m16 tiles share every converted weight fragment
constexpr float kScaleLift = 4096.f; // block scales are lifted by 2^12 before their f16 conversion (small scales would be
                                     // f16 subnormals) and the accumulators are lowered by 2^-12 in the epilogue (exact)

template <int MODE>
__global__ void __launch_bounds__(kGThreads) moe_grouped_kernel(const GroupedParams p) {
  __shared__ __align__(16) __half xs[kTileRows][128 + 8];     // one 128-wide K block of the tile's rows, f16
  const int tile = blockIdx.x, nblk = blockIdx.y;
  if (p.n_tiles_dev && tile >= *p.n_tiles_dev) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int e = p.tile_expert[tile], r0 = p.tile_row0[tile], nr = min(p.tile_rows[tile], kTileRows);
  const int NO = MODE == 0 ? p.N / 2 : p.N;             // output columns
  const int col0 = nblk * 128 + warp * 32;              // this warp's first output column
  const int KB = p.K / 128;
  const uint8_t* we = p.w + (size_t)e * p.N * p.K;
  const float* se = p.scale + (size_t)e * p.N * KB;
  constexpr int NB = MODE == 0 ? 2 : 1;                 // weight row groups per output column (gate, up)
  constexpr int MTL = kTileRows / 16;
  const bool two = nr > 16;                             // second m tile in use
  float acc[MTL][NB][4][4];
#pragma unroll
  for (int m = 0; m < MTL; ++m)
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][b][i][c] = 0.f;

  for (int kb = 0; kb < KB; ++kb) {
    __syncthreads();
    // stage x rows [32][128] as f16 (rows beyond the tile are zero)
    for (int i = tid; i < kTileRows * 16; i += kGThreads) {
      const int r = i >> 4, c8 = i & 15;
      uint4 o = make_uint4(0u, 0u, 0u, 0u);
      if (r < nr) {
        const int src = p.row_ids ? p.row_ids[r0 + r] : (r0 + r);
        const uint4 v = *reinterpret_cast<const uint4*>(p.x + (size_t)src * p.ldx + kb * 128 + c8 * 8);
        const uint32_t in[4] = {v.x, v.y, v.z, v.w};
        uint32_t ou[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const __half2 h2 = __floats2half2_rn(bf16lo_to_f(in[q]), bf16hi_to_f(in[q]));
          ou[q] = *reinterpret_cast<const uint32_t*>(&h2);
        }
        o = make_uint4(ou[0], ou[1], ou[2], ou[3]);
      }
      *reinterpret_cast<uint4*>(&xs[r][c8 * 8]) = o;
    }
    // block scale of this 128-wide K block for the weight row (= B column) this lane converts: n = col0 + 8 i + g.
    // The scale is folded into the f16 weights before the MMA (e4m3 * scale is the weight itself, well inside
    // f16 range), so the products accumulate straight into fp32.
    __half2 sc2[NB][4];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = col0 + i * 8 + g;
        sc2[b][i] = __float2half2_rn(n < NO ? se[(size_t)(n + b * NO) * KB + kb] * kScaleLift : 0.f);
      }
    __syncthreads();
    // two 64-wide halves; lane t owns k columns [16t, 16t+16) of a half (A and B use the same K order)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint4 wv[NB][4];
#pragma unroll
      for (int b = 0; b < NB; ++b)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int n = col0 + i * 8 + g + b * NO;
          wv[b][i] = (col0 + i * 8 + g < NO)
                         ? ldg_stream_v4(we + (size_t)n * p.K + kb * 128 + half * 64 + t * 16) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // A fragment: rows g / g+8, k slots (2t,2t+1) <- columns 16t+4j, +1 ; (2t+8,2t+9) <- 16t+4j+2, +3
        const uint2 xa = *reinterpret_cast<const uint2*>(&xs[g][half * 64 + t * 16 + j * 4]);
        const uint2 xb = *reinterpret_cast<const uint2*>(&xs[g + 8][half * 64 + t * 16 + j * 4]);
        uint2 xc = make_uint2(0u, 0u), xd = xc;
        if (two) {
          xc = *reinterpret_cast<const uint2*>(&xs[g + 16][half * 64 + t * 16 + j * 4]);
          xd = *reinterpret_cast<const uint2*>(&xs[g + 24][half * 64 + t * 16 + j * 4]);
        }
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t wq = j == 0 ? wv[b][i].x : (j == 1 ? wv[b][i].y : (j == 2 ? wv[b][i].z : wv[b][i].w));
            uint32_t b0, b1;
            cvt_e4m3x4_to_f16x2x2(wq, b0, b1);
            const __half2 h0 = __hmul2(*reinterpret_cast<const __half2*>(&b0), sc2[b][i]);
            const __half2 h1 = __hmul2(*reinterpret_cast<const __half2*>(&b1), sc2[b][i]);
            b0 = *reinterpret_cast<const uint32_t*>(&h0); b1 = *reinterpret_cast<const uint32_t*>(&h1);
            mma_f16_16816(acc[0][b][i], xa.x, xb.x, xa.y, xb.y, b0, b1);
            if (two) mma_f16_16816(acc[1][b][i], xc.x, xd.x, xc.y, xd.y, b0, b1);
          }
      }
    }
  }
  constexpr float kInvLift = 1.f / kScaleLift;
  // epilogue: c0,c1 = (row g, cols 2t, 2t+1); c2,c3 = (row g+8, same cols)
#pragma unroll
  for (int m = 0; m < MTL; ++m)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = 16 * m + g + 8 * (c >> 1), n = col0 + i * 8 + 2 * t + (c & 1);
        if (r >= nr || n >= NO) continue;
        if (MODE == 4) {
          p.peer_y[p.tile_src[tile]][(size_t)p.row_dst[r0 + r] * p.ldo + n] = (acc[m][0][i][c] * kInvLift);
          continue;
        }
        const size_t o = (size_t)(r0 + r) * p.ldo + n;
        if (MODE == 0) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(silu_f((acc[m][0][i][c] * kInvLift)) * (acc[m][NB - 1][i][c] * kInvLift));
        else if (MODE == 1) reinterpret_cast<float*>(p.out)[o] = (acc[m][0][i][c] * kInvLift);
        else if (MODE == 2) reinterpret_cast<float*>(p.out)[o] += (acc[m][0][i][c] * kInvLift);
        else reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16((acc[m][0][i][c] * kInvLift));
      }
  if (MODE == 4) {
    __syncthreads();
    if (tid == 0) {
      __threadfence_system();
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.peer_done[p.tile_src[tile]]), "r"((unsigned)nr) : "memory");
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Small-row form of the grouped product (decode: every tile has at most 8 rows): a weight-streaming
// GEMV.  CTA = (tile, block of `opc` output columns); the tile's activation rows are staged once in
// shared memory as f16; each warp owns output columns and streams their weight rows with 16-byte loads
// (four in flight per lane), expands e4m3 pairs with the hardware conversion, accumulates a lane's 16
// products of one 128-block in packed f16 and folds them into fp32 with the block scale, then
// reduces across the warp.  Same tile descriptors, modes and expert-parallel push as the MMA kernel.
// ---------------------------------------------------------------------------------------------
constexpr int kVThreads = 256;
constexpr int kVRows = 8;

template <int MODE>
__global__ void __launch_bounds__(kVThreads) moe_gemv_kernel(const GroupedParams p, int opc) {
  extern __shared__ __align__(16) __half xs16[];        // [kVRows][K]
  const int tile = blockIdx.x;
  if (p.n_tiles_dev && tile >= *p.n_tiles_dev) return;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int e = p.tile_expert[tile], r0 = p.tile_row0[tile], nr = min(p.tile_rows[tile], kVRows);
  if (nr <= 0) return;   // an empty tile (expert-parallel decode: the choice belongs to another rank) streams no weights
  const int NO = MODE == 0 ? p.N / 2 : p.N;
  const int KB = p.K / 128;
  const uint8_t* we = p.w + (size_t)e * p.N * p.K;
  const float* se = p.scale + (size_t)e * p.N * KB;
  for (int i = tid; i < nr * (p.K / 8); i += kVThreads) {
    const int r = i / (p.K / 8), c8 = i - r * (p.K / 8);
    const int src = p.row_ids ? p.row_ids[r0 + r] : (r0 + r);
    const uint4 v = *reinterpret_cast<const uint4*>(p.x + (size_t)src * p.ldx + c8 * 8);
    const uint32_t in[4] = {v.x, v.y, v.z, v.w};
    uint32_t ou[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __half2 h2 = __floats2half2_rn(bf16lo_to_f(in[q]), bf16hi_to_f(in[q]));
      ou[q] = *reinterpret_cast<const uint32_t*>(&h2);
    }
    *reinterpret_cast<uint4*>(xs16 + (size_t)r * p.K + c8 * 8) = make_uint4(ou[0], ou[1], ou[2], ou[3]);
  }
  __syncthreads();
  constexpr int NB = MODE == 0 ? 2 : 1;
  const int n_lo = blockIdx.y * opc, n_hi = min(n_lo + opc, NO);
  for (int n = n_lo + warp; n < n_hi; n += kVThreads / 32) {
    float acc[NB][kVRows];
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
      for (int r = 0; r < kVRows; ++r) acc[b][r] = 0.f;
    // lane l covers bytes [512 i + 16 l, +16) of the row: one 128-block per 8 lanes and iteration
    for (int k0 = lane * 16; k0 < p.K; k0 += 512 * 4) {
      uint4 wv[NB][4];
      float sc[NB][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u * 512;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          if (k < p.K) {
            wv[b][u] = ldg_stream_v4(we + (size_t)(n + b * NO) * p.K + k);
            sc[b][u] = se[(size_t)(n + b * NO) * KB + (k >> 7)];
          } else {
            wv[b][u] = make_uint4(0u, 0u, 0u, 0u); sc[b][u] = 0.f;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int k = k0 + u * 512;
        if (k >= p.K) break;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          uint32_t wh[8];
          cvt_e4m3x4_to_f16x2x2(wv[b][u].x, wh[0], wh[1]); cvt_e4m3x4_to_f16x2x2(wv[b][u].y, wh[2], wh[3]);
          cvt_e4m3x4_to_f16x2x2(wv[b][u].z, wh[4], wh[5]); cvt_e4m3x4_to_f16x2x2(wv[b][u].w, wh[6], wh[7]);
#pragma unroll
          for (int r = 0; r < kVRows; ++r) {
            if (r < nr) {
              const uint4 xa = *reinterpret_cast<const uint4*>(xs16 + (size_t)r * p.K + k);
              const uint4 xb = *reinterpret_cast<const uint4*>(xs16 + (size_t)r * p.K + k + 8);
              const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
              __half2 s2 = __float2half2_rn(0.f);
#pragma unroll
              for (int q = 0; q < 8; ++q)
                s2 = __hfma2(*reinterpret_cast<const __half2*>(&wh[q]), *reinterpret_cast<const __half2*>(&xw[q]), s2);
              const float2 f = __half22float2(s2);
              acc[b][r] = fmaf(sc[b][u], f.x + f.y, acc[b][r]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b)
#pragma unroll
      for (int r = 0; r < kVRows; ++r) acc[b][r] = warp_sum(acc[b][r]);
    if (lane == 0) {
      for (int r = 0; r < nr; ++r) {
        const float v0 = acc[0][r];
        if (MODE == 4) { p.peer_y[p.tile_src[tile]][(size_t)p.row_dst[r0 + r] * p.ldo + n] = v0; continue; }
        const size_t o = (size_t)(r0 + r) * p.ldo + n;
        if (MODE == 0) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(silu_f(v0) * acc[NB - 1][r]);
        else if (MODE == 1) reinterpret_cast<float*>(p.out)[o] = v0;
        else if (MODE == 2) reinterpret_cast<float*>(p.out)[o] += v0;
        else reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(v0);
      }
    }
  }
  if (MODE == 4) {
    __syncthreads();
    if (tid == 0) {
      __threadfence_system();
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.peer_done[p.tile_src[tile]]), "r"((unsigned)nr) : "memory");
    }
  }
}

template <int MODE>
int launch_gemv(const GroupedParams& p, int n_tiles, int opc, cudaStream_t st) {
  const int NO = MODE == 0 ? p.N / 2 : p.N;
  const size_t smem = (size_t)kVRows * p.K * sizeof(__half);
  static size_t attr_max = 48 * 1024;
  if (smem > 160 * 1024) return -2;
  if (smem > attr_max) {
    cudaError_t e = cudaFuncSetAttribute(moe_gemv_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_max = smem;
  }
  dim3 grid(n_tiles, (NO + opc - 1) / opc);
  moe_gemv_kernel<MODE><<<grid, kVThreads, smem, st>>>(p, opc);
  GRM_LAUNCH_RET();
}

// output columns per CTA: enough CTAs (>= ~2 per SM) without dropping below one column per warp
int gemv_opc(int n_tiles, int NO) {
  int opc = 128;
  while (opc > 8 && (long)n_tiles * ((NO + opc - 1) / opc) < 296) opc >>= 1;
  return opc;
}

// h[token] += sum_j w[token][j] * y[pos[token][j]]  (fixed j order -> deterministic)
__global__ void moe_combine_kernel(float* __restrict__ h, int ldh, const float* __restrict__ y, int ldy, const int* __restrict__ pos,
                                   const float* __restrict__ wts, int slots, int H) {
  const int tok = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float acc = 0.f;
#pragma unroll 4
  for (int j = 0; j < slots; ++j) {
    const int ps = pos[(size_t)tok * slots + j];
    if (ps >= 0) acc = fmaf(wts[(size_t)tok * slots + j], y[(size_t)ps * ldy + c], acc);
  }
  h[(size_t)tok * ldh + c] += acc;
}

}  // namespace

GRM_API int grm_moe_route(const void* logits, int ld, int M, int E, int top_k, int renorm, void* ids, int ld_ids, void* weights,
                          int ld_w, void* counts, int shared_gate, void* stream) {
  if (E < 1 || E > 32 * kMaxExpertsPerLane || top_k < 1 || top_k > 32 || top_k > E) return -2;
  const int threads = 128;
  const int blocks = (M * 32 + threads - 1) / threads;
  moe_route_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((const float*)logits, ld, M, E, top_k, renorm, (int*)ids, ld_ids,
                                                                (float*)weights, ld_w, (int*)counts, shared_gate);
  GRM_LAUNCH_RET();
}

// mode 0: out bf16 [total_rows][N/2] = silu(x Wg^T) * (x Wu^T) with W = [gate rows | up rows];
// mode 1: out fp32 [total_rows][N] = x W^T; mode 2: out += ; mode 3: bf16 store.  K % 128 == 0; weights e4m3 with fp32 scales [E][N][K/128].
GRM_API int grm_moe_grouped_gemm(const void* x, int ldx, const void* row_ids, const void* tile_expert, const void* tile_row0,
                                 const void* tile_rows, int n_tiles, const void* w, const void* scale, void* out, int ldo, int N,
                                 int K, int mode, void* stream) {
  if (n_tiles < 1 || (K % 128) || (ldx & 7) || (mode == 0 && (N & 1))) return -2;
  GroupedParams p;
  p.x = (const bf16*)x; p.ldx = ldx; p.row_ids = (const int*)row_ids; p.tile_expert = (const int*)tile_expert;
  p.tile_row0 = (const int*)tile_row0; p.tile_rows = (const int*)tile_rows; p.w = (const uint8_t*)w; p.scale = (const float*)scale;
  p.out = out; p.ldo = ldo; p.N = N; p.K = K; p.mode = mode;
  p.n_tiles_dev = nullptr; p.tile_src = nullptr; p.row_dst = nullptr;
  for (int i = 0; i < 8; ++i) { p.peer_y[i] = nullptr; p.peer_done[i] = nullptr; }
  const int NO = mode == 0 ? N / 2 : N;
  dim3 grid(n_tiles, (NO + 127) / 128);
  cudaStream_t st = (cudaStream_t)stream;
  switch (mode) {
    case 0: moe_grouped_kernel<0><<<grid, kGThreads, 0, st>>>(p); break;
    case 1: moe_grouped_kernel<1><<<grid, kGThreads, 0, st>>>(p); break;
    case 2: moe_grouped_kernel<2><<<grid, kGThreads, 0, st>>>(p); break;
    case 3: moe_grouped_kernel<3><<<grid, kGThreads, 0, st>>>(p); break;
    default: return -1;
  }
  GRM_LAUNCH_RET();
}

// Small-row entry point (every tile has at most 8 rows): the weight-streaming GEMV above.
GRM_API int grm_moe_grouped_gemv(const void* x, int ldx, const void* row_ids, const void* tile_expert, const void* tile_row0,
                                 const void* tile_rows, int n_tiles, const void* w, const void* scale, void* out, int ldo, int N,
                                 int K, int mode, void* stream) {
  if (n_tiles < 1 || (K % 128) || (ldx & 7) || (mode == 0 && (N & 1))) return -2;
  GroupedParams p;
  p.x = (const bf16*)x; p.ldx = ldx; p.row_ids = (const int*)row_ids; p.tile_expert = (const int*)tile_expert;
  p.tile_row0 = (const int*)tile_row0; p.tile_rows = (const int*)tile_rows; p.w = (const uint8_t*)w; p.scale = (const float*)scale;
  p.out = out; p.ldo = ldo; p.N = N; p.K = K; p.mode = mode;
  p.n_tiles_dev = nullptr; p.tile_src = nullptr; p.row_dst = nullptr;
  for (int i = 0; i < 8; ++i) { p.peer_y[i] = nullptr; p.peer_done[i] = nullptr; }
  const int opc = gemv_opc(n_tiles, mode == 0 ? N / 2 : N);
  cudaStream_t st = (cudaStream_t)stream;
  switch (mode) {
    case 0: return launch_gemv<0>(p, n_tiles, opc, st);
    case 1: return launch_gemv<1>(p, n_tiles, opc, st);
    case 2: return launch_gemv<2>(p, n_tiles, opc, st);
    case 3: return launch_gemv<3>(p, n_tiles, opc, st);
    default: return -1;
  }
}

// Expert-parallel form: tile descriptors and the tile count live on the device (built by grm_ep_plan),
// the grid is the upper bound ``max_tiles``.  mode 0: SwiGLU into the local activation buffer;
// mode 4: rows go back to their source rank (see MODE 4 above).
GRM_API int grm_moe_grouped_gemm_ep(const void* x, int ldx, const void* tile_expert, const void* tile_row0, const void* tile_rows,
                                    const void* tile_src, const void* n_tiles_dev, int max_tiles, const void* w, const void* scale,
                                    void* out, int ldo, int N, int K, int mode, const void* row_dst, void* const* peer_y,
                                    void* const* peer_done, int world, int small_rows, void* stream) {
  if (max_tiles < 1 || (K % 128) || (ldx & 7) || (mode == 0 && (N & 1)) || world < 1 || world > 8) return -2;
  GroupedParams p;
  p.x = (const bf16*)x; p.ldx = ldx; p.row_ids = nullptr; p.tile_expert = (const int*)tile_expert;
  p.tile_row0 = (const int*)tile_row0; p.tile_rows = (const int*)tile_rows; p.w = (const uint8_t*)w; p.scale = (const float*)scale;
  p.out = out; p.ldo = ldo; p.N = N; p.K = K; p.mode = mode;
  p.n_tiles_dev = (const int*)n_tiles_dev; p.tile_src = (const int*)tile_src; p.row_dst = (const int*)row_dst;
  for (int i = 0; i < 8; ++i) {
    p.peer_y[i] = (mode == 4 && i < world) ? (float*)peer_y[i] : nullptr;
    p.peer_done[i] = (mode == 4 && i < world) ? (unsigned int*)peer_done[i] : nullptr;
  }
  const int NO = mode == 0 ? N / 2 : N;
  dim3 grid(max_tiles, (NO + 127) / 128);
  cudaStream_t st = (cudaStream_t)stream;
  if (small_rows) {     // every tile has <= 8 rows: GEMV form, 128 columns per CTA so the arrival counts match
    if (mode == 0) return launch_gemv<0>(p, max_tiles, 128, st);
    if (mode == 4) return launch_gemv<4>(p, max_tiles, 128, st);
    return -1;
  }
  if (mode == 0) moe_grouped_kernel<0><<<grid, kGThreads, 0, st>>>(p);
  else if (mode == 4) moe_grouped_kernel<4><<<grid, kGThreads, 0, st>>>(p);
  else return -1;
  GRM_LAUNCH_RET();
}

namespace {
// block-scaled e4m3 [N][K] -> bf16 [N][K]; one thread per 16 values
__global__ void __launch_bounds__(256) dequant_fp8_block_kernel(const uint8_t* __restrict__ w, const float* __restrict__ s, bf16* __restrict__ out,
                                                                long n16, int K) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n16) return;
  const long e0 = i * 16;
  const long row = e0 / K;
  const int k = (int)(e0 - row * K);
  const float sc = s[row * (K / 128) + (k >> 7)];
  const uint4 v = *reinterpret_cast<const uint4*>(w + e0);
  const uint32_t words[4] = {v.x, v.y, v.z, v.w};
  uint32_t r[8];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t lo, hi;
    cvt_e4m3x4_to_f16x2x2(words[q], lo, hi);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo)), b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    r[2 * q] = pack_bf16x2(a.x * sc, a.y * sc);
    r[2 * q + 1] = pack_bf16x2(b.x * sc, b.y * sc);
  }
  uint4* o = reinterpret_cast<uint4*>(out + e0);
  o[0] = make_uint4(r[0], r[1], r[2], r[3]);
  o[1] = make_uint4(r[4], r[5], r[6], r[7]);
}
}  // namespace

// Dequantise a block-scaled fp8 matrix once into bf16 (tall prefill inputs then use the tcgen05 GEMM).
GRM_API int grm_dequant_fp8_block(const void* w, const void* scale, void* out, int N, int K, void* stream) {
  if (K % 128) return -2;
  const long n16 = (long)N * K / 16;
  dequant_fp8_block_kernel<<<(unsigned)((n16 + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint8_t*)w, (const float*)scale, (bf16*)out,
                                                                                            n16, K);
  GRM_LAUNCH_RET();
}

GRM_API int grm_moe_combine(void* h, int ldh, const void* y, int ldy, const void* pos, const void* wts, int M, int slots, int H,
                            void* stream) {
  moe_combine_kernel<<<dim3(M, (H + 255) / 256), 256, 0, (cudaStream_t)stream>>>((float*)h, ldh, (const float*)y, ldy, (const int*)pos, (const float*)wts, slots, H);
  GRM_LAUNCH_RET();
}
