// flash_prefill: causal attention of M query rows of ONE sequence over its T = q_pos0 + M keys
// (chunk-resumed prefill: q_pos0 > 0 means earlier chunks are already in K/V), GQA, optional
// sliding window and sigmoid output gate.  K and V are dense bf16 [T][Hkv][D] (the current chunk's
// roped K / V written by rope_kvwrite, earlier chunks re-materialised by kv_gather_dequant).
//
// Role in the reference: flash_esimd / flash_fast_impl / launch_flash_prefill_fast(+_window)
// (src/gemm_fast.cpp:832-1375) and the SIMT launch_flash_prefill (src/prefill.cpp:1978).
//
// This version is the warp-MMA (m16n8k16 bf16, fp32 softmax) flash kernel: 64 query rows per CTA
// (16 per warp), 64-key blocks double-buffered through cp.async with an XOR swizzle, ldmatrix
// operand loads, online softmax in the exp2 domain.  Attention is ~6 % of the prefill FLOPs of the
// 27B dense model at 4K tokens; the tcgen05/TMEM path is reserved for the GEMMs that carry the
// other 94 % (gemm_tcgen05.cu).
#include "common.cuh"

namespace {

constexpr int BQ = 64, BKV = 64, kWarps = 4, kThreads = 128;

struct PfParams {
  const bf16* q; int ld_q;
  const bf16* k; const bf16* v; int ld_kv;
  const bf16* gate;
  bf16* out; int ld_o;
  int M, T, Hq, Hkv, q_pos0, window;
  float scale_log2;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* g, bool pred) {
  const uint32_t s = smem_u32(smem);
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(g), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

// element (row, col) of a [rows][D] bf16 tile with 16-byte chunks XOR-swizzled by row&7
template <int D>
__device__ __forceinline__ bf16* sw(bf16* base, int row, int col) {
  const int chunk = (col >> 3) ^ (row & 7);
  return base + row * D + (chunk << 3) + (col & 7);
}

template <int D>
__device__ __forceinline__ void load_tile(bf16* dst, const bf16* src, int ld, int row0, int nrows_valid, int tid) {
  constexpr int CH = D / 8;
  for (int i = tid; i < 64 * CH; i += kThreads) {
    const int r = i / CH, c = i % CH;
    const bool ok = (row0 + r) < nrows_valid;
    const bf16* g = src + (size_t)(ok ? row0 + r : 0) * ld + c * 8;
    cp_async16(sw<D>(dst, r, c * 8), g, ok);
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads) flash_prefill_kernel(const PfParams p) {
  extern __shared__ __align__(128) uint8_t smraw[];
  bf16* sQ = reinterpret_cast<bf16*>(smraw);
  bf16* sK = sQ + BQ * D;           // 2 buffers
  bf16* sV = sK + 2 * BKV * D;      // 2 buffers
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  // heavy (late) query blocks first so the tail of the grid is made of short CTAs
  const int mb = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, kvh = h / (p.Hq / p.Hkv);
  const int m0 = mb * BQ;
  const bf16* qg = p.q + (size_t)h * D;
  const bf16* kg = p.k + (size_t)kvh * D;
  const bf16* vg = p.v + (size_t)kvh * D;

  const int q_last = p.q_pos0 + min(p.M, m0 + BQ) - 1;          // last key position needed
  const int q_first = p.q_pos0 + m0;
  const int kv_end = min(p.T, q_last + 1);
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, q_first - p.window + 1) / BKV * BKV;
  const int nblk = (kv_end - kv_begin + BKV - 1) / BKV;

  load_tile<D>(sQ, qg, p.ld_q, m0, p.M, tid);
  load_tile<D>(sK, kg, p.ld_kv, kv_begin, kv_end, tid);
  load_tile<D>(sV, vg, p.ld_kv, kv_begin, kv_end, tid);
  cp_async_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int qrow0 = p.q_pos0 + m0 + warp * 16 + g;   // absolute position of this thread's row g (row g+8 = +8)

  for (int b = 0; b < nblk; ++b) {
    const int buf = b & 1;
    if (b + 1 < nblk) {
      load_tile<D>(sK + (buf ^ 1) * BKV * D, kg, p.ld_kv, kv_begin + (b + 1) * BKV, kv_end, tid);
      load_tile<D>(sV + (buf ^ 1) * BKV * D, vg, p.ld_kv, kv_begin + (b + 1) * BKV, kv_end, tid);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    bf16* cK = sK + buf * BKV * D;
    bf16* cV = sV + buf * BKV * D;

    // ---- S = Q K^T (16 x 64 per warp) ----
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      ldsm_x4(a, sw<D>(sQ, warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), kk * 16 + 8 * (lane >> 4)));
#pragma unroll
      for (int np = 0; np < 4; ++np) {   // pairs of n8 tiles
        uint32_t bq[4];
        ldsm_x4(bq, sw<D>(cK, np * 16 + (lane & 7) + 8 * (lane >> 4), kk * 16 + 8 * ((lane >> 3) & 1)));
        mma_bf16_16816(s[2 * np], a[0], a[1], a[2], a[3], bq[0], bq[1]);
        mma_bf16_16816(s[2 * np + 1], a[0], a[1], a[2], a[3], bq[2], bq[3]);
      }
    }
    // ---- mask + online softmax ----
    const int kv0 = kv_begin + b * BKV;
    const bool need_mask = (kv0 + BKV - 1 > p.q_pos0 + m0 + warp * 16) || (kv0 + BKV > kv_end) || p.window > 0;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float v = s[i][c] * p.scale_log2;
        if (need_mask) {
          const int key = kv0 + i * 8 + 2 * t + (c & 1);
          const int qp = qrow0 + 8 * (c >> 1);
          const bool ok = key <= qp && key < kv_end && (p.window <= 0 || key > qp - p.window);
          v = ok ? v : -INFINITY;
        }
        s[i][c] = v;
        mx[c >> 1] = fmaxf(mx[c >> 1], v);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float mnew = fmaxf(mrow[r], mx[r]);
      alpha[r] = (mrow[r] == -INFINITY) ? 0.f : exp2f(mrow[r] - mnew);
      mrow[r] = mnew;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = c >> 1;
        const float pv = (s[i][c] == -INFINITY) ? 0.f : exp2f(s[i][c] - mrow[r]);
        s[i][c] = pv;
        rs[r] += pv;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) lrow[r] = lrow[r] * alpha[r] + rs[r];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1]; }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < BKV / 16; ++kk) {
      const uint32_t a0 = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
      const uint32_t a1 = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
      const uint32_t a2 = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      const uint32_t a3 = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {   // pairs of d tiles
        uint32_t bv[4];
        ldsm_x4_t(bv, sw<D>(cV, kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), dp * 16 + 8 * (lane >> 4)));
        mma_bf16_16816(o[2 * dp], a0, a1, a2, a3, bv[0], bv[1]);
        mma_bf16_16816(o[2 * dp + 1], a0, a1, a2, a3, bv[2], bv[3]);
      }
    }
    __syncthreads();
  }

  // ---- finalize ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
  }
  const float inv[2] = {lrow[0] > 0.f ? 1.f / lrow[0] : 0.f, lrow[1] > 0.f ? 1.f / lrow[1] : 0.f};
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = m0 + warp * 16 + g + 8 * r;
    if (row >= p.M) continue;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + 2 * t;
      float v0 = o[i][2 * r] * inv[r], v1 = o[i][2 * r + 1] * inv[r];
      const size_t oi = (size_t)row * p.ld_o + (size_t)h * D + col;
      if (p.gate) {
        const uint32_t gv = *reinterpret_cast<const uint32_t*>(p.gate + oi);
        v0 *= sigmoid_f(bf16lo_to_f(gv)); v1 *= sigmoid_f(bf16hi_to_f(gv));
      }
      *reinterpret_cast<uint32_t*>(p.out + oi) = pack_bf16x2(v0, v1);
    }
  }
}

template <int D>
int launch(const PfParams& p, cudaStream_t st) {
  const size_t smem = (size_t)(BQ * D + 4 * BKV * D) * sizeof(bf16);
  auto kfn = flash_prefill_kernel<D>;
  static bool done = false;
  if (!done) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    done = true;
  }
  dim3 grid((p.M + BQ - 1) / BQ, p.Hq);
  kfn<<<grid, kThreads, smem, st>>>(p);
  GRM_LAUNCH_RET();
}

}  // namespace

// q: bf16 [M][ld_q] (head h at column h*D), k/v: bf16 [T][ld_kv], out: bf16 [M][ld_o]; T >= q_pos0 + M.
GRM_API int grm_flash_prefill(const void* q, int ld_q, const void* k, const void* v, int ld_kv, const void* gate, void* out,
                              int ld_o, int M, int T, int Hq, int Hkv, int D, int q_pos0, int window, float scale,
                              void* stream) {
  if (M < 1 || Hq % Hkv || (ld_q & 7) || (ld_kv & 7) || (ld_o & 1) || T < q_pos0 + M) return -2;
  PfParams p;
  p.q = (const bf16*)q; p.ld_q = ld_q; p.k = (const bf16*)k; p.v = (const bf16*)v; p.ld_kv = ld_kv; p.gate = (const bf16*)gate;
  p.out = (bf16*)out; p.ld_o = ld_o; p.M = M; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.q_pos0 = q_pos0; p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t st = (cudaStream_t)stream;
  switch (D) {
    case 64: return launch<64>(p, st);
    case 128: return launch<128>(p, st);
    case 256: return launch<256>(p, st);
    default: return -2;
  }
}
