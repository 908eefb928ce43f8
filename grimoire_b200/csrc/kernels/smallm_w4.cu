// smallm_w4: Y[M<=64][N] = X[M][K](bf16) . W[N][K]^T with W = GPTQ-style int4 (group 64/128/256,
// fp16 scale, 4-bit zero), the weight stream read exactly once -- the decode GEMV (M=1), batched
// decode (M = live conversations) and speculative-verify rows (M = users x (1+K)) all run here.
//
// Role in the reference: gemv_impl / gemv_int4sym_* (src/gemv_decode.cpp:77-566) and the w4a16
// small-M DPAS kernel int4_smallm_impl (src/int4_smallm.hpp:45).  This is a different design:
//
//  * the op is HBM-bound (0.5 byte per weight), so the weight is re-tiled at load time into the
//    exact per-lane order of the m16n8k16 A fragment: one 16-byte load per lane brings 4 k16 steps
//    of a 16-row tile, a warp-wide load is 512 contiguous bytes, a 32-row super-tile is 1 KiB;
//  * nibbles are turned into exact bf16 integers with one logic op per pair (0x4300 | nibble is
//    128+q in bf16), the zero point is removed with one bf16x2 subtract (exact), products are
//    accumulated per quantisation group in fp32 on the tensor core and the fp16 scale is applied in
//    fp32 when the group ends -- so the result equals the fp32 dequantised dot product up to fp32
//    summation order, and rows 1..8 of a batch cost the same weight pass as one row;
//  * batch rows sit in the MMA N dimension (8 per tile, MT tiles), weight rows in M;
//  * the 8 warps of a CTA split K; an optional grid-level split-K (for short-N, long-K shapes)
//    goes through a scratch buffer and a per-tile arrival counter, the last CTA summing the slices
//    in slice order so the result does not depend on arrival order.
//
// Tiled layout (built by grimoire_b200/formats/w4_tile_layout.py, checked by tests/test_w4_layout.py):
//   w   : [N/32][K/64][2][32 lanes] uint4.  Lane L (g=L/4, t=L%4), word j (k16 step j), nibble i:
//         row = 16*rowtile + g + 8*(i&1), k = 64*kt + 16*j + 2*t + 8*((i>>1)&1) + (i>>2)
//   sz  : [N/16][K/group][16] uint32: low 16 bits = fp16 scale, high 16 bits = bf16(128 + zero)
#include "common.cuh"

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kRing = 8;                // bulk-copy stages in flight per warp

enum Epi : int { EPI_BF16 = 0, EPI_F32 = 1, EPI_ADD_F32 = 2, EPI_SWIGLU = 3, EPI_AR_ADD = 4 };

struct W4Params {
  const uint4* w;
  const uint32_t* sz;
  const bf16* x;
  void* out;
  float* scratch;           // [ksplit][tiles][R*MT*128] when ksplit > 1
  unsigned int* counters;   // [tiles], zero before first use, left zero on exit
  int M, N, K;
  int ldx, ldo;
  int g64;                  // group size / 64 (1, 2 or 4)
  int ksplit;               // grid-level K slices
  // ---- fused tensor-parallel all-reduce (EPI_AR_ADD): out(fp32) += sum over ranks of the partials ----
  float* ar_recv[8];        // rank p's receive region: [2 parity][world][tiles][NV] floats (peer-mapped)
  unsigned int* ar_flags[8];// rank p's arrival flags:   [tiles][world]
  unsigned int* ar_epochs;  // local, [tiles]: number of fused launches this tile has completed
  unsigned int* status;     // device status block (timeouts)
  int ar_world, ar_rank;
  unsigned int ar_spin;     // poll limit of the arrival wait
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t lop3_or_and(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
  return r;
}
__device__ __forceinline__ uint32_t bf16x2_sub(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

template <int MT, int R, int EPI>
__device__ __forceinline__ void epilogue_store(const W4Params& p, int tile, int v, float val, float val_up) {
  // v indexes (r, mt, c, lane) with lane fastest; R folded out for SWIGLU (val = gate, val_up = up)
  const int lane = v & 31;
  const int c = (v >> 5) & 3;
  const int mt = (v >> 7) % MT;
  const int r = (v >> 7) / MT;
  const int g = lane >> 2, t = lane & 3;
  const int m = mt * 8 + 2 * t + (c & 1);
  if (m >= p.M) return;
  if (EPI == EPI_SWIGLU) {
    const int n = tile * 16 + g + ((c >> 1) << 3);
    float o = silu_f(val) * val_up;
    reinterpret_cast<bf16*>(p.out)[(size_t)m * p.ldo + n] = __float2bfloat16(o);
  } else {
    const int n = (tile * R + r) * 16 + g + ((c >> 1) << 3);
    if (n >= p.N) return;
    const size_t o = (size_t)m * p.ldo + n;
    if (EPI == EPI_BF16) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16(val);
    else if (EPI == EPI_F32) reinterpret_cast<float*>(p.out)[o] = val;
    else reinterpret_cast<float*>(p.out)[o] += val;   // EPI_ADD_F32 and EPI_AR_ADD
  }
}

template <int MT, int R, int EPI>
__global__ void __launch_bounds__(kThreads) smallm_w4_kernel(const W4Params p) {
  // dynamic shared memory: [kWarps][kRing][R*512] weight ring | [kWarps][R*MT*4][32] reduce | barriers
  extern __shared__ __align__(128) uint8_t smem_dyn[];
  constexpr int kStageBytes = R * 512;
  constexpr int NVc = R * MT * 4 * 32;
  uint8_t* ring = smem_dyn + (size_t)(threadIdx.x >> 5) * kRing * kStageBytes;
  float* red = reinterpret_cast<float*>(smem_dyn + (size_t)kWarps * kRing * kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + (size_t)kWarps * NVc) + (threadIdx.x >> 5) * kRing;
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int tile = blockIdx.x;          // super-tile of R row tiles
  const int KT = p.K >> 6;              // k tiles of 64
  const int G = KT / p.g64;             // groups per row
  // K range of this CTA, then of this warp; both aligned to group boundaries
  const int cta_groups = G / p.ksplit;
  const int gbeg_cta = blockIdx.y * cta_groups;
  const int per_warp = (cta_groups + kWarps - 1) / kWarps;
  const int gbeg = gbeg_cta + warp * per_warp;
  const int gend = min(gbeg + per_warp, gbeg_cta + cta_groups);

  float acc[R][MT][4];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][mt][c] = 0.f;

  if (gbeg < gend) {
    const int kt0 = gbeg * p.g64, kt1 = gend * p.g64;
    const int nkt = kt1 - kt0;
    // The weight stream of this warp: k tile kt of its row tile(s) is kStageBytes contiguous bytes.
    // R == 2: super-tile `tile`, both halves (1 KiB).  R == 1: row tile `tile`, one half (512 B).
    const uint4* wsrc = (R == 2) ? p.w + ((size_t)tile * KT) * 64
                                 : p.w + ((size_t)(tile >> 1) * KT) * 64 + (tile & 1) * 32;
    // Per-warp ring fed by bulk async copies (TMA engine, completion on an mbarrier): kRing stages
    // stay in flight per warp regardless of register pressure, which is what saturates HBM.
    if (lane == 0) {
      for (int i = 0; i < kRing; ++i) mbar_init(&bars[i], 1);
      mbar_fence_init();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      const int pre = nkt < kRing ? nkt : kRing;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&bars[i], kStageBytes);
        bulk_load(ring + i * kStageBytes, wsrc + (size_t)(kt0 + i) * 64, kStageBytes, &bars[i]);
      }
    }
    __syncwarp();

    float accg[R][MT][4];
    uint32_t zc[R][2];
    float sc[R][2];
    const uint32_t* xw = reinterpret_cast<const uint32_t*>(p.x);
    const int ldxw = p.ldx >> 1;
    bool alive = true;

    for (int it = 0; it < nkt; ++it) {
      const int kt = kt0 + it;
      const int stg = it % kRing;
      if (alive && !mbar_wait(&bars[stg], (uint32_t)(it / kRing) & 1u, p.status, 0x500u | stg)) alive = false;
      uint4 wuse[R];
#pragma unroll
      for (int r = 0; r < R; ++r)
        wuse[r] = *reinterpret_cast<const uint4*>(ring + stg * kStageBytes + r * 512 + lane * 16);
      __syncwarp();   // every lane has its words in registers: the stage may be refilled
      if (lane == 0 && alive && it + kRing < nkt) {
        mbar_expect_tx(&bars[stg], kStageBytes);
        bulk_load(ring + stg * kStageBytes, wsrc + (size_t)(kt + kRing) * 64, kStageBytes, &bars[stg]);
      }
      if ((kt & (p.g64 - 1)) == 0) {
        const int gi = kt / p.g64;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int nt = tile * R + r;
          const uint32_t* s = p.sz + ((size_t)nt * G + gi) * 16;
          const uint32_t s0 = __ldg(s + g), s1 = __ldg(s + g + 8);
          sc[r][0] = __half2float(__ushort_as_half((unsigned short)(s0 & 0xffffu)));
          sc[r][1] = __half2float(__ushort_as_half((unsigned short)(s1 & 0xffffu)));
          zc[r][0] = (s0 >> 16) | (s0 & 0xffff0000u);
          zc[r][1] = (s1 >> 16) | (s1 & 0xffff0000u);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) accg[r][mt][c] = 0.f;
        }
      }
      // activation fragments for the 4 k16 steps of this k tile
      uint32_t b[4][MT][2];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m = mt * 8 + g;
        const bool ok = m < p.M;
        const uint32_t* xr = xw + (size_t)m * ldxw + (kt << 5) + t;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          b[j][mt][0] = ok ? __ldg(xr + j * 8) : 0u;
          b[j][mt][1] = ok ? __ldg(xr + j * 8 + 4) : 0u;
        }
      }
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t wj[4] = {wuse[r].x, wuse[r].y, wuse[r].z, wuse[r].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t u = wj[j];
          uint32_t a0 = lop3_or_and(u, 0x000f000fu, 0x43004300u);
          uint32_t a1 = lop3_or_and(u >> 4, 0x000f000fu, 0x43004300u);
          uint32_t a2 = lop3_or_and(u >> 8, 0x000f000fu, 0x43004300u);
          uint32_t a3 = lop3_or_and(u >> 12, 0x000f000fu, 0x43004300u);
          a0 = bf16x2_sub(a0, zc[r][0]);
          a1 = bf16x2_sub(a1, zc[r][1]);
          a2 = bf16x2_sub(a2, zc[r][0]);
          a3 = bf16x2_sub(a3, zc[r][1]);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(accg[r][mt], a0, a1, a2, a3, b[j][mt][0], b[j][mt][1]);
        }
      }
      if (((kt + 1) & (p.g64 - 1)) == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            acc[r][mt][0] = fmaf(sc[r][0], accg[r][mt][0], acc[r][mt][0]);
            acc[r][mt][1] = fmaf(sc[r][0], accg[r][mt][1], acc[r][mt][1]);
            acc[r][mt][2] = fmaf(sc[r][1], accg[r][mt][2], acc[r][mt][2]);
            acc[r][mt][3] = fmaf(sc[r][1], accg[r][mt][3], acc[r][mt][3]);
          }
      }
    }
  }

  // ---- reduce the K slices of the 8 warps (fixed order) -----------------------------------------
  constexpr int NV = R * MT * 4 * 32;  // values per tile
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) red[warp * NV + ((r * MT + mt) * 4 + c) * 32 + lane] = acc[r][mt][c];
  __syncthreads();

  if (EPI == EPI_AR_ADD) {
    // One-shot all-reduce fused into the epilogue: push this rank's partial tile into every rank's
    // receive region over NVLink, raise a per-(tile, source) flag with release semantics, wait
    // (bounded) for the flags of all sources, then sum the W partials in rank order -- every rank
    // adds the same numbers in the same order, so all ranks hold bit-identical results (the
    // property the reference keeps with its rank-ordered shared-memory sums, grimoire.cpp:6263-6366).
    // Receive regions are double-buffered by launch parity: a peer can be at most one fused launch
    // ahead, because its next launch needs this rank's next push.
    __shared__ int s_fail;
    const int W = p.ar_world;
    const unsigned int e = p.ar_epochs[tile] + 1u;
    const size_t tiles = gridDim.x;
    const size_t par = e & 1u;
    if (tid == 0) s_fail = 0;
    for (int v = tid; v < NV; v += kThreads) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += red[w * NV + v];
      const size_t off = ((par * W + p.ar_rank) * tiles + tile) * NV + v;
      for (int r = 0; r < W; ++r) p.ar_recv[r][off] = s;
    }
    __threadfence_system();
    __syncthreads();
    if (tid < W) st_release_sys(p.ar_flags[tid] + (size_t)tile * W + p.ar_rank, e);
    if (tid < W) {
      const unsigned int* f = p.ar_flags[p.ar_rank] + (size_t)tile * W + tid;
      bool ok = false;
      for (unsigned int i = 0; i < p.ar_spin; ++i) {
        if ((int)(ld_acquire_sys(f) - e) >= 0) { ok = true; break; }
        if (i > 16) __nanosleep(20);
      }
      if (!ok) { s_fail = 1; grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x10000u | (tid << 12) | (tile & 0xfff)); }
    }
    __syncthreads();
    if (!s_fail) {
      const float* mine = p.ar_recv[p.ar_rank];
      for (int v = tid; v < NV; v += kThreads) {
        float s = 0.f;
        for (int r = 0; r < W; ++r) s += __ldcg(mine + ((par * W + r) * tiles + tile) * NV + v);
        epilogue_store<MT, R, EPI>(p, tile, v, s, 0.f);
      }
    }
    if (tid == 0) p.ar_epochs[tile] = e;   // advance even after a timeout so later launches stay aligned
    return;
  }

  if (p.ksplit == 1) {
    if (EPI == EPI_SWIGLU) {
      constexpr int NH = NV / 2;  // r = 0 half holds the gate rows, r = 1 the up rows
      for (int v = tid; v < NH; v += kThreads) {
        float sg = 0.f, su = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) { sg += red[w * NV + v]; su += red[w * NV + NH + v]; }
        epilogue_store<MT, R, EPI>(p, tile, v, sg, su);
      }
    } else {
      for (int v = tid; v < NV; v += kThreads) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) s += red[w * NV + v];
        epilogue_store<MT, R, EPI>(p, tile, v, s, 0.f);
      }
    }
    return;
  }

  // ---- grid-level split-K: publish this slice, last CTA of the tile sums slices in order --------
  float* mine = p.scratch + ((size_t)blockIdx.y * gridDim.x + tile) * NV;
  for (int v = tid; v < NV; v += kThreads) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += red[w * NV + v];
    mine[v] = s;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int prev = atomicAdd(&p.counters[tile], 1u);
    s_last = (prev == (unsigned int)p.ksplit - 1u);
    if (s_last) p.counters[tile] = 0u;   // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (EPI == EPI_SWIGLU) {
    constexpr int NH = NV / 2;
    for (int v = tid; v < NH; v += kThreads) {
      float sg = 0.f, su = 0.f;
      for (int k = 0; k < p.ksplit; ++k) {
        const float* sl = p.scratch + ((size_t)k * gridDim.x + tile) * NV;
        sg += __ldcg(sl + v); su += __ldcg(sl + NH + v);
      }
      epilogue_store<MT, R, EPI>(p, tile, v, sg, su);
    }
  } else {
    for (int v = tid; v < NV; v += kThreads) {
      float s = 0.f;
      for (int k = 0; k < p.ksplit; ++k) s += __ldcg(p.scratch + ((size_t)k * gridDim.x + tile) * NV + v);
      epilogue_store<MT, R, EPI>(p, tile, v, s, 0.f);
    }
  }
}

template <int MT, int R, int EPI>
int launch(const W4Params& p, cudaStream_t st) {
  constexpr int NV = R * MT * 4 * 32;
  const size_t smem = (size_t)kWarps * kRing * R * 512 + (size_t)kWarps * NV * sizeof(float) + (size_t)kWarps * kRing * 8;
  auto kfn = smallm_w4_kernel<MT, R, EPI>;
  static bool attr_done = false;
  if (!attr_done && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  dim3 grid(p.N / (16 * R), p.ksplit);
  if (EPI == EPI_AR_ADD) {
    // CTAs of different ranks wait for one another's pushes: every CTA of this grid must be
    // resident at once, otherwise resident CTAs could wait for peers whose partner CTA has no SM.
    int per_sm = 0, dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kfn, kThreads, smem) != cudaSuccess) return -2;
    if ((long)per_sm * sms < (long)grid.x * grid.y) return -2;
  }
  kfn<<<grid, kThreads, smem, st>>>(p);
  GRM_LAUNCH_RET();
}

template <int MT, int R>
int launch_epi(const W4Params& p, int epi, cudaStream_t st) {
  switch (epi) {
    case EPI_BF16: return launch<MT, R, EPI_BF16>(p, st);
    case EPI_F32: return launch<MT, R, EPI_F32>(p, st);
    case EPI_ADD_F32: return launch<MT, R, EPI_ADD_F32>(p, st);
    case EPI_AR_ADD: return launch<MT, R, EPI_AR_ADD>(p, st);
    default: return -1;
  }
}

}  // namespace

namespace {
int dispatch(W4Params& p, int epi, int rows_per_cta, cudaStream_t st) {
  const int MT = (p.M + 7) / 8;
  if (epi == EPI_SWIGLU) {
    if (MT <= 1) return launch<1, 2, EPI_SWIGLU>(p, st);
    if (MT <= 2) return launch<2, 2, EPI_SWIGLU>(p, st);
    if (MT <= 4) return launch<4, 2, EPI_SWIGLU>(p, st);
    return launch<8, 2, EPI_SWIGLU>(p, st);
  }
  const bool r2 = rows_per_cta == 32;
  if (MT <= 1) return r2 ? launch_epi<1, 2>(p, epi, st) : launch_epi<1, 1>(p, epi, st);
  if (MT <= 2) return r2 ? launch_epi<2, 2>(p, epi, st) : launch_epi<2, 1>(p, epi, st);
  if (MT <= 4) return launch_epi<4, 1>(p, epi, st);
  return launch_epi<8, 1>(p, epi, st);
}
}  // namespace

// out: EPI 0 bf16 [M][ldo], 1 fp32 [M][ldo], 2 fp32 accumulate (out += y), 3 SwiGLU bf16 [M][ldo]
// (weight rows interleaved per 16: tile 2s = gate rows 16s.., tile 2s+1 = up rows 16s..; N = 2*I).
// rows_per_cta: 16 or 32 (R = 1 or 2); ksplit >= 1 needs scratch of ksplit*(N/(16R))*R*MT*128 floats
// and N/(16R) zeroed counters.  Returns -2 on an unsupported shape.
GRM_API int grm_smallm_w4(const void* w, const void* sz, const void* x, void* out, void* scratch, void* counters,
                          int M, int N, int K, int ldx, int ldo, int group, int epi, int rows_per_cta, int ksplit,
                          void* stream) {
  if (M < 1 || M > 64 || (N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || (ldx & 1)) return -2;
  const int G = K / group;
  if (ksplit < 1 || (G % ksplit)) return -2;
  if (ksplit > 1 && (!scratch || !counters)) return -2;
  W4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = (const bf16*)x; p.out = out;
  p.scratch = (float*)scratch; p.counters = (unsigned int*)counters;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldo = ldo; p.g64 = group / 64; p.ksplit = ksplit;
  p.status = grm_status_ptr(); p.ar_world = 1; p.ar_rank = 0; p.ar_epochs = nullptr; p.ar_spin = 0;
  for (int i = 0; i < 8; ++i) { p.ar_recv[i] = nullptr; p.ar_flags[i] = nullptr; }
  if (epi == EPI_AR_ADD) return -1;   // use grm_smallm_w4_allreduce
  return dispatch(p, epi, rows_per_cta, (cudaStream_t)stream);
}

// Row-parallel projection fused with the tensor-parallel all-reduce: h[M][ldo] (fp32) += sum over
// ranks of X_r . W_r^T.  recv / flags are arrays of `world` peer-mapped device pointers (see the
// W4Params comment for their layouts; recv needs 2*world*(N/16)*MT*128 floats per rank, flags
// (N/16)*world uints, epochs N/16 uints, all zero before first use).  Every rank must issue the same
// sequence of calls with the same M.  spin = poll limit of the arrival wait (0 = default ~0.1 s).
GRM_API int grm_smallm_w4_allreduce(const void* w, const void* sz, const void* x, void* h, int M, int N, int K, int ldx,
                                    int ldo, int group, const void* const* recv, const void* const* flags, void* epochs,
                                    int world, int rank, unsigned int spin, void* stream) {
  if (M < 1 || M > 64 || (N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || (ldx & 1)) return -2;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !recv || !flags || !epochs) return -2;
  W4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = (const bf16*)x; p.out = h;
  p.scratch = nullptr; p.counters = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldo = ldo; p.g64 = group / 64; p.ksplit = 1;
  for (int i = 0; i < 8; ++i) {
    p.ar_recv[i] = i < world ? (float*)const_cast<void*>(recv[i]) : nullptr;
    p.ar_flags[i] = i < world ? (unsigned int*)const_cast<void*>(flags[i]) : nullptr;
  }
  p.ar_epochs = (unsigned int*)epochs; p.status = grm_status_ptr(); p.ar_world = world; p.ar_rank = rank;
  p.ar_spin = spin ? spin : 2000000u;
  return dispatch(p, EPI_AR_ADD, 16, (cudaStream_t)stream);
}
