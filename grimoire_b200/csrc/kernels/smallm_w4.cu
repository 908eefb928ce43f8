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
//         row = 16*rowtile + g + 8*(i&1), k = 64*kt + 16*t + 4*j + 2*((i>>1)&1) + (i>>2)
//         (a lane's 16 columns of a k tile are contiguous, so its activation fragment is two 16-byte reads)
//   sz  : [N/16][K/group][16] uint32: low 16 bits = fp16 scale, high 16 bits = bf16(128 + zero)
#include "common.cuh"
#include <type_traits>
#include <cstdlib>

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

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
  int szg;                  // groups per warp (capacity of the per-warp scale staging area)
  int stage;                // bytes of one ring stage: R*512 + M*144
  // ---- fused tensor-parallel all-reduce (EPI_AR_ADD): out(fp32) += sum over ranks of the partials ----
  float* ar_recv[8];        // rank p's receive region: [2 parity halves of ar_half floats][world][tiles][NV] {value, epoch} pairs (peer-mapped)
  unsigned int* ar_flags[8];// rank p's arrival flags:   [tiles][world]
  unsigned int* ar_epochs;  // local, [tiles]: number of fused launches this tile has completed
  unsigned int* status;     // device status block (timeouts)
  int ar_world, ar_rank;
  unsigned int ar_spin;     // poll limit of the arrival wait
  size_t ar_half;           // floats between the two parity halves of a receive region: fixed for the buffer, so that launches
                            // with different row counts (different values per tile) never share bytes across parities
  // ---- integer activation path (I8 kernels): x carried as two int8 levels per quantisation group ----
  const int8_t* xq_hi;      // [M][ldq] high level  (x ~ delta * (128*hi + lo)), columns permuted (0,2,1,3) within 4
  const int8_t* xq_lo;      // [M][ldq] low level
  const float2* xtab;       // [M][ldtab] per (row, group): {delta, delta * sum_k(128*hi + lo)}
  int ldq, ldtab;
  // ---- warp layout inside a CTA: rt row super-tiles x ks K slices, rt * ks == kWarps ----
  int rt, ks, ntiles;
  int mx;                   // MATH == 2: weights are MXFP4 tiles (see tile_mx), sz holds e8m0 bytes, x is f16 in lane order
  int szw;                  // 32-bit words of scale data per (16-row tile, group): 16 for int4, 8 for MXFP4 (group = one k tile)
  int min_ctas;             // smallest grid the row-tile grouping may produce (GRIMOIRE_SMALLM_MIN_CTAS, default 222 = 1.5 per SM)
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
__device__ __forceinline__ void mma_s8_16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t cvt_e2m1x2_f16(uint32_t byte) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b0;\n\t}" : "=r"(r) : "r"(byte));
  return r;
}
__device__ __forceinline__ void mma_f16_16816_w4(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
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

// Ring depth (stages of R*512 weight bytes in flight per warp) by batch width.
// A ring stage holds kSK consecutive k tiles (one bulk copy of kSK KiB when R == 2: requests of a few KiB
// keep the copy engine's request rate off the critical path); two stages per warp are in flight.
template <int MT> struct RingDepth { static constexpr int v = 2; };
constexpr int kSK = 4;

// slow path of the stage wait, kept out of line so the hot loop carries only one try_wait
__device__ __noinline__ bool stage_wait_slow(uint64_t* bar, uint32_t parity, unsigned int* status, uint32_t tag) {
  return mbar_wait(bar, parity, status, tag);
}

// One ring stage <- k tiles [kt, min(kt + kSK, kt1)) of the warp's weight stream (issued by one lane).
template <int R>
__device__ __forceinline__ void fill_stage(uint8_t* dst, const uint8_t* wsrc, int kt, int kt1, uint64_t* bar) {
  const int n = min(kSK, kt1 - kt);
  if (n <= 0) return;
  mbar_expect_tx(bar, (uint32_t)n * R * 512u);
  if (R == 2) {
    bulk_load(dst, wsrc + (size_t)kt * 1024, (uint32_t)n * 1024u, bar);
  } else {
    for (int i = 0; i < n; ++i) bulk_load(dst + i * 512, wsrc + (size_t)(kt + i) * 1024, 512u, bar);
  }
}

// I8 = true: the products run on the int8 tensor-core path.  The activations arrive quantised per weight
// group to 15 bits as two int8 levels (grm_quant_x_i8), a weight word splits into the int8 A fragments of
// rows g and g+8 with three logic ops (even nibbles / odd nibbles), group sums are exact int32 and the
// zero point is removed with the group's pre-computed activation sum -- about a third of the ALU work
// of the bf16 path, with a smaller activation rounding error than bf16 inputs have.
template <int MT, int R, int EPI, int MATH>
__global__ void __launch_bounds__(kThreads) smallm_w4_kernel(const W4Params p) {
  constexpr bool I8 = MATH == 1;
  constexpr bool MX = MATH == 2;
  // dynamic shared memory: [kWarps][RING][R*512] weight ring | [kWarps][R*MT*4][32] reduce | barriers | scales
  extern __shared__ __align__(128) uint8_t smem_dyn[];
  constexpr int RING = RingDepth<MT>::v;
  constexpr int kStage = kSK * R * 512;
  constexpr int NVc = R * MT * 4 * 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* ring = smem_dyn + warp * (RING * kStage);
  float* red = reinterpret_cast<float*>(smem_dyn + kWarps * RING * kStage);
  uint64_t* bars = reinterpret_cast<uint64_t*>(red + kWarps * NVc) + warp * (RING + 1);
  // scale / zero words of this warp's groups: [R][p.szg][16] uint32, staged once by a bulk copy
  uint32_t* szs = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(red + kWarps * NVc) + kWarps * (RING + 1) * 8) +
                  (size_t)warp * R * p.szg * p.szw;
  __shared__ int s_last;
  const int g = lane >> 2, t = lane & 3;
  // The CTA's 8 warps cover rt row super-tiles (of R row tiles each) x ks K slices.  Few, long-lived
  // CTAs with long per-warp weight streams keep HBM busy: the fixed start-up (scale staging, first
  // ring fill) and the reduction tail are paid once per 8 * (K / ks) tiles of work instead of once per
  // (K / 8) tiles.
  const int wr = warp / p.ks, wk = warp - wr * p.ks;
  const int tile = blockIdx.x * p.rt + wr;   // super-tile of R row tiles owned by this warp
  const bool live = tile < p.ntiles;
  const int KT = p.K >> 6;              // k tiles of 64
  const int G = KT / p.g64;             // groups per row
  // K range of this CTA, then of this warp; both aligned to group boundaries
  const int cta_groups = G / p.ksplit;
  const int gbeg_cta = blockIdx.y * cta_groups;
  const int per_warp = (cta_groups + p.ks - 1) / p.ks;
  const int gbeg = gbeg_cta + wk * per_warp;
  const int gend = min(gbeg + per_warp, gbeg_cta + cta_groups);

  float acc[R][MT][4];
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][mt][c] = 0.f;

  if (live && gbeg < gend) {
    const int kt0 = gbeg * p.g64, kt1 = gend * p.g64;
    // The weight stream of this warp: k tile kt of its row tile(s) is R*512 contiguous bytes, and
    // consecutive k tiles are 1 KiB apart.  R == 2: both halves of super-tile `tile`; R == 1: one half.
    const uint8_t* wsrc = reinterpret_cast<const uint8_t*>(
        (R == 2) ? p.w + ((size_t)tile * KT) * 64 : p.w + ((size_t)(tile >> 1) * KT) * 64 + (tile & 1) * 32);
    // Per-warp ring fed by bulk async copies (TMA engine, completion on an mbarrier): RING stages of
    // weights stay in flight per warp regardless of register pressure.
    if (lane == 0) {
      for (int i = 0; i <= RING; ++i) mbar_init(&bars[i], 1);
      mbar_fence_init();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      // scales first: a load at the point of use would expose a DRAM latency per group
      const uint32_t szbytes = (uint32_t)(gend - gbeg) * 4u * (uint32_t)p.szw;
      mbar_expect_tx(&bars[RING], szbytes * R);
#pragma unroll
      for (int r = 0; r < R; ++r)
        bulk_load(szs + (size_t)r * p.szg * p.szw, p.sz + ((size_t)(tile * R + r) * G + gbeg) * p.szw, szbytes, &bars[RING]);
      for (int i = 0; i < RING; ++i) fill_stage<R>(ring + i * kStage, wsrc, kt0 + i * kSK, kt1, &bars[i]);
    }
    __syncwarp();

    if constexpr (I8) {
      // int8 activation fragments: lane (g, t) reads the 16 bytes [64 kt + 16 t, +16) of row 8*mt+g per level
      const uint4* xh[MT];
      const uint4* xl[MT];
      bool xok[MT];
      uint4 xhv[MT], xlv[MT];
      const float2* tab0[MT];
      const float2* tab1[MT];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int m = mt * 8 + g;
        xok[mt] = m < p.M;
        const size_t ro = (size_t)(xok[mt] ? m : 0) * p.ldq + (size_t)kt0 * 64 + t * 16;
        xh[mt] = reinterpret_cast<const uint4*>(p.xq_hi + ro);
        xl[mt] = reinterpret_cast<const uint4*>(p.xq_lo + ro);
        xhv[mt] = xlv[mt] = make_uint4(0u, 0u, 0u, 0u);
        if (xok[mt]) { xhv[mt] = __ldg(xh[mt]); xlv[mt] = __ldg(xl[mt]); }
        tab0[mt] = p.xtab + (size_t)min(mt * 8 + 2 * t, p.M - 1) * p.ldtab;
        tab1[mt] = p.xtab + (size_t)min(mt * 8 + 2 * t + 1, p.M - 1) * p.ldtab;
      }
      // Main loop, one ring stage (kSK k tiles) per iteration, fully unrolled inside: constant shared-memory
      // offsets, no per-tile loop control, one barrier wait and one refill per stage.
      static_assert(RING == 2, "the stage toggle below assumes two ring stages");
      auto run = [&](auto g64c) {
        constexpr int G64 = decltype(g64c)::value;       // k tiles per quantisation group (1, 2 or 4)
        constexpr int GPS = kSK / G64;                   // groups per full stage
        uint32_t stg = 0, phase = 0;
        bool dead = !mbar_wait(&bars[RING], 0u, p.status, 0x5ffu);
        const uint32_t* szp = szs + g;
        int grp = gbeg;
#pragma unroll 1
        for (int kt = kt0; kt < kt1 && !dead; kt += kSK, grp += GPS, szp += 16 * GPS) {
          const int nt = min(kSK, kt1 - kt);
          if (!mbar_try_wait(&bars[stg], phase)) {
            if (!stage_wait_slow(&bars[stg], phase, p.status, 0x500u | stg)) { dead = true; break; }
          }
          const uint8_t* sbase = ring + stg * kStage + lane * 16;
          float2 ta[GPS][MT], tb[GPS][MT];
#pragma unroll
          for (int gi = 0; gi < GPS; ++gi)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              const int gq = min(grp + gi, gend - 1);
              ta[gi][mt] = __ldg(tab0[mt] + gq); tb[gi][mt] = __ldg(tab1[mt] + gq);
            }
          int sh[R][MT][4], sl[R][MT][4];
#pragma unroll
          for (int s = 0; s < kSK; ++s) {
            if (s < nt) {
              if (s % G64 == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) { sh[r][mt][c] = 0; sl[r][mt][c] = 0; }
              }
              uint4 wuse[R];
#pragma unroll
              for (int r = 0; r < R; ++r) wuse[r] = *reinterpret_cast<const uint4*>(sbase + s * (R * 512) + r * 512);
              uint32_t bh[MT][4], bl[MT][4];
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) {
                bh[mt][0] = xhv[mt].x; bh[mt][1] = xhv[mt].y; bh[mt][2] = xhv[mt].z; bh[mt][3] = xhv[mt].w;
                bl[mt][0] = xlv[mt].x; bl[mt][1] = xlv[mt].y; bl[mt][2] = xlv[mt].z; bl[mt][3] = xlv[mt].w;
              }
              if (s == nt - 1) {
                __syncwarp();   // every lane has read the stage: it may be refilled
                if (lane == 0) fill_stage<R>(ring + stg * kStage, wsrc, kt + RING * kSK, kt1, &bars[stg]);
              }
              if (kt + s + 1 < kt1) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                  if (xok[mt]) { xhv[mt] = __ldg(xh[mt] + 4 * (s + 1)); xlv[mt] = __ldg(xl[mt] + 4 * (s + 1)); }
              }
#pragma unroll
              for (int s2 = 0; s2 < 2; ++s2) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                  const uint32_t u0 = s2 == 0 ? wuse[r].x : wuse[r].z, u1 = s2 == 0 ? wuse[r].y : wuse[r].w;
                  const uint32_t a0 = u0 & 0x0f0f0f0fu, a1 = (u0 >> 4) & 0x0f0f0f0fu;
                  const uint32_t a2 = u1 & 0x0f0f0f0fu, a3 = (u1 >> 4) & 0x0f0f0f0fu;
#pragma unroll
                  for (int mt = 0; mt < MT; ++mt) {
                    mma_s8_16832(sh[r][mt], a0, a1, a2, a3, bh[mt][2 * s2], bh[mt][2 * s2 + 1]);
                    mma_s8_16832(sl[r][mt], a0, a1, a2, a3, bl[mt][2 * s2], bl[mt][2 * s2 + 1]);
                  }
                }
              }
              if ((s + 1) % G64 == 0) {
                // group flush: sum_k (q - z) x = delta * S - z * (delta * X), then the fp16 weight scale
                const int gi = s / G64;
#pragma unroll
                for (int r = 0; r < R; ++r) {
                  const uint32_t s0 = szp[gi * 16 + r * p.szg * 16], s1 = szp[gi * 16 + r * p.szg * 16 + 8];
                  const float sc0 = __half2float(__ushort_as_half((unsigned short)(s0 & 0xffffu)));
                  const float sc1 = __half2float(__ushort_as_half((unsigned short)(s1 & 0xffffu)));
                  const float z0 = bf16hi_to_f(s0) - 128.f, z1 = bf16hi_to_f(s1) - 128.f;
#pragma unroll
                  for (int mt = 0; mt < MT; ++mt) {
                    const float v0 = (float)(128 * sh[r][mt][0] + sl[r][mt][0]), v1 = (float)(128 * sh[r][mt][1] + sl[r][mt][1]);
                    const float v2 = (float)(128 * sh[r][mt][2] + sl[r][mt][2]), v3 = (float)(128 * sh[r][mt][3] + sl[r][mt][3]);
                    acc[r][mt][0] = fmaf(sc0, fmaf(v0, ta[gi][mt].x, -z0 * ta[gi][mt].y), acc[r][mt][0]);
                    acc[r][mt][1] = fmaf(sc0, fmaf(v1, tb[gi][mt].x, -z0 * tb[gi][mt].y), acc[r][mt][1]);
                    acc[r][mt][2] = fmaf(sc1, fmaf(v2, ta[gi][mt].x, -z1 * ta[gi][mt].y), acc[r][mt][2]);
                    acc[r][mt][3] = fmaf(sc1, fmaf(v3, tb[gi][mt].x, -z1 * tb[gi][mt].y), acc[r][mt][3]);
                  }
                }
              }
            }
          }
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            xh[mt] += 4 * kSK; xl[mt] += 4 * kSK;
            if (xok[mt] && t == 0 && kt + 3 * kSK < kt1) {
              asm volatile("prefetch.global.L1 [%0];" ::"l"(xh[mt] + 4 * kSK)); asm volatile("prefetch.global.L1 [%0];" ::"l"(xh[mt] + 4 * kSK + 8));
              asm volatile("prefetch.global.L1 [%0];" ::"l"(xl[mt] + 4 * kSK)); asm volatile("prefetch.global.L1 [%0];" ::"l"(xl[mt] + 4 * kSK + 8));
            }
          }
          stg ^= 1u;
          phase ^= (stg == 0u);
        }
      };
      if (p.g64 == 1) run(std::integral_constant<int, 1>{});
      else if (p.g64 == 2) run(std::integral_constant<int, 2>{});
      else run(std::integral_constant<int, 4>{});
    } else {
    // Activation fragments: lane (g, t) owns columns 16t..16t+15 of batch row 8*mt+g in every k tile
    // (the weight tiles use the same K order), i.e. two 16-byte loads per k tile, fetched one k tile
    // ahead into registers; the L1 line of a later k tile is requested with a prefetch.
    const uint4* xp[MT];
    bool xok[MT];
    uint4 xa[MT], xb[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int m = mt * 8 + g;
      xok[mt] = m < p.M;
      xp[mt] = reinterpret_cast<const uint4*>(p.x + (size_t)(xok[mt] ? m : 0) * p.ldx + (size_t)kt0 * 64 + t * 16);
      xa[mt] = xb[mt] = make_uint4(0u, 0u, 0u, 0u);
      if (xok[mt]) { xa[mt] = __ldg(xp[mt]); xb[mt] = __ldg(xp[mt] + 1); }
    }
    // Main loop, one ring stage (kSK k tiles) per iteration, fully unrolled inside (constant shared-memory offsets, one
    // barrier wait and one refill per stage, the instruction streams of neighbouring k tiles interleave).
    static_assert(RING == 2, "the stage toggle below assumes two ring stages");
    auto run16 = [&](auto g64c) {
      constexpr int G64 = decltype(g64c)::value;       // k tiles per quantisation group (MXFP4: 1, two blocks per k tile)
      constexpr int GPS = kSK / G64;                   // groups per full stage
      uint32_t stg = 0, phase = 0;
      bool dead = !mbar_wait(&bars[RING], 0u, p.status, 0x5ffu);
      const uint32_t* szp = szs + g;
      const uint32_t ones = 0x3f803f80u;   // bf16 {1, 1}
#pragma unroll 1
      for (int kt = kt0; kt < kt1 && !dead; kt += kSK, szp += GPS * p.szw) {
        const int nt = min(kSK, kt1 - kt);
        if (!mbar_try_wait(&bars[stg], phase)) {
          if (!stage_wait_slow(&bars[stg], phase, p.status, 0x500u | stg)) { dead = true; break; }
        }
        const uint8_t* sbase = ring + stg * kStage + lane * 16;
        float accg[R][MT][4], xsum[MT][4];
        float accg2[MX ? R : 1][MX ? MT : 1][4];      // MXFP4: the k tile's second 32-wide block
#pragma unroll
        for (int s = 0; s < kSK; ++s) {
          if (s < nt) {
            if (s % G64 == 0) {
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  xsum[mt][c] = 0.f;
#pragma unroll
                  for (int r = 0; r < R; ++r) {
                    accg[r][mt][c] = 0.f;
                    if constexpr (MX) accg2[r][mt][c] = 0.f;
                  }
                }
            }
            uint4 wuse[R];
#pragma unroll
            for (int r = 0; r < R; ++r) wuse[r] = *reinterpret_cast<const uint4*>(sbase + s * (R * 512) + r * 512);
            uint32_t b[MT][8];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              b[mt][0] = xa[mt].x; b[mt][1] = xa[mt].y; b[mt][2] = xa[mt].z; b[mt][3] = xa[mt].w;
              b[mt][4] = xb[mt].x; b[mt][5] = xb[mt].y; b[mt][6] = xb[mt].z; b[mt][7] = xb[mt].w;
            }
            if (s == nt - 1) {
              __syncwarp();   // every lane has read the stage: it may be refilled
              if (lane == 0) fill_stage<R>(ring + stg * kStage, wsrc, kt + RING * kSK, kt1, &bars[stg]);
            }
            if (kt + s + 1 < kt1) {
#pragma unroll
              for (int mt = 0; mt < MT; ++mt)
                if (xok[mt]) { xa[mt] = __ldg(xp[mt] + 8 * (s + 1)); xb[mt] = __ldg(xp[mt] + 8 * (s + 1) + 1); }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if constexpr (MX) {
                // MXFP4: a word holds the four A-fragment bytes of k16 step j (two e2m1 per byte), expanded by the hardware
                // e2m1x2 -> f16x2 conversion; steps 0,1 belong to block 0 of the k tile, steps 2,3 to block 1
#pragma unroll
                for (int r = 0; r < R; ++r) {
                  const uint32_t u = j == 0 ? wuse[r].x : (j == 1 ? wuse[r].y : (j == 2 ? wuse[r].z : wuse[r].w));
                  const uint32_t a0 = cvt_e2m1x2_f16(u), a1 = cvt_e2m1x2_f16(u >> 8), a2 = cvt_e2m1x2_f16(u >> 16), a3 = cvt_e2m1x2_f16(u >> 24);
#pragma unroll
                  for (int mt = 0; mt < MT; ++mt)
                    mma_f16_16816_w4(j < 2 ? accg[r][mt] : accg2[r][mt], a0, a1, a2, a3, b[mt][2 * j], b[mt][2 * j + 1]);
                }
              } else {
                // int4: nibbles -> bf16 integers 128+q (one logic op per pair).  The zero point is NOT subtracted per
                // element: an extra MMA with an all-ones A operand accumulates sum_k x, and (128 + zero) * sum_k x is
                // removed when the group is flushed.
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(xsum[mt], ones, ones, ones, ones, b[mt][2 * j], b[mt][2 * j + 1]);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                  const uint32_t u = j == 0 ? wuse[r].x : (j == 1 ? wuse[r].y : (j == 2 ? wuse[r].z : wuse[r].w));
                  const uint32_t a0 = lop3_or_and(u, 0x000f000fu, 0x43004300u);
                  const uint32_t a1 = lop3_or_and(u >> 4, 0x000f000fu, 0x43004300u);
                  const uint32_t a2 = lop3_or_and(u >> 8, 0x000f000fu, 0x43004300u);
                  const uint32_t a3 = lop3_or_and(u >> 12, 0x000f000fu, 0x43004300u);
#pragma unroll
                  for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(accg[r][mt], a0, a1, a2, a3, b[mt][2 * j], b[mt][2 * j + 1]);
                }
              }
            }
            if ((s + 1) % G64 == 0) {
              const int gi = s / G64;
#pragma unroll
              for (int r = 0; r < R; ++r) {
                float sc0, sc1, zf0, zf1;
                if constexpr (MX) {
                  // e8m0 bytes of the two 32-wide blocks of this k tile: [block][16 rows]; rows g and g + 8 of each
                  const uint8_t* sb = reinterpret_cast<const uint8_t*>(szp - g + (size_t)gi * p.szw + (size_t)r * p.szg * p.szw);
                  sc0 = __uint_as_float((uint32_t)sb[g] << 23); sc1 = __uint_as_float((uint32_t)sb[g + 8] << 23);
                  zf0 = __uint_as_float((uint32_t)sb[16 + g] << 23); zf1 = __uint_as_float((uint32_t)sb[24 + g] << 23);
                } else {
                  const uint32_t s0 = szp[gi * 16 + r * p.szg * 16], s1 = szp[gi * 16 + r * p.szg * 16 + 8];
                  sc0 = __half2float(__ushort_as_half((unsigned short)(s0 & 0xffffu)));
                  sc1 = __half2float(__ushort_as_half((unsigned short)(s1 & 0xffffu)));
                  zf0 = bf16hi_to_f(s0);      // 128 + zero
                  zf1 = bf16hi_to_f(s1);
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                  if constexpr (MX) {
                    acc[r][mt][0] = fmaf(sc0, accg[r][mt][0], fmaf(zf0, accg2[r][mt][0], acc[r][mt][0]));
                    acc[r][mt][1] = fmaf(sc0, accg[r][mt][1], fmaf(zf0, accg2[r][mt][1], acc[r][mt][1]));
                    acc[r][mt][2] = fmaf(sc1, accg[r][mt][2], fmaf(zf1, accg2[r][mt][2], acc[r][mt][2]));
                    acc[r][mt][3] = fmaf(sc1, accg[r][mt][3], fmaf(zf1, accg2[r][mt][3], acc[r][mt][3]));
                  } else {
                    acc[r][mt][0] = fmaf(sc0, fmaf(-zf0, xsum[mt][0], accg[r][mt][0]), acc[r][mt][0]);
                    acc[r][mt][1] = fmaf(sc0, fmaf(-zf0, xsum[mt][1], accg[r][mt][1]), acc[r][mt][1]);
                    acc[r][mt][2] = fmaf(sc1, fmaf(-zf1, xsum[mt][2], accg[r][mt][2]), acc[r][mt][2]);
                    acc[r][mt][3] = fmaf(sc1, fmaf(-zf1, xsum[mt][3], accg[r][mt][3]), acc[r][mt][3]);
                  }
                }
              }
            }
          }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          xp[mt] += 8 * kSK;
          if (xok[mt] && t == 0 && kt + 3 * kSK < kt1) {
#pragma unroll
            for (int l = 0; l < kSK; ++l) asm volatile("prefetch.global.L1 [%0];" ::"l"(xp[mt] + 8 * kSK + 8 * l));
          }
        }
        stg ^= 1u;
        phase ^= (stg == 0u);
      }
    };
    if constexpr (MX) run16(std::integral_constant<int, 1>{});
    else if (p.g64 == 1) run16(std::integral_constant<int, 1>{});
    else if (p.g64 == 2) run16(std::integral_constant<int, 2>{});
    else run16(std::integral_constant<int, 4>{});
    }   // bf16 path
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
    // receive region over NVLink, wait (bounded) for the partials of all sources, then sum the W
    // partials in rank order -- every rank
    // adds the same numbers in the same order, so all ranks hold bit-identical results (the
    // property the reference keeps with its rank-ordered shared-memory sums, grimoire.cpp:6263-6366).
    // Receive regions are double-buffered by launch parity: a peer can be at most one fused launch
    // ahead, because its next launch needs this rank's next push.
    const int W = p.ar_world;
    const unsigned int e = p.ar_epochs[tile] + 1u;
    const size_t tiles = gridDim.x;
    const size_t par = e & 1u;
    // Every partial travels as one 8-byte {value, epoch} store (an aligned 8-byte store lands as a whole), so the
    // receiver polls the data slot itself: no system-scope fences and no separate flag, one one-way NVLink latency.
    for (int v = tid; v < NV; v += kThreads) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += red[w * NV + v];
      const size_t slot = par * (p.ar_half >> 1) + ((size_t)p.ar_rank * tiles + tile) * NV + v;
      for (int r = 0; r < W; ++r) {
        uint2* dst = reinterpret_cast<uint2*>(p.ar_recv[r]) + slot;
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(s)), "r"(e) : "memory");
      }
    }
    const uint2* mine = reinterpret_cast<const uint2*>(p.ar_recv[p.ar_rank]);
    for (int v = tid; v < NV; v += kThreads) {
      float s = 0.f;
      bool ok = true;
      for (int r = 0; r < W && ok; ++r) {
        const uint2* src = mine + par * (p.ar_half >> 1) + ((size_t)r * tiles + tile) * NV + v;
        uint32_t vx = 0u, vy = 0u;
        ok = false;
        for (unsigned int i = 0; i < p.ar_spin; ++i) {
          asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(vx), "=r"(vy) : "l"(src) : "memory");
          if (vy == e) { ok = true; break; }
          if (i > 64) __nanosleep(20);
        }
        if (!ok) grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x10000u | (r << 12) | (tile & 0xfff));
        s += __uint_as_float(vx);
      }
      if (ok) epilogue_store<MT, R, EPI>(p, tile, v, s, 0.f);
    }
    __syncthreads();
    if (tid == 0) p.ar_epochs[tile] = e;   // advance even after a timeout so later launches stay aligned
    return;
  }

  if (p.ksplit == 1) {
    if (EPI == EPI_SWIGLU) {
      constexpr int NH = NV / 2;  // r = 0 half holds the gate rows, r = 1 the up rows
      for (int i = tid; i < p.rt * NH; i += kThreads) {
        const int w0 = i / NH, v = i - w0 * NH, tl = blockIdx.x * p.rt + w0;
        if (tl >= p.ntiles) continue;
        float sg = 0.f, su = 0.f;
        for (int k = 0; k < p.ks; ++k) { sg += red[(w0 * p.ks + k) * NV + v]; su += red[(w0 * p.ks + k) * NV + NH + v]; }
        epilogue_store<MT, R, EPI>(p, tl, v, sg, su);
      }
    } else {
      for (int i = tid; i < p.rt * NV; i += kThreads) {
        const int w0 = i / NV, v = i - w0 * NV, tl = blockIdx.x * p.rt + w0;
        if (tl >= p.ntiles) continue;
        float s = 0.f;
        for (int k = 0; k < p.ks; ++k) s += red[(w0 * p.ks + k) * NV + v];
        epilogue_store<MT, R, EPI>(p, tl, v, s, 0.f);
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

static int grm_smallm_min_ctas() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("GRIMOIRE_SMALLM_MIN_CTAS"); v = e ? atoi(e) : 222; if (v < 1) v = 222; }
  return v;
}

template <int MT, int R, int EPI, int MATH>
int launch_i(const W4Params& p_in, cudaStream_t st) {
  constexpr int NV = R * MT * 4 * 32;
  constexpr int RING = RingDepth<MT>::v;
  const W4Params& p = p_in;
  W4Params q = p;
  q.ntiles = p.N / (16 * R);
  q.rt = 1;
  if (EPI != EPI_AR_ADD && p.ksplit == 1) {
    // as many row super-tiles per CTA as still leave one full wave of CTAs on 148 SMs
    while (q.rt < kWarps && q.ntiles / (q.rt * 2) >= p.min_ctas) q.rt *= 2;
  }
  q.ks = kWarps / q.rt;
  {
    const int G = (p.K >> 6) / p.g64;
    const int cta_groups = G / p.ksplit;
    q.szg = (cta_groups + q.ks - 1) / q.ks;
  }
  const size_t smem = (size_t)kWarps * RING * kSK * R * 512 + (size_t)kWarps * NV * sizeof(float) +
                      (size_t)kWarps * (RING + 1) * 8 + (size_t)kWarps * R * q.szg * 4 * q.szw;
  auto kfn = smallm_w4_kernel<MT, R, EPI, MATH>;
  static size_t attr_max = 48 * 1024;
  if (smem > 200 * 1024) return -2;
  if (smem > attr_max) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_max = smem;
  }
  dim3 grid((q.ntiles + q.rt - 1) / q.rt, p.ksplit);
  if (EPI == EPI_AR_ADD) {
    // CTAs of different ranks wait for one another's pushes: every CTA of this grid must be
    // resident at once, otherwise resident CTAs could wait for peers whose partner CTA has no SM.
    int per_sm = 0, dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kfn, kThreads, smem) != cudaSuccess) return -2;
    if ((long)per_sm * sms < (long)grid.x * grid.y) return -2;
  }
  kfn<<<grid, kThreads, smem, st>>>(q);
  GRM_LAUNCH_RET();
}

template <int MT, int R, int EPI>
int launch(const W4Params& p, cudaStream_t st) {
  if (p.mx) return launch_i<MT, R, EPI, 2>(p, st);
  return p.xq_hi ? launch_i<MT, R, EPI, 1>(p, st) : launch_i<MT, R, EPI, 0>(p, st);
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
// The instantiation the dispatcher picks for (M, epilogue, rows_per_cta): MT = 8-row batch tiles the kernel is built for
// (1, 2, 4 or 8), R = 16-row weight tiles per CTA.  The scratch of a split-K launch is ksplit * (N / (16 R)) * R * MT * 128
// floats and N / (16 R) counters; every entry point sizes it from this one function.
struct SmallMShape { int MT, R; };
inline SmallMShape smallm_shape(int M, int epi, int rows_per_cta) {
  const int mt8 = (M + 7) / 8;
  const int MT = mt8 <= 1 ? 1 : (mt8 <= 2 ? 2 : (mt8 <= 4 ? 4 : 8));
  const int R = (epi == EPI_SWIGLU) ? 2 : ((rows_per_cta == 32 && MT <= 2) ? 2 : 1);
  return {MT, R};
}

int dispatch(W4Params& p, int epi, int rows_per_cta, cudaStream_t st) {
  const SmallMShape shp = smallm_shape(p.M, epi, rows_per_cta);
  const int MT = shp.MT;
  {
    const int G = (p.K >> 6) / p.g64;
    const int cta_groups = G / p.ksplit;
    p.szg = (cta_groups + kWarps - 1) / kWarps;
  }
  if (epi == EPI_SWIGLU) {
    if (MT <= 1) return launch<1, 2, EPI_SWIGLU>(p, st);
    if (MT <= 2) return launch<2, 2, EPI_SWIGLU>(p, st);
    if (MT <= 4) return launch<4, 2, EPI_SWIGLU>(p, st);
    return launch<8, 2, EPI_SWIGLU>(p, st);
  }
  const bool r2 = shp.R == 2;
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
  if (M < 1 || M > 64 || (N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || (ldx & 7) || ((uintptr_t)x & 15)) return -2;
  const int G = K / group;
  if (ksplit < 1 || (G % ksplit)) return -2;
  if (ksplit > 1 && (!scratch || !counters)) return -2;
  W4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = (const bf16*)x; p.out = out;
  p.scratch = (float*)scratch; p.counters = (unsigned int*)counters;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldo = ldo; p.g64 = group / 64; p.ksplit = ksplit;
  p.status = grm_status_ptr(); p.ar_world = 1; p.ar_rank = 0; p.ar_epochs = nullptr; p.ar_spin = 0; p.ar_half = 0;
  for (int i = 0; i < 8; ++i) { p.ar_recv[i] = nullptr; p.ar_flags[i] = nullptr; }
  p.xq_hi = p.xq_lo = nullptr; p.xtab = nullptr; p.ldq = p.ldtab = 0; p.min_ctas = grm_smallm_min_ctas(); p.mx = 0; p.szw = 16;
  if (epi == EPI_AR_ADD) return -1;   // use grm_smallm_w4_allreduce
  return dispatch(p, epi, rows_per_cta, (cudaStream_t)stream);
}

// Row-parallel projection fused with the tensor-parallel all-reduce: h[M][ldo] (fp32) += sum over
// ranks of X_r . W_r^T.  recv / flags are arrays of `world` peer-mapped device pointers (see the
// W4Params comment for their layouts; recv needs 2*world*(N/16)*2048 floats per rank (two parity halves of {value, epoch}
// pairs sized for the widest launch, zero before first use), flags (unused since the pairs carry the epoch)
// (N/16)*world uints, epochs N/16 uints, all zero before first use).  Every rank must issue the same
// sequence of calls with the same M.  spin = poll limit of the arrival wait (0 = default ~0.1 s).
GRM_API int grm_smallm_w4_allreduce(const void* w, const void* sz, const void* x, void* h, int M, int N, int K, int ldx,
                                    int ldo, int group, const void* const* recv, const void* const* flags, void* epochs,
                                    int world, int rank, unsigned int spin, void* stream) {
  if (M < 1 || M > 64 || (N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || (ldx & 7) || ((uintptr_t)x & 15)) return -2;
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
  p.ar_half = (size_t)world * (size_t)(N / 16) * 2048;   // floats per parity half: the widest launch has 8 x 128 {value, epoch} pairs per 16-row tile
  p.xq_hi = p.xq_lo = nullptr; p.xtab = nullptr; p.ldq = p.ldtab = 0; p.min_ctas = grm_smallm_min_ctas(); p.mx = 0; p.szw = 16;
  return dispatch(p, EPI_AR_ADD, 16, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// Integer activation path: grm_quant_x_i8 turns bf16 rows into two int8 levels per quantisation group,
// grm_smallm_w4_i8 / grm_smallm_w4_allreduce_i8 are the products over them (same contracts as above).
// ---------------------------------------------------------------------------------------------
namespace {

// One CTA per row; a warp quantises one group at a time: delta = max|x| / 16256, Q = round(x / delta)
// = 128 * hi + lo with hi in [-127, 127], lo in [-64, 63].  Bytes are stored with columns (1, 2) of every
// 4 swapped, the order in which a weight word's even / odd nibbles enumerate k.
__global__ void __launch_bounds__(256) quant_x_i8_kernel(const bf16* __restrict__ x, int ldx, int K, int group, int8_t* __restrict__ qh,
                                                         int8_t* __restrict__ ql, int ldq, float2* __restrict__ tab, int ldtab) {
  const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int G = K / group;
  const int per = group / 32;              // elements per lane: 2, 4 or 8 (contiguous)
  for (int gi = warp; gi < G; gi += 8) {
    const bf16* src = x + (size_t)m * ldx + (size_t)gi * group + lane * per;
    float v[8];
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      v[i] = i < per ? __bfloat162float(src[i]) : 0.f;
      mx = fmaxf(mx, fabsf(v[i]));
    }
    mx = warp_max(mx);
    const float delta = mx > 0.f ? mx / 16256.f : 1.f;
    const float inv = 1.f / delta;
    int sum = 0;
    const size_t base = (size_t)m * ldq + (size_t)gi * group + lane * per;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i < per) {
        const int q = __float2int_rn(v[i] * inv);
        const int hi = (q + 64) >> 7;
        sum += q;
        const int k = lane * per + i;                                  // column inside the group (group % 4 == 0)
        const int pos = (k & ~3) | ((k & 1) << 1) | ((k >> 1) & 1);    // swap bits 0 and 1
        qh[base - (size_t)(lane * per) + pos] = (int8_t)hi;
        ql[base - (size_t)(lane * per) + pos] = (int8_t)(q - 128 * hi);
      }
    }
#pragma unroll
    for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (lane == 0) tab[(size_t)m * ldtab + gi] = make_float2(delta, delta * (float)sum);
  }
}

}  // namespace

// x bf16 [M][ldx] -> xq_hi / xq_lo int8 [M][ldq] (ldq % 16 == 0) and xtab float2 [M][ldtab] (ldtab >= K / group).
GRM_API int grm_quant_x_i8(const void* x, int ldx, int M, int K, int group, void* xq_hi, void* xq_lo, int ldq, void* xtab, int ldtab,
                           void* stream) {
  if (M < 1 || (group != 64 && group != 128 && group != 256) || (K % group) || (ldq & 15) || ldq < K || ldtab < K / group) return -2;
  quant_x_i8_kernel<<<M, 256, 0, (cudaStream_t)stream>>>((const bf16*)x, ldx, K, group, (int8_t*)xq_hi, (int8_t*)xq_lo, ldq,
                                                        (float2*)xtab, ldtab);
  GRM_LAUNCH_RET();
}

GRM_API int grm_smallm_w4_i8(const void* w, const void* sz, const void* xq_hi, const void* xq_lo, int ldq, const void* xtab, int ldtab,
                             void* out, void* scratch, void* counters, int M, int N, int K, int ldo, int group, int epi,
                             int rows_per_cta, int ksplit, void* stream) {
  if (M < 1 || M > 64 || (N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || (ldq & 15) ||
      ((uintptr_t)xq_hi & 15) || ((uintptr_t)xq_lo & 15) || !xtab)
    return -2;
  const int G = K / group;
  if (ksplit < 1 || (G % ksplit)) return -2;
  if (ksplit > 1 && (!scratch || !counters)) return -2;
  W4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = nullptr; p.out = out;
  p.scratch = (float*)scratch; p.counters = (unsigned int*)counters;
  p.M = M; p.N = N; p.K = K; p.ldx = 0; p.ldo = ldo; p.g64 = group / 64; p.ksplit = ksplit;
  p.status = grm_status_ptr(); p.ar_world = 1; p.ar_rank = 0; p.ar_epochs = nullptr; p.ar_spin = 0; p.ar_half = 0;
  for (int i = 0; i < 8; ++i) { p.ar_recv[i] = nullptr; p.ar_flags[i] = nullptr; }
  p.xq_hi = (const int8_t*)xq_hi; p.xq_lo = (const int8_t*)xq_lo; p.xtab = (const float2*)xtab; p.ldq = ldq; p.ldtab = ldtab; p.min_ctas = grm_smallm_min_ctas(); p.mx = 0; p.szw = 16;
  if (epi == EPI_AR_ADD) return -1;
  return dispatch(p, epi, rows_per_cta, (cudaStream_t)stream);
}

GRM_API int grm_smallm_w4_allreduce_i8(const void* w, const void* sz, const void* xq_hi, const void* xq_lo, int ldq, const void* xtab,
                                       int ldtab, void* h, int M, int N, int K, int ldo, int group, const void* const* recv,
                                       const void* const* flags, void* epochs, int world, int rank, unsigned int spin, void* stream) {
  if (M < 1 || M > 64 || (N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || (ldq & 15) ||
      ((uintptr_t)xq_hi & 15) || ((uintptr_t)xq_lo & 15) || !xtab)
    return -2;
  if (world < 1 || world > 8 || rank < 0 || rank >= world || !recv || !flags || !epochs) return -2;
  W4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = nullptr; p.out = h;
  p.scratch = nullptr; p.counters = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldx = 0; p.ldo = ldo; p.g64 = group / 64; p.ksplit = 1;
  for (int i = 0; i < 8; ++i) {
    p.ar_recv[i] = i < world ? (float*)const_cast<void*>(recv[i]) : nullptr;
    p.ar_flags[i] = i < world ? (unsigned int*)const_cast<void*>(flags[i]) : nullptr;
  }
  p.ar_epochs = (unsigned int*)epochs; p.status = grm_status_ptr(); p.ar_world = world; p.ar_rank = rank;
  p.ar_spin = spin ? spin : 2000000u;
  p.ar_half = (size_t)world * (size_t)(N / 16) * 2048;   // floats per parity half: the widest launch has 8 x 128 {value, epoch} pairs per 16-row tile
  p.xq_hi = (const int8_t*)xq_hi; p.xq_lo = (const int8_t*)xq_lo; p.xtab = (const float2*)xtab; p.ldq = ldq; p.ldtab = ldtab; p.min_ctas = grm_smallm_min_ctas(); p.mx = 0; p.szw = 16;
  return dispatch(p, EPI_AR_ADD, 16, (cudaStream_t)stream);
}

// MXFP4 weights in the tiled layout of tile_mx (formats/w4_tile_layout.py); x16p: f16 activations in lane order
// (grm_x16_lane_order in smallm_mx.cu).  Same epilogues and split-K contract as grm_smallm_w4.
GRM_API int grm_smallm_mx_tiled(const void* w, const void* sz, const void* x16p, void* out, void* scratch, void* counters, int M, int N,
                                int K, int ldx, int ldo, int epi, int rows_per_cta, int ksplit, void* stream) {
  if (M < 1 || M > 64 || (N % 32) || (K % 64) || (ldx & 7) || ((uintptr_t)x16p & 15)) return -2;
  const int G = K / 64;
  if (ksplit < 1 || (G % ksplit)) return -2;
  if (ksplit > 1 && (!scratch || !counters)) return -2;
  W4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = (const bf16*)x16p; p.out = out;
  p.scratch = (float*)scratch; p.counters = (unsigned int*)counters;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldo = ldo; p.g64 = 1; p.ksplit = ksplit;
  p.status = grm_status_ptr(); p.ar_world = 1; p.ar_rank = 0; p.ar_epochs = nullptr; p.ar_spin = 0; p.ar_half = 0;
  for (int i = 0; i < 8; ++i) { p.ar_recv[i] = nullptr; p.ar_flags[i] = nullptr; }
  p.xq_hi = p.xq_lo = nullptr; p.xtab = nullptr; p.ldq = p.ldtab = 0; p.min_ctas = grm_smallm_min_ctas();
  p.mx = 1; p.szw = 8;
  if (epi == EPI_AR_ADD) return -1;
  return dispatch(p, epi, rows_per_cta, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// grm_smallm_w4_noalloc: the split-K small-M product for callers that must not allocate.
// Declared and documented in smallm_w4_noalloc.h.
// ---------------------------------------------------------------------------------------------
#include <mutex>

#include "smallm_w4_noalloc.h"

namespace {

// Scratch that the ordinary entry point receives from its caller lives here instead, inside the
// library image: every GPU that loads the library carries these 4 MiB + 16 KiB until the process exits.
static __device__ __align__(256) float g_noalloc_partials[GRM_NOALLOC_MAX_PARTIAL_FLOATS];
static __device__ __align__(256) unsigned int g_noalloc_counters[GRM_NOALLOC_MAX_TILES];

struct NoAllocDev {
  float* partials = nullptr;
  unsigned int* counters = nullptr;
  int rc = 0;
  std::once_flag once;
};
NoAllocDev g_noalloc_dev[64];

// In host code the two array names above are only stand-ins; a kernel needs the device addresses,
// which cudaGetSymbolAddress hands out for the device that is current at the time of the call.
// Runs once per device ordinal, also when several host threads make their first call together.
int noalloc_setup(int dev) {
  NoAllocDev& d = g_noalloc_dev[dev];
  std::call_once(d.once, [&d]() {
    void* a = nullptr;
    void* b = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&a, g_noalloc_partials);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&b, g_noalloc_counters);
    d.partials = (float*)a;
    d.counters = (unsigned int*)b;
    d.rc = (int)e;
  });
  return d.rc;
}

}  // namespace

GRM_API int grm_smallm_w4_noalloc(const void* w, const void* sz, const void* x, void* out, int M, int N, int K, int ldx,
                                  int ldo, int group, int epi, int rows_per_cta, int ksplit, void* stream) {
  if (M < 1 || M > 64 || (N % 32) || (K % 64) || (group != 64 && group != 128 && group != 256) || (K % group) || (ldx & 7) || ((uintptr_t)x & 15)) return -2;
  if (epi < EPI_BF16 || epi > EPI_SWIGLU) return -1;
  const int G = K / group;
  if (ksplit < 1 || (G % ksplit)) return -2;
  const SmallMShape shp = smallm_shape(M, epi, rows_per_cta);
  const long tiles = N / (16 * shp.R);
  const long need = (long)ksplit * tiles * shp.R * shp.MT * 128;
  // a single K slice touches neither the partial sums nor the counters: no limit applies and nothing is cleared
  if (ksplit > 1 && (tiles > GRM_NOALLOC_MAX_TILES || need > GRM_NOALLOC_MAX_PARTIAL_FLOATS)) return GRM_NOALLOC_TOO_LARGE;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -2;
  int rc = noalloc_setup(dev);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (ksplit > 1) {
    // The counters are shared by every call and must start at zero; a previous call that was cut short
    // could have left them otherwise, so they are cleared on the caller's stream each time.
    e = cudaMemsetAsync(g_noalloc_dev[dev].counters, 0, sizeof(unsigned int) * (size_t)tiles, st);
    if (e != cudaSuccess) return (int)e;
  }
  W4Params p;
  p.w = (const uint4*)w; p.sz = (const uint32_t*)sz; p.x = (const bf16*)x; p.out = out;
  p.scratch = g_noalloc_dev[dev].partials; p.counters = g_noalloc_dev[dev].counters;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldo = ldo; p.g64 = group / 64; p.ksplit = ksplit;
  p.status = grm_status_ptr(); p.ar_world = 1; p.ar_rank = 0; p.ar_epochs = nullptr; p.ar_spin = 0; p.ar_half = 0;
  for (int i = 0; i < 8; ++i) { p.ar_recv[i] = nullptr; p.ar_flags[i] = nullptr; }
  p.xq_hi = p.xq_lo = nullptr; p.xtab = nullptr; p.ldq = p.ldtab = 0; p.min_ctas = grm_smallm_min_ctas(); p.mx = 0; p.szw = 16;
  return dispatch(p, epi, rows_per_cta, st);
}
