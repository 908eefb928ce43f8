// decode_mega: the single-row decode step of a dense int4 decoder as a chain of weight-streaming phases inside ONE
// persistent kernel (one CTA per SM), instead of one launch per projection (the reference replays ~29 launches per layer
// and token from a command graph, src/grimoire.cpp:23640-23712; its int4 GEMV is src/gemv_decode.cpp:77-347).
//
// A phase is y = epilogue(W . prologue(x)) for one int4 (group 64/128/256) weight in the tiled execution layout of
// formats/w4_tile_layout.py.  A launch runs `count` consecutive phases of a device-resident table, e.g. for layer l:
//   o_proj (+= h)  |  RMSNorm + gate|up + SwiGLU  |  down_proj (+= h)  |  RMSNorm + q|k|v of layer l + 1
// with a grid-wide barrier between phases.  What makes it fast:
//   * the weight bytes of a phase are cut into equal contiguous ranges, one per CTA (a 32-row pair of the tiled layout
//     is one contiguous K-major run, so a range is a byte range of the weight array); a producer warp streams its
//     range through a shared-memory ring with cp.async.bulk and simply keeps going into the NEXT phase's range while
//     the consumers sit in the grid barrier -- weight addresses do not depend on activations, so HBM never drains at
//     a phase boundary;
//   * the product runs on the half2 multiply-add pipe at 13 instructions per eight weights (one logic op per nibble
//     pair builds fp16 {1024 + q}, one subtract / fma removes bias and zero point exactly, one fma multiplies); for a
//     single activation row that beats the legacy tensor-core path on this part (see word_fma);
//   * a row pair whose K range straddles two CTAs is finished by the CTA that owns its first stage: the others publish
//     their partial sums (they meet that row pair first in their range, the owner meets it last), the owner adds them
//     in CTA order, so results do not depend on timing;
//   * activations are staged once per phase and CTA as fp16 scaled by a power of two so that |x| <= 256: the fp16
//     partial sums of a 64-column unit cannot overflow whatever the activations are, the scale is undone in fp32.
// The row-parallel phases can all-reduce their result over tensor-parallel ranks in the same epilogue ({value, epoch}
// pushes into the peers' receive regions, as in gemv_w4.cu).
//
// Every wait (ring barriers, grid barrier, partial-sum flags, peer pushes) is bounded; after the first expiry the
// kernel sets an abort word, every later wait returns at once, outstanding bulk copies are drained and the kernel
// exits normally with GRM_ERR_* recorded in the status block.
#include "common.cuh"

namespace {

constexpr int kCW = 16;                               // consumer warps
constexpr int kThreads = (kCW + 1) * 32;              // + one producer warp
constexpr int kUnits = 16;                            // 1 KB units (32 rows x 64 columns) per ring stage: one per consumer warp
constexpr int kSzSeg = kUnits * 64;                   // scale words of one 16-row tile for a stage (<= one group per unit)
constexpr int kSlotBytes = kUnits * 1024 + 2 * kSzSeg;
constexpr int kMaxSlots = 12;
constexpr int kMaxK = 20480;                          // kVec vectors of 8 per consumer thread; fp16 row leaves room for the ring

enum { PRO_X = 0, PRO_NORM = 1 };
enum { EPI_BF16 = 0, EPI_F32 = 1, EPI_ADD = 2, EPI_SWIGLU = 3 };

struct MegaPhase {
  const void* w;        // tiles [rp][K/64][2][32] x 16 bytes
  const void* sz;       // [2 rp][K/group][16] words: fp16 scale | bf16(128 + zero) << 16
  const void* x;        // PRO_X: bf16 [K]
  const void* nw;       // PRO_NORM: fp32 [K] norm weight (the input is the residual row h)
  void* out;            // bf16 [N] | fp32 [N] | fp32 [N] accumulated | bf16 [N / 2]
  int N, rp, K, g64;
  int pro, epi;
  float eps, offset;
  int ar_region;        // >= 0: all-reduce the result over ranks before the accumulate (EPI_ADD only)
  int pad;
};
static_assert(sizeof(MegaPhase) == 80, "host mirror in ops/mega.py");

struct MegaParams {
  const MegaPhase* phases;
  int first, count;
  const float* h;                 // fp32 residual row (PRO_NORM input)
  unsigned int* sync;             // [0] barrier arrivals (monotonic), [1] unused, [2] abort
  uint2* parts;                   // [row pair][pstride][32] {partial sum, epoch} of the CTAs that do not own the row pair
  int pstride;
  unsigned int* status;
  unsigned int spin;
  int nslots, xs_bytes, xsum_bytes;
  // tensor-parallel exchange (world > 1): receive regions [2][world][ar_rows] x {value, epoch}
  float* ar_recv[8];
  int ar_world, ar_rank, ar_rows;
  // optional timeline (null = off): [phase][CTA][5] SM clock values of thread 0 -- phase entered, grid barrier passed,
  // activations staged, last ring stage consumed, row pairs finalised
  long long* timeline;
};

struct Ctx {
  unsigned int* status;
  unsigned int* sync;
  volatile int* s_abort;
  unsigned int spin;
};

__host__ __device__ inline long long part_begin(long long T, int c, int nC) { return (long long)c * T / nC; }
__host__ __device__ inline int cta_of(long long T, long long s, int nC) { return (int)(((s + 1) * nC - 1) / T); }

__device__ __forceinline__ void cons_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory"); }

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void raise_abort(const Ctx& c, unsigned int code, unsigned int tag) {
  grm_set_error(c.status, code, tag);
  *c.s_abort = 1;
  atomicExch(c.sync + 2, 1u);
}
// true when some wait of this grid already gave up (checked inside every poll loop)
__device__ __forceinline__ bool aborted(const Ctx& c, unsigned int i) {
  if (*c.s_abort) return true;
  if ((i & 255u) == 255u && ld_relaxed_gpu(c.sync + 2) != 0u) { *c.s_abort = 1; return true; }
  return false;
}

// shared-memory accessors on 32-bit addresses (no generic-pointer arithmetic in the hot loop)
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_arrive_s(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool ring_wait(uint64_t* bar, uint32_t parity, const Ctx& c, uint32_t tag) {
  if (mbar_try_wait(bar, parity)) return true;
  for (unsigned int i = 0; i < c.spin; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (aborted(c, i)) return false;
    if (i > 64) __nanosleep(32);
  }
  raise_abort(c, GRM_ERR_MBAR_TIMEOUT, tag);
  return false;
}

// One thread per CTA, between two CTA-level barriers.  A single counter that only grows: a CTA's arrival is one
// release-add, the round is over when the count reaches the next multiple of the grid size -- one L2 round trip for the
// last arriver, about two for the others, no reset and no second word.  The count survives launches (a captured
// launch can be replayed); comparisons are wrap-safe.
__device__ __forceinline__ void grid_barrier(const Ctx& c, unsigned int nblocks, uint32_t tag) {
  if (*c.s_abort) return;
  unsigned int old;
  asm volatile("atom.add.release.gpu.global.u32 %0, [%1], 1;" : "=r"(old) : "l"(c.sync) : "memory");
  const unsigned int target = (old / nblocks + 1u) * nblocks;
  if (old + 1u != target) {
    bool ok = false;
    for (unsigned int i = 0; i < c.spin; ++i) {
      if ((int)(ld_acquire_gpu(c.sync) - target) >= 0) { ok = true; break; }
      if (aborted(c, i)) return;
      if (i > 200) __nanosleep(20);
    }
    if (!ok) { raise_abort(c, GRM_ERR_FLAG_TIMEOUT, 0x30000u | tag); return; }
  } else {
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
  }
}

__device__ __forceinline__ uint32_t lop3_or_and(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));   // (a & mask) | orv
  return r;
}
// Eight weights of one 32-bit word (rows g and g + 8, four consecutive columns) times their activations on the half2
// multiply-add pipe: one logic op per nibble pair builds {1024 + q, 1024 + q'} (odd nibbles: {1024 + 16 q, ...}), one
// half2 subtract / fma removes the bias together with the zero point exactly, one half2 fma multiplies.  (A legacy
// mma.sync would do the eight products in one instruction, but on this part it occupies its sub-partition for about nine
// cycles and does not overlap with the logic ops feeding it: measured, the tensor-core form of this loop runs at half
// the rate of this one for a single activation row.)
__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
__device__ __forceinline__ void word_fma(uint32_t w, __half2 x01, __half2 x23, __half2 c_lo, __half2 c_hi, __half2& a0, __half2& a1) {
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  const uint32_t w2 = __umulhi(w, 1u << 24);          // w >> 8 on the multiply pipe (the logic pipe is the busy one)
  const __half2 l0 = as_h2(lop3_or_and(w, 0x000f000fu, 0x64006400u)), h0 = as_h2(lop3_or_and(w, 0x00f000f0u, 0x64006400u));
  const __half2 l1 = as_h2(lop3_or_and(w2, 0x000f000fu, 0x64006400u)), h1 = as_h2(lop3_or_and(w2, 0x00f000f0u, 0x64006400u));
  a0 = __hfma2(__hsub2(l0, c_lo), x01, a0);                    // row g,     columns 4j, 4j + 1
  a1 = __hfma2(__hfma2(h0, sixteenth, c_hi), x01, a1);         // row g + 8
  a0 = __hfma2(__hsub2(l1, c_lo), x23, a0);                    // row g,     columns 4j + 2, 4j + 3
  a1 = __hfma2(__hfma2(h1, sixteenth, c_hi), x23, a1);
}

// One 64-column unit of one 16-row tile: 16 products per row and lane in fp16 (|x| <= 256 after the staging scale and
// |q - zero| <= 16, so a half accumulates at most 8 * 16 * 256 < 65504), folded into the fp32 row sums with the scale.
// sz word: fp16 scale | bf16(128 + zero).
__device__ __forceinline__ void unit_fma(const uint4& w, const uint4& xa, const uint4& xb, uint32_t s_lo, uint32_t s_hi, float& f_lo, float& f_hi) {
  const __half2 c_lo = __float2half2_rn(bf16hi_to_f(s_lo) + 896.f);        // 1024 + zero
  const __half2 c_hi = __float2half2_rn(64.f - bf16hi_to_f(s_hi));         // -(64 + zero) = 64 - (128 + zero)
  __half2 a0 = __float2half2_rn(0.f), a1 = a0, b0 = a0, b1 = a0;
  word_fma(w.x, as_h2(xa.x), as_h2(xa.y), c_lo, c_hi, a0, a1);
  word_fma(w.y, as_h2(xa.z), as_h2(xa.w), c_lo, c_hi, b0, b1);
  word_fma(w.z, as_h2(xb.x), as_h2(xb.y), c_lo, c_hi, a0, a1);
  word_fma(w.w, as_h2(xb.z), as_h2(xb.w), c_lo, c_hi, b0, b1);
  const float2 r0 = __half22float2(__hadd2(a0, b0)), r1 = __half22float2(__hadd2(a1, b1));
  f_lo = fmaf(__low2float(as_h2(s_lo)), r0.x + r0.y, f_lo);
  f_hi = fmaf(__low2float(as_h2(s_hi)), r1.x + r1.y, f_hi);
}

// Stage geometry of a phase
struct Geo {
  int KT, SPR, g64s;        // k tiles, stages per row pair, log2(k tiles per group)
  long long T, sb, se;      // stages in total, this CTA's range
};
__device__ __forceinline__ Geo make_geo(const MegaPhase& ph, int cta, int nC) {
  Geo g;
  g.KT = ph.K >> 6;
  g.SPR = (g.KT + kUnits - 1) / kUnits;
  g.g64s = ph.g64 == 4 ? 2 : (ph.g64 == 2 ? 1 : 0);
  g.T = (long long)ph.rp * g.SPR;
  g.sb = part_begin(g.T, cta, nC);
  g.se = part_begin(g.T, cta + 1, nC);
  return g;
}

// ---- activations of a phase -> fp16 in shared memory, scaled by a power of two; per-unit sums -------------------------
// One global round trip: every thread pulls all of its 8-element vectors first (up to kVec of them live in registers;
// wider inputs take further rounds), the block agrees on the sum of squares and the largest magnitude, then each
// thread converts what it holds.  A 64-column unit is 8 neighbouring lanes' vectors, so its sum is three shuffles.
constexpr int kVec = 5;

__device__ __forceinline__ void unpack8(const uint4& q, float (&v)[8]) {
  v[0] = bf16lo_to_f(q.x); v[1] = bf16hi_to_f(q.x); v[2] = bf16lo_to_f(q.y); v[3] = bf16hi_to_f(q.y);
  v[4] = bf16lo_to_f(q.z); v[5] = bf16hi_to_f(q.z); v[6] = bf16lo_to_f(q.w); v[7] = bf16hi_to_f(q.w);
}

__device__ void stage_x(const MegaPhase& ph, const float* h, __half* xs, float* xsum, float* red_a, float* red_b, int tid,
                        float& inv_scale) {
  const int lane = tid & 31, warp = tid >> 5;
  const int nv = ph.K >> 3;
  const bool norm = ph.pro == PRO_NORM;
  // what a thread keeps between the two steps: its bf16 vectors (PRO_X), or the fp32 residual values of its first
  // kVecN vectors (PRO_NORM; hidden sizes up to 8192 -- wider rows re-read the rest, the norm weights always come back
  // from the read-only cache)
  constexpr int kVecN = 2;
  uint4 raw[kVec];
  float4 ha[kVecN], hb[kVecN];
  float ss = 0.f, amax = 0.f;
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = tid + i * (kCW * 32);
    if (idx < nv && !norm) raw[i] = __ldcg(reinterpret_cast<const uint4*>(ph.x) + idx);
  }
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = tid + i * (kCW * 32);
    if (idx < nv) {
      if (norm) {
        const float4 a = __ldcg(reinterpret_cast<const float4*>(h) + 2 * idx), b = __ldcg(reinterpret_cast<const float4*>(h) + 2 * idx + 1);
        const float4 wa = __ldg(reinterpret_cast<const float4*>(ph.nw) + 2 * idx), wb = __ldg(reinterpret_cast<const float4*>(ph.nw) + 2 * idx + 1);
        if (i < kVecN) { ha[i] = a; hb[i] = b; }
        const float hv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) { ss += hv[j] * hv[j]; amax = fmaxf(amax, fabsf(hv[j] * (ph.offset + wv[j]))); }
      } else {
        float v[8];
        unpack8(raw[i], v);
#pragma unroll
        for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
      }
    }
  }
  ss = warp_sum(ss);
  amax = warp_max(amax);
  if (lane == 0) { red_a[warp] = ss; red_b[warp] = amax; }
  cons_bar();
  float tot = 0.f;
  amax = 0.f;
#pragma unroll
  for (int k = 0; k < kCW; ++k) { tot += red_a[k]; amax = fmaxf(amax, red_b[k]); }
  float rnorm = 1.f;
  if (norm) {
    rnorm = rsqrtf(tot / (float)ph.K + ph.eps);
    amax *= rnorm * 1.01f;                                           // bound of |x| after the bf16 rounding below
  }
  int e = 0;
  if (amax > 256.f && amax < 3.0e38f) e = ilogbf(amax) - 7;         // amax * 2^-e < 256
  const float scale = __int_as_float((127 - e) << 23);
  inv_scale = __int_as_float((127 + e) << 23);
#pragma unroll
  for (int i = 0; i < kVec; ++i) {
    const int idx = tid + i * (kCW * 32);
    float v[8];
    if (idx < nv) {
      if (norm) {
        float4 a, b;
        if (i < kVecN) { a = ha[i]; b = hb[i]; }
        else { a = __ldcg(reinterpret_cast<const float4*>(h) + 2 * idx); b = __ldcg(reinterpret_cast<const float4*>(h) + 2 * idx + 1); }
        const float4 wa = __ldg(reinterpret_cast<const float4*>(ph.nw) + 2 * idx), wb = __ldg(reinterpret_cast<const float4*>(ph.nw) + 2 * idx + 1);
        const float hv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        const float wv[8] = {wa.x, wa.y, wa.z, wa.w, wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(__float2bfloat16(hv[j] * rnorm * (ph.offset + wv[j])));   // the norm kernel's rounding
      } else {
        unpack8(raw[i], v);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = 0.f;
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 hh = __floats2half2_rn(v[2 * j] * scale, v[2 * j + 1] * scale);
      o[j] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    if (idx < nv) *reinterpret_cast<uint4*>(xs + 8 * idx) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  cons_bar();
}

// ---- one finished row pair: sum the warps' partials, meet the other CTAs' shares, apply the epilogue ------------------
__device__ void finalize_pair(const MegaParams& p, const MegaPhase& ph, const Geo& geo, const Ctx& c, const float (*red)[32], int rp,
                              int si0, int cta, int nC, int lane, float inv_scale, unsigned int epoch) {
  const int tp = lane >> 4, r = lane & 15;
  const bool owner = si0 == 0;             // this CTA holds the row pair's first stage
  float sum = 0.f;
#pragma unroll
  for (int u = 0; u < kCW; ++u) sum += red[u][lane];        // lane = 16 * tile + row, warps in a fixed order
  sum *= inv_scale;
  // CTAs that share this row pair, and this CTA's place among them.  With at least one stage per CTA every CTA between
  // the first and the last stage's owner takes part; with fewer stages than CTAs each stage has a CTA of its own.
  const long long s_first = (long long)rp * geo.SPR;
  int nparts, my_part;
  if (geo.T >= nC) {
    const int c_first = cta_of(geo.T, s_first, nC);
    nparts = cta_of(geo.T, s_first + geo.SPR - 1, nC) - c_first + 1;
    my_part = cta - c_first;
  } else {
    nparts = geo.SPR;
    my_part = si0;
  }
  // Partial sums travel as aligned 8-byte {value, epoch} pairs: the store lands as a whole, so the owner polls the
  // slot itself until its epoch word is this phase's -- no fence, no counter, one L2 round trip.
  if (!owner) {
    uint2* dst = p.parts + ((size_t)rp * p.pstride + (my_part - 1)) * 32 + lane;
    asm volatile("st.relaxed.gpu.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(sum)), "r"(epoch) : "memory");
    return;
  }
  const int row = rp * 32 + lane;
  // the accumulate epilogue's old value is fetched while the partial sums are awaited
  float hold = 0.f;
  const bool add_local = ph.epi == EPI_ADD && row < ph.N;
  if (add_local) hold = __ldcg(reinterpret_cast<const float*>(ph.out) + row);
  if (nparts > 1) {
    bool ok = true;
    for (int j = 0; j < nparts - 1 && ok; ++j) {
      const uint2* src = p.parts + ((size_t)rp * p.pstride + j) * 32 + lane;
      uint32_t vx = 0u, vy = 0u;
      bool got = false;
      if (!*c.s_abort) {
        for (unsigned int i = 0; i < c.spin; ++i) {
          asm volatile("ld.relaxed.gpu.global.v2.b32 {%0, %1}, [%2];" : "=r"(vx), "=r"(vy) : "l"(src) : "memory");
          if (vy == epoch) { got = true; break; }
          if (aborted(c, i)) break;
          if (i > 64) __nanosleep(20);
        }
        if (!got && !*c.s_abort) raise_abort(c, GRM_ERR_FLAG_TIMEOUT, 0x40000u | (unsigned int)(rp & 0xffff));
      }
      ok = __all_sync(0xffffffffu, got);
      sum += __uint_as_float(vx);
    }
    if (!ok) return;
  }
  if (ph.epi == EPI_SWIGLU) {
    const float up = __shfl_down_sync(0xffffffffu, sum, 16);
    const int col = rp * 16 + r;
    if (tp == 0 && col < (ph.N >> 1)) reinterpret_cast<bf16*>(ph.out)[col] = __float2bfloat16(silu_f(sum) * up);
    return;
  }
  if (ph.epi == EPI_ADD && ph.ar_region >= 0 && p.ar_world > 1) {
    // one-shot all-reduce of the 32 partial sums: an aligned 8-byte {value, epoch} store per peer, the receiver polls
    // the slot itself until its epoch word is this phase's; partials are added in rank order on every rank
    const int W = p.ar_world;
    const size_t base = (size_t)ph.ar_region * W * p.ar_rows;
    for (int rk = 0; rk < W; ++rk) {
      if (rk == p.ar_rank) continue;
      uint2* dst = reinterpret_cast<uint2*>(p.ar_recv[rk]) + base + (size_t)p.ar_rank * p.ar_rows + row;
      asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(sum)), "r"(epoch) : "memory");
    }
    float tot = 0.f;
    bool ok = true;
    for (int rk = 0; rk < W && ok; ++rk) {
      if (rk == p.ar_rank) { tot += sum; continue; }
      const uint2* src = reinterpret_cast<const uint2*>(p.ar_recv[p.ar_rank]) + base + (size_t)rk * p.ar_rows + row;
      uint32_t vx = 0u, vy = 0u;
      bool got = false;
      if (!*c.s_abort) {
        for (unsigned int i = 0; i < c.spin; ++i) {
          asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(vx), "=r"(vy) : "l"(src) : "memory");
          if (vy == epoch) { got = true; break; }
          if (aborted(c, i)) break;
          if (i > 64) __nanosleep(20);
        }
        if (!got && !*c.s_abort) raise_abort(c, GRM_ERR_FLAG_TIMEOUT, 0x50000u | (unsigned int)(rk << 12) | (unsigned int)(rp & 0xfff));
      }
      ok = got;
      tot += __uint_as_float(vx);
    }
    sum = tot;
    if (!__all_sync(0xffffffffu, ok)) return;
  }
  if (row < ph.N) {
    if (ph.epi == EPI_BF16) reinterpret_cast<bf16*>(ph.out)[row] = __float2bfloat16(sum);
    else if (ph.epi == EPI_F32) reinterpret_cast<float*>(ph.out)[row] = sum;
    else reinterpret_cast<float*>(ph.out)[row] = hold + sum;
  }
}

// BPS = CTAs per SM.  Two CTAs of 16 consumer warps each double the warps that hide the latency of the dependent
// half2 chains (at 56 registers a thread and half the ring each); one CTA keeps the deeper ring.
template <int BPS>
__global__ void __launch_bounds__(kThreads, BPS) decode_mega_kernel(const MegaParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __half* xs = reinterpret_cast<__half*>(smem);
  float* xsum = reinterpret_cast<float*>(smem + p.xs_bytes);
  float* red = xsum + p.xsum_bytes / 4;                           // [2][kCW][32]
  float* red_a = red + 2 * kCW * 32;                              // [kCW]
  float* red_b = red_a + kCW;                                     // [kCW]
  uint64_t* full = reinterpret_cast<uint64_t*>(red_b + kCW);      // 8-byte aligned: every size above is a multiple of 64
  uint64_t* empty = full + kMaxSlots;
  int* s_abort = reinterpret_cast<int*>(empty + kMaxSlots);
  uint8_t* ring = smem + ((p.xs_bytes + p.xsum_bytes + (2 * kCW * 32 + 2 * kCW) * 4 + 2 * kMaxSlots * 8 + 64 + 1023) & ~1023);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, nC = gridDim.x;
  const int S = p.nslots;
  if (tid == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(full + i, 1); mbar_init(empty + i, kCW); }
    *s_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  Ctx c;
  c.status = p.status; c.sync = p.sync; c.s_abort = s_abort; c.spin = p.spin;

  if (warp == kCW) {
    // ================= producer: this CTA's byte range of every phase, through the ring =================
    // Three lanes issue the three copies of a stage with ONE instruction each step (lane 0: the weights, lanes 1 / 2:
    // the scale words of the two 16-row tiles): the producer is a single warp competing with sixteen busy ones for
    // issue slots, so its per-stage instruction chain is kept as short as possible.
    if (lane < 3) {
      const uint32_t ring_s = smem_u32(ring), full_s = smem_u32(full), empty_s = smem_u32(empty);
      const uint32_t dst_off = lane == 0 ? 0u : (uint32_t)(kUnits * 1024 + (lane - 1) * kSzSeg);
      uint32_t issued = 0;
      const uint32_t smask = (uint32_t)S - 1u, sshift = (uint32_t)__ffs(S) - 1u;
      bool live = true;
      for (int pi = 0; pi < p.count && live; ++pi) {
        const MegaPhase ph = p.phases[p.first + pi];
        const Geo geo = make_geo(ph, cta, nC);
        if (geo.sb >= geo.se) continue;
        int rp = (int)(geo.sb / geo.SPR), si = (int)(geo.sb - (long long)rp * geo.SPR);
        const int G = geo.KT >> geo.g64s;
        // lane 0 walks one contiguous byte range of the weight array; the scale lanes recompute their short offsets
        const uint8_t* wsrc = reinterpret_cast<const uint8_t*>(ph.w) + ((size_t)rp * geo.KT + (size_t)kUnits * si) * 1024;
        const uint8_t* szb = reinterpret_cast<const uint8_t*>(ph.sz);
        for (long long s = geo.sb; s < geo.se; ++s) {
          const uint32_t slot = issued & smask, par = (issued >> sshift) & 1u;
          // slot reuse: wait until the consumers released its previous contents (parity of the previous round)
          if (issued >= (uint32_t)S && !mbar_test(empty_s + slot * 8u, par ^ 1u) && !ring_wait(empty + slot, par ^ 1u, c, 0x100u | slot)) live = false;
          live = __all_sync(0x7u, live);
          if (!live) break;
          const int nu = min(kUnits, geo.KT - kUnits * si);
          const int ng = nu >> geo.g64s, g0 = (kUnits * si) >> geo.g64s;
          const uint32_t fb = full_s + slot * 8u;
          if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"((uint32_t)(nu * 1024 + 2 * ng * 64)) : "memory");
          const uint8_t* src = lane == 0 ? wsrc : szb + ((size_t)((2 * rp + lane - 1) * G + g0) << 6);
          const uint32_t bytes = lane == 0 ? (uint32_t)nu << 10 : (uint32_t)ng << 6;
          __syncwarp(0x7u);
          asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                       ::"r"(ring_s + slot * (uint32_t)kSlotBytes + dst_off), "l"(src), "r"(bytes), "r"(fb) : "memory");
          wsrc += (size_t)nu << 10;
          ++issued;
          if (++si == geo.SPR) { si = 0; ++rp; }
        }
      }
      if (!live && lane == 0) {
        // a wait gave up: make sure none of this CTA's copies is still in flight before shared memory goes away
        const uint32_t back = issued < (uint32_t)S ? issued : (uint32_t)S;
        for (uint32_t k = issued - back; k < issued; ++k) {
          const uint32_t sl = k & smask, pr = (k >> sshift) & 1u;
          for (unsigned int i = 0; i < c.spin && !mbar_try_wait(full + sl, pr); ++i) __nanosleep(64);
        }
      }
    }
  } else {
    // ================= consumers =================
    const int g = lane >> 2, t = lane & 3;
    const int u = warp;                                // this warp's unit of every stage (both 16-row tiles)
    const uint32_t ring_s = smem_u32(ring), xs_s = smem_u32(xs);
    const uint32_t full_s = smem_u32(full), empty_s = smem_u32(empty);
    const uint32_t w_off = (uint32_t)(u * 1024 + lane * 16);
    uint32_t it = 0, flushes = 0;
    const uint32_t smask = (uint32_t)S - 1u, sshift = (uint32_t)__ffs(S) - 1u;      // S is a power of two
    const unsigned int gen0 = ld_acquire_gpu(p.sync) / (unsigned int)nC;      // barrier rounds completed before this launch
    for (int pi = 0; pi < p.count; ++pi) {
      const MegaPhase ph = p.phases[p.first + pi];
      const Geo geo = make_geo(ph, cta, nC);
      long long* tl = (p.timeline != nullptr && tid == 0) ? p.timeline + ((size_t)pi * nC + cta) * 5 : nullptr;
      if (tl) tl[0] = clock64();
      if (pi > 0) {
        cons_bar();
        if (tid == 0) grid_barrier(c, (unsigned int)nC, (uint32_t)pi);
        cons_bar();
      }
      if (tl) tl[1] = clock64();
      if (geo.sb >= geo.se) continue;               // nothing to do in this phase (tiny weights): skip the staging too
      float inv_scale = 1.f;
      stage_x(ph, p.h, xs, xsum, red_a, red_b, tid, inv_scale);
      if (tl) tl[2] = clock64();
      if (pi + 1 < p.count) {
        // the next phase's norm weights are cold in L2 (read once per token): start fetching them now so that its
        // staging step, which sits on the critical path right after the grid barrier, finds them there
        const MegaPhase* nx = p.phases + p.first + pi + 1;
        if (nx->pro == PRO_NORM) {
          const char* nwp = reinterpret_cast<const char*>(nx->nw);
          for (int i = tid * 128; i < nx->K * 4; i += kCW * 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(nwp + i));
        }
      }
      const unsigned int epoch = gen0 + (unsigned int)pi + 1u;
      const uint32_t sz_off = (uint32_t)(kUnits * 1024 + (u >> geo.g64s) * 64 + 4 * g);   // this lane's scale word of tile 0 in a slot
      long long s = geo.sb;
      while (s < geo.se) {
        const int rp = (int)(s / geo.SPR);
        const int si0 = (int)(s - (long long)rp * geo.SPR);
        const int si1 = (int)min((long long)geo.SPR, si0 + (geo.se - s));
        float f00 = 0.f, f01 = 0.f, f10 = 0.f, f11 = 0.f;      // tile 0 rows g, g + 8; tile 1 rows g, g + 8
        // Hot loop.  Everything is addressed by 32-bit shared-memory offsets computed once per row pair; a stage costs a
        // warp one barrier test, nine shared loads, one arrive, eight (shift + 4 logic + MMA) groups and two folds.
        uint32_t x_addr = xs_s + (uint32_t)(kUnits * si0 + u) * 128u + (uint32_t)t * 32u;     // this lane's 16 activations
        int left = geo.KT - kUnits * si0 - u;              // > 0 while this warp's unit exists in the stage
        for (int si = si0; si < si1; ++si, ++it, x_addr += kUnits * 128u, left -= kUnits) {
          // the ring has a power-of-two number of slots: slot and parity are bit fields of the running stage counter
          const uint32_t slot = it & smask, par = (it >> sshift) & 1u;
          const uint32_t fbar = full_s + slot * 8u;
          bool ok = mbar_test(fbar, par);
          if (!ok) ok = ring_wait(full + slot, par, c, 0x200u | slot);
          const uint32_t sl = ring_s + slot * (uint32_t)kSlotBytes;
          if (ok && left > 0) {
            const uint4 w0 = lds128(sl + w_off), w1 = lds128(sl + w_off + 512u);
            const uint4 xa = lds128(x_addr), xb = lds128(x_addr + 16u);
            const uint32_t s00 = lds32(sl + sz_off), s01 = lds32(sl + sz_off + 32u);
            const uint32_t s10 = lds32(sl + sz_off + kSzSeg), s11 = lds32(sl + sz_off + kSzSeg + 32u);
            __syncwarp();
            if (lane == 0) mbar_arrive_s(empty_s + slot * 8u);   // the unit is in registers: the producer may refill the slot
            unit_fma(w0, xa, xb, s00, s01, f00, f01);
            unit_fma(w1, xa, xb, s10, s11, f10, f11);
          } else {
            __syncwarp();
            if (lane == 0) mbar_arrive_s(empty_s + slot * 8u);
          }
        }
        // ---- this CTA's share of row pair rp is complete ----
        if (tl) tl[3] = clock64();
        float (*rb)[32] = reinterpret_cast<float (*)[32]>(red + (flushes & 1u) * kCW * 32);
        // the four lanes of a row group hold disjoint column quarters
        f00 += __shfl_xor_sync(0xffffffffu, f00, 1); f00 += __shfl_xor_sync(0xffffffffu, f00, 2);
        f01 += __shfl_xor_sync(0xffffffffu, f01, 1); f01 += __shfl_xor_sync(0xffffffffu, f01, 2);
        f10 += __shfl_xor_sync(0xffffffffu, f10, 1); f10 += __shfl_xor_sync(0xffffffffu, f10, 2);
        f11 += __shfl_xor_sync(0xffffffffu, f11, 1); f11 += __shfl_xor_sync(0xffffffffu, f11, 2);
        if (t == 0) { rb[warp][g] = f00; rb[warp][g + 8] = f01; rb[warp][16 + g] = f10; rb[warp][24 + g] = f11; }
        cons_bar();
        if (warp == (int)(flushes % kCW)) finalize_pair(p, ph, geo, c, rb, rp, si0, cta, nC, lane, inv_scale, epoch);
        ++flushes;
        s += si1 - si0;
      }
      if (tl) tl[4] = clock64();
    }
    // Every launch advances the arrival count by one more round (nobody waits for it): the epochs derived from the
    // count stay unique per phase also across launches that contain no barrier.
    if (tid == 0 && !*s_abort) asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" ::"l"(p.sync) : "memory");
  }
  __syncthreads();
}

int g_mega_sms = 0;
int g_mega_slot_cap = 0;
int g_mega_bps = 1;            // CTAs per SM (1 or 2)       // tuning: fewer ring slots than fit (0 = all that fit)
bool g_mega_configured = false;

int mega_sms() {
  if (g_mega_sms == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    g_mega_sms = sms;
  }
  return g_mega_sms;
}

}  // namespace

GRM_API int grm_mega_phase_bytes() { return (int)sizeof(MegaPhase); }

// Tuning knob: cap the number of ring slots per CTA (0 = as many as shared memory holds).
GRM_API void grm_mega_set_slot_cap(int slots) { g_mega_slot_cap = slots; }

// CTAs per SM of the launches that follow (1 or 2); tables sized for one value must not be run with the other.
GRM_API void grm_mega_set_ctas_per_sm(int n) { g_mega_bps = n == 2 ? 2 : 1; }

// CTAs of a launch; 0 when no device is current.
GRM_API int grm_mega_grid() { return mega_sms() * (g_mega_bps == 2 ? 2 : 1); }

// Largest number of CTAs that share one 32-row pair of an [rp * 32][K] weight when `grid` CTAs split it evenly: the
// partial-sum scratch needs (that - 1) slots of 32 floats per row pair.
GRM_API int grm_mega_max_parts(int rp, int K, int grid) {
  if (rp < 1 || K < 64 || grid < 1) return 1;
  const int KT = K / 64, SPR = (KT + kUnits - 1) / kUnits;
  const long long T = (long long)rp * SPR;
  if (T < grid) return SPR;
  int mx = 1;
  for (int r = 0; r < rp; ++r) {
    const int a = cta_of(T, (long long)r * SPR, grid), b = cta_of(T, (long long)r * SPR + SPR - 1, grid);
    mx = b - a + 1 > mx ? b - a + 1 : mx;
  }
  return mx;
}

// Runs phases [first, first + count) of the device-resident table `phases` (MegaPhase records, see ops/mega.py) for one
// activation row.  h: the fp32 residual row read by the PRO_NORM phases.  sync: 4 zeroed uints that live as long as
// the table ([0] barrier arrivals, which only grow: every launch adds count * grid; [2] abort word; zero both again after
// a reported timeout).  parts: partial sum scratch, [max row pairs][pstride][32] {value, epoch} pairs (8 bytes each),
// zero before first use.  max_k: largest K of the table.
// recv / world / rank / ar_rows: tensor-parallel exchange regions ([2][world][ar_rows] {value, epoch} pairs per rank,
// zero before first use) for phases with ar_region >= 0; world <= 1 disables.  Every rank must run the same launch
// sequence.  cooperative = 0 launches without the co-residency guarantee (one CTA per SM fits when nothing else runs on
// the device).  timeline: optional device buffer of count * grid * 5 int64 that receives per-phase SM clock stamps of
// every CTA (see MegaParams), null in normal operation.  Returns -2 on an unsupported shape.
GRM_API int grm_decode_mega(const void* phases, int first, int count, const void* h, void* sync, void* parts, int pstride,
                            int max_k, const void* const* recv, int world, int rank, int ar_rows, unsigned int spin, int cooperative,
                            void* timeline, void* stream) {
  if (!phases || count < 1 || !sync || !parts || pstride < 1 || max_k < 64 || (max_k & 63) || max_k > kMaxK)
    return -2;
  if (world > 8 || (world > 1 && (!recv || rank < 0 || rank >= world || ar_rows < 32))) return -2;
  const int sms = mega_sms();
  if (sms < 1) return (int)cudaErrorInvalidDevice;
  MegaParams p;
  p.phases = (const MegaPhase*)phases; p.first = first; p.count = count; p.h = (const float*)h;
  p.sync = (unsigned int*)sync; p.parts = (uint2*)parts; p.pstride = pstride;
  p.status = grm_status_ptr(); p.spin = spin ? spin : 2000000u;
  p.xs_bytes = (max_k * 2 + 127) & ~127;
  p.xsum_bytes = ((max_k / 64) * 4 + 127) & ~127;
  const int fixed = (p.xs_bytes + p.xsum_bytes + (2 * kCW * 32 + 2 * kCW) * 4 + 2 * kMaxSlots * 8 + 64 + 1023) & ~1023;
  const int bps = g_mega_bps == 2 ? 2 : 1;
  // shared memory of an SM is 228 KB in total, 1 KB of it reserved per resident CTA; one CTA may take 227 KB
  const int avail = (bps == 2 ? (228 * 1024 / 2 - 1024) : 227 * 1024) - fixed;
  p.nslots = avail / kSlotBytes < kMaxSlots ? avail / kSlotBytes : kMaxSlots;
  if (g_mega_slot_cap > 0 && p.nslots > g_mega_slot_cap) p.nslots = g_mega_slot_cap;
  if (p.nslots < 2) return -2;
  while (p.nslots & (p.nslots - 1)) p.nslots &= p.nslots - 1;          // a power of two: slot and parity are bit fields of a counter
  for (int i = 0; i < 8; ++i) p.ar_recv[i] = (world > 1 && i < world) ? (float*)const_cast<void*>(recv[i]) : nullptr;
  p.ar_world = world > 1 ? world : 1; p.ar_rank = world > 1 ? rank : 0; p.ar_rows = ar_rows;
  p.timeline = (long long*)timeline;
  const size_t smem = (size_t)fixed + (size_t)p.nslots * kSlotBytes;
  if (!g_mega_configured) {
    cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_mega_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 228 * 1024 / 2 - 1024);
    if (e != cudaSuccess) return (int)e;
    g_mega_configured = true;
  }
  // the CTAs wait for one another (grid barrier, partial sums): a cooperative launch guarantees co-residency
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(sms * bps)); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = smem; cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative; at[0].val.cooperative = 1;
  cfg.attrs = at; cfg.numAttrs = cooperative ? 1 : 0;
  cudaError_t e = bps == 2 ? cudaLaunchKernelEx(&cfg, decode_mega_kernel<2>, p) : cudaLaunchKernelEx(&cfg, decode_mega_kernel<1>, p);
  if (e != cudaSuccess) return (int)e;
  GRM_LAUNCH_RET();
}
