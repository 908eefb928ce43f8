// gemv_w4_tc: Y[1][N] = X[1][K] . W[N][K]^T for int4 (group 128) weights on the tcgen05 tensor cores -- the single-row
// decode projection as a weight STREAM: the CUDA-core kernel (gemv_w4.cu) spends ~2.6 instructions per weight and is
// issue-bound at 0.4-0.65 of the memory rate; here a weight costs ~0.6 instructions (three logic operations per eight
// nibbles plus its share of a tensor-memory store) and the multiply-accumulate runs on the tensor cores.
//
//   weights   row-block records of formats/w4_rowblock.py: 128 rows x 128 k = 8704 contiguous bytes, one bulk copy each
//             into an 8-deep shared-memory ring (producer warp);
//   A operand one thread per weight row reads its 64 bytes, splits the nibbles into 32 words of four unsigned bytes and
//             stores them to TENSOR MEMORY (tcgen05.st 32x32b.x32): A never touches shared memory again, which would
//             otherwise cost more shared-memory bandwidth than the stream has;
//   B operand the activation row, quantised per 128-k group to 15 bits as 128 * hi + lo with int8 hi / lo (two B columns),
//             in shared memory as [k / 16][level][16 bytes].  The no-swizzle K-major core matrix of the MMA is 8 rows x 16
//             bytes = 128 contiguous bytes; with a 32-byte stride between the core matrices along K its rows 0 and 1 are
//             this chunk's hi and lo bytes and rows 2..7 are the following chunks' bytes, which land in accumulator
//             columns nobody reads -- so one row of activations needs 2 bytes of shared memory per k instead of 16;
//   MMA       one thread of the set that unpacked the stage issues tcgen05.mma kind::i8 (M 128, N 16, K 32; A unsigned from
//             tensor memory, B signed from shared memory, int32 results) four times, each K = 32 step into its own
//             accumulator columns (a central MMA thread fed through mbarriers was measured: the two hand-overs per stage
//             cost ~900 cycles a stage even with the MMAs switched off);
//   epilogue  the row's thread reads its two int32 sums back (tcgen05.ld), removes the zero point with the group's
//             activation sum (sum q x - z sum x, exact in int32), scales by (weight scale x activation scale) and adds
//             into its fp32 accumulator.
//
// The grid is persistent (one CTA per SM) and walks the (row block, k group) stages in row-block-major order, an equal
// contiguous share per CTA (stream-K).  A row block shared by several CTAs is finished by the CTA that holds its last
// first stage (that part is the CTA's last piece of work): the others leave their fp32 partial rows in a scratch slot and
// raise a flag; the finisher waits (bounded) and adds the slots in CTA order to its own part, so the result does not
// depend on timing, and no CTA waits for a CTA that may itself be waiting.  Several sets of four row warps
// take the stages in turn, so one set unpacks while the others' tensor-memory stores, MMAs and read-backs are in flight
// (one set's iteration is a chain of ~1200 cycles of latencies; the stream needs a stage every ~350).
//
// Measured (B200, 27B shapes, one row, us per call in a replayed graph; gemv_w4.cu in brackets): qkv 14.5 (7.7), o 14.2
// (6.9), gate_up 29.1 (23.5), down 23.2 (17.7).  Per CTA: ~2 us until the activations are quantised, ~560 cycles per
// stage (470 with the MMAs switched off, i.e. the bulk-copy stream alone runs at ~5.5 TB/s), ~2 us hand-over of shared
// row blocks, and the launch.  What holds the stream: a tcgen05.mma with A in tensor memory takes ~140 cycles whatever N
// is (8 or 16), so four of them per 8.7 KB stage cap a SM at ~15 bytes per cycle = 4.4 TB/s over 148 SMs; with A in
// shared memory instead the unpacked bytes cross shared memory twice more and that pipe saturates at about the same rate.
// So one row of int4 weights is not faster through the tensor cores than through the CUDA cores on this part, and the
// kernel is opt-in (GRIMOIRE_W4_TC=1); it stays because its cost does not grow with the number of activation rows up
// to the MMA's N (an 8-row step would cost the same stream), which the CUDA-core kernel cannot offer.
//
// The reference's int4 row product is src/gemv_decode.cpp:77-347 (fp32 FMA over the checkpoint layout).
#include "common.cuh"

namespace {

constexpr int kRows = 128;
constexpr int kStageBytes = 8704, kWeightBytes = 8192;
constexpr int kSlots = 12;
constexpr int kSets = 4;                       // sets of four row warps; set s takes the stages with index % kSets == s
// Tensor memory: per set two A buffers of 32 columns (the next stage is stored while the previous MMAs still read the
// other one) and one D buffer of 4 x 16 columns: the four K = 32 steps of a stage write four separate accumulators, summed
// by the row's thread.
constexpr int kNCols = 8;                      // MMA N: two columns carry data (hi, lo), the instruction's minimum is 8
constexpr int kACol0 = 0, kDCol0 = 64 * kSets, kDStage = 4 * kNCols;      // per set: A 2 x 32 columns, D 2 x kDStage columns
constexpr int kTmemCols = 512;
constexpr int kRowThreads = kSets * 128;
constexpr int kProducerWarp = 4 * kSets;
constexpr int kMmaWarps = 2;                   // MMA warp m issues the stages of the sets with set % kMmaWarps == m
constexpr int kThreads = kRowThreads + 32 + 32 * kMmaWarps;     // row warps, producer warp, MMA warps
constexpr int kPrepWarps = 4 * kSets;          // warps that quantise the activations (the row warps)
constexpr int kMaxContrib = 8;
constexpr uint32_t kIdesc = (2u << 4) | (0u << 7) | (1u << 10) | ((uint32_t)(kNCols >> 3) << 17) | ((128u >> 4) << 24);

struct TcParams {
  const uint8_t* w;          // [NB][KG][8704]
  const bf16* x;             // [K] (ignored with h)
  const float* h;            // fused RMSNorm prologue: fp32 residual row and norm weight, or null
  const float* nw;
  float eps, offset;
  void* out;
  int n_out;                 // logical output columns (rows of W; SwiGLU: N / 2)
  int K, NB, KG, epi;
  float* partial;            // [NB][kMaxContrib][128]
  unsigned int* flags;       // [NB][kMaxContrib], zero between launches
  unsigned int* status;
  unsigned int spin;
  int dbg;                   // experiment switch (timing only): 1 = no MMA is issued
  unsigned long long* tl;    // optional timeline: 16 words per CTA (clock64 at the marks in the kernel)
};

unsigned long long* g_tc_timeline = nullptr;
int g_tc_dbg = 0;
__device__ __forceinline__ void tl_mark(const TcParams& p, int slot) {
  if (p.tl) p.tl[(size_t)blockIdx.x * 16 + slot] = (unsigned long long)clock64();
}

struct Ctl {
  unsigned int* status;
  unsigned int spin;
  volatile int* abort;
};

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0u;
}
// bounded wait; false after a time-out or once another thread has given up (the kernel then drains without touching
// tensor memory again and returns through its normal exit)
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, const Ctl& c, unsigned int tag) {
  if (mbar_try(bar, parity)) return true;
  for (unsigned int i = 0; i < c.spin; ++i) {
    if (mbar_try(bar, parity)) return true;
    if ((i & 255u) == 255u && *c.abort) return false;
    if (i > 2048u) __nanosleep(64);
  }
  if (!*c.abort) { *c.abort = 1; grm_set_error(c.status, GRM_ERR_MBAR_TIMEOUT, tag); }
  return false;
}
__device__ __forceinline__ void mbar_arrive_local(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void named_bar(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void named_bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_x2(uint32_t taddr, uint32_t& a, uint32_t& b) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(taddr));
}
// D[tmem] (+)= A[tmem] * B[smem], 8-bit integer inputs, int32 accumulate
__device__ __forceinline__ void tc_mma_i8_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// K-major operand without swizzle: core matrices of 8 rows x 16 bytes; lbo = bytes between core matrices along K, sbo =
// bytes between 8-row groups
__device__ __forceinline__ uint64_t make_noswizzle_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ long unit_begin(long cta, long T, long G) { return cta * T / G; }
__device__ __forceinline__ int cta_of_unit(long u, long T, long G) {
  long c = u * G / T;
  while (c + 1 < G && unit_begin(c + 1, T, G) <= u) ++c;
  while (c > 0 && unit_begin(c, T, G) > u) --c;
  return (int)c;
}

__global__ void __launch_bounds__(kThreads, 1) gemv_w4_tc_kernel(const TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int K = p.K, KG = p.KG;
  uint8_t* ring = smem;
  uint8_t* xq = ring + kSlots * kStageBytes;                         // [K / 16][2][16] + 128 bytes the MMA may read past
  float* xscale = reinterpret_cast<float*>(xq + (size_t)K * 2 + 128);
  int* xsum = reinterpret_cast<int*>(xscale + KG);
  float* comb = reinterpret_cast<float*>(xsum + KG);                 // [kSets - 1][128] the other sets' parts -> set 0
  float* red = comb + (kSets - 1) * kRows;                            // [32]
  uint64_t* bars = reinterpret_cast<uint64_t*>((reinterpret_cast<uintptr_t>(red + 32) + 7) & ~(uintptr_t)7);
  uint64_t* raw_full = bars;
  uint64_t* raw_empty = raw_full + kSlots;
  uint64_t* d_full = raw_empty + kSlots;                              // [kSets][2] per D buffer: one phase per use
  uint64_t* x_ready = d_full + 2 * kSets;                                 // the activations are quantised (one arrival per row warp)
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(x_ready + 1);
  int* s_abort = reinterpret_cast<int*>(tmem_holder + 1);
  int* s_flag_ok = s_abort + 1;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long T = (long)p.NB * KG, G = gridDim.x;
  const long u0 = unit_begin(blockIdx.x, T, G), u1 = unit_begin(blockIdx.x + 1, T, G);
  const int n = (int)(u1 - u0);
  Ctl c{p.status, p.spin, s_abort};
  if (tid == 0) tl_mark(p, 0);

  if (tid == 0) {
    for (int i = 0; i < kSlots; ++i) { mbar_init(raw_full + i, 1); mbar_init(raw_empty + i, 4); }
    for (int i = 0; i < 2 * kSets; ++i) mbar_init(d_full + i, 1);
    mbar_init(x_ready, kPrepWarps);
    *s_abort = 0;
    *s_flag_ok = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kProducerWarp) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = *tmem_holder;
  if (tid == 0) tl_mark(p, 1);

  if (warp == kProducerWarp) {
    // ---- producer: one bulk copy per stage, kSlots stages ahead; starts before the activations are ready ----
    if (lane == 0) {
      const uint8_t* src = p.w + (size_t)u0 * kStageBytes;
      tl_mark(p, 8);
      for (int i = 0; i < n; ++i) {
        const int slot = i % kSlots;
        // only two stages are requested while the row warps still load and quantise the activations: a full ring of
        // weight requests ahead of them was measured to triple the latency of those few loads
        if (i == 2 && !wait_bar(smem_u32(x_ready), 0u, c, 0x180u)) break;
        if (i >= kSlots && !wait_bar(smem_u32(raw_empty + slot), ((i / kSlots) - 1) & 1, c, 0x100u | slot)) break;
        mbar_expect_tx(raw_full + slot, kStageBytes);
        bulk_load(ring + (size_t)slot * kStageBytes, src + (size_t)i * kStageBytes, kStageBytes, raw_full + slot);
      }
      tl_mark(p, 9);
    }
  } else if (warp > kProducerWarp) {
    // ---- MMA warps: wait (hardware barrier 5 + set: the set's 128 row threads arrive, this warp syncs) until a stage's A
    // operand is in tensor memory and the set's previous results are read, then one lane issues its four MMAs ----
    const int m = warp - kProducerWarp - 1;
    const uint32_t xq_addr = smem_u32(xq);
    int own_of_set[kSets];
#pragma unroll
    for (int i = 0; i < kSets; ++i) own_of_set[i] = 0;
    for (int i = 0; i < n; ++i) {
      const int set = i % kSets;
      if (set % kMmaWarps != m) continue;
      const int kg = (int)((u0 + i) % KG);
      int own = 0;
#pragma unroll
      for (int q = 0; q < kSets; ++q) if (q == set) { own = own_of_set[q]; own_of_set[q] = own + 1; }
      // two barrier ids per set, by the parity of the set's stage count: the row threads may be one stage ahead of this
      // warp (never two: their next read-back waits for this stage's commit), and each of the two stages needs its own count
      named_bar(5 + 2 * set + (own & 1), 128 + 32);
      if (lane == 0 && !*s_abort) {
        tc_fence_after();
        const uint32_t a_col = kACol0 + 64 * set + 32 * (own & 1), d_col = kDCol0 + kDStage * (2 * set + (own & 1));
        const int nmma = (p.dbg & 1) ? 0 : 4;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          if (ks < nmma) {
            const uint64_t db = make_noswizzle_desc(xq_addr + (uint32_t)kg * 256u + (uint32_t)ks * 64u, 32u, 256u);
            tc_mma_i8_ts(tb + d_col + kNCols * ks, tb + a_col + 8 * ks, db, kIdesc, 0u);
          }
        }
        tc_commit(d_full + 2 * set + (own & 1));
      }
      __syncwarp();
    }
  } else {
    // ---- activations -> two int8 levels per 128-k group (the row warps), optional RMSNorm first ----
    // All of this warp's loads are issued first (each warp owns the groups warp, warp + 16, ...: at most kMaxG of them), so
    // that they travel together instead of one dependent round trip per group.
    constexpr int kMaxG = (20480 / 128 + kPrepWarps - 1) / kPrepWarps;
    const int pw = warp;
    float xv[kMaxG][4];
    if (p.h != nullptr) {
      float4 wn[kMaxG];
#pragma unroll
      for (int g = 0; g < kMaxG; ++g) {
        const int kg = pw + g * kPrepWarps;
        if (kg < KG) {
          const float4 a = *reinterpret_cast<const float4*>(p.h + kg * 128 + 4 * lane);
          xv[g][0] = a.x; xv[g][1] = a.y; xv[g][2] = a.z; xv[g][3] = a.w;
          wn[g] = *reinterpret_cast<const float4*>(p.nw + kg * 128 + 4 * lane);
        } else {
          xv[g][0] = xv[g][1] = xv[g][2] = xv[g][3] = 0.f;
          wn[g] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int g = 0; g < kMaxG; ++g) ss += xv[g][0] * xv[g][0] + xv[g][1] * xv[g][1] + xv[g][2] * xv[g][2] + xv[g][3] * xv[g][3];
      ss = warp_sum(ss);
      if (lane == 0) red[pw] = ss;
      named_bar(1, kRowThreads);
      ss = 0.f;
#pragma unroll
      for (int k = 0; k < kPrepWarps; ++k) ss += red[k];
      const float rnorm = rsqrtf(ss / (float)K + p.eps);
#pragma unroll
      for (int g = 0; g < kMaxG; ++g) {
        xv[g][0] = __bfloat162float(__float2bfloat16(xv[g][0] * rnorm * (p.offset + wn[g].x)));
        xv[g][1] = __bfloat162float(__float2bfloat16(xv[g][1] * rnorm * (p.offset + wn[g].y)));
        xv[g][2] = __bfloat162float(__float2bfloat16(xv[g][2] * rnorm * (p.offset + wn[g].z)));
        xv[g][3] = __bfloat162float(__float2bfloat16(xv[g][3] * rnorm * (p.offset + wn[g].w)));
      }
    } else {
#pragma unroll
      for (int g = 0; g < kMaxG; ++g) {
        const int kg = pw + g * kPrepWarps;
        uint2 raw = make_uint2(0u, 0u);
        if (kg < KG) raw = *reinterpret_cast<const uint2*>(p.x + kg * 128 + 4 * lane);
        xv[g][0] = bf16lo_to_f(raw.x); xv[g][1] = bf16hi_to_f(raw.x); xv[g][2] = bf16lo_to_f(raw.y); xv[g][3] = bf16hi_to_f(raw.y);
      }
    }
#pragma unroll
    for (int g = 0; g < kMaxG; ++g) {
      const int kg = pw + g * kPrepWarps;
      if (kg >= KG) break;
      const int k = kg * 128 + 4 * lane;
      const float (&v)[4] = xv[g];
      float mx = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
      mx = warp_max(mx);
      const float delta = mx > 0.f ? mx / 16256.f : 1.f;
      const float inv = 1.f / delta;
      uint32_t hw = 0u, lw = 0u;
      int qs = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int q = __float2int_rn(v[e] * inv);
        const int hi = (q + 64) >> 7, lo = q - 128 * hi;
        hw |= (uint32_t)(hi & 0xff) << (8 * e);
        lw |= (uint32_t)(lo & 0xff) << (8 * e);
        qs += q;
      }
      uint8_t* dst = xq + (size_t)(k >> 4) * 32 + (k & 15);
      *reinterpret_cast<uint32_t*>(dst) = hw;
      *reinterpret_cast<uint32_t*>(dst + 16) = lw;
      qs = warp_sum_int(qs);
      if (lane == 0) { xsum[kg] = qs; xscale[kg] = delta; }
    }
    if (pw == 0) reinterpret_cast<uint32_t*>(xq + (size_t)K * 2)[lane] = 0u;   // the bytes the MMA reads past the last chunk
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // generic writes -> visible to the tensor core's reads
    named_bar(1, kRowThreads);
    if (lane == 0) mbar_arrive_local(smem_u32(x_ready));
    if (tid == 0) tl_mark(p, 2);

    // ---- row threads: set s = warps 4 s .. 4 s + 3; thread = weight row of the stage.  Per own stage: unpack into the
    // set's free A buffer, read back the previous own stage (its MMAs have had that long to finish; the D buffer is free
    // afterwards), set-wide barrier, then one thread of the set issues this stage's four MMAs. ----
    const int set = warp >> 2, row = tid & 127, quad = warp & 3;
    const uint32_t lane_base = tb + ((uint32_t)(32 * quad) << 16);
    const uint32_t a_col = kACol0 + 64 * set, d_col = kDCol0 + 2 * kDStage * set;
    const int swz = (row >> 1) & 3;
    bool live = true;
    long long t_raw = 0, t_unp = 0, t_st = 0, t_epi = 0, t_issue = 0;      // timeline: cycles per phase (thread 0 only)
    const bool prof = p.tl != nullptr && tid == 0;
    int own = 0;                      // own stages so far: A and D buffer = own & 1, d_full phase = own >> 1
    int i0 = 0;                       // CTA-local index of the segment's first stage
    long u = u0;
    while (u < u1) {
      const int b = (int)(u / KG), kg0 = (int)(u % KG);
      const int segn = (int)min((long)(KG - kg0), u1 - u);
      float acc = 0.f;
      // Two stages of the set are in flight behind the one being unpacked (their MMAs take ~800 cycles from the hand-over
      // to the commit): pend[0] is the older one.  (kg, scale / zero word) of each is kept for its read-back.
      int pend_kg[2] = {-1, -1}, pend_own[2] = {0, 0};
      uint32_t pend_szw[2] = {0u, 0u};
      // read-back of the set's oldest pending stage: four pairs of int32 sums -> fp32
      auto epilogue = [&]() {
        const int po = pend_own[0], pkg = pend_kg[0];
        const uint32_t pend_sz = pend_szw[0];
        pend_kg[0] = pend_kg[1]; pend_own[0] = pend_own[1]; pend_szw[0] = pend_szw[1]; pend_kg[1] = -1;
        bool ok = live && wait_bar(smem_u32(d_full + 2 * set + (po & 1)), (po >> 1) & 1, c, 0x400u | set);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { live = false; return; }
        tc_fence_after();
        uint32_t q0[4], q1[4];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) tmem_ld_x2(lane_base + d_col + kDStage * (po & 1) + kNCols * ks, q0[ks], q1[ks]);
        tmem_ld_wait();
        tc_fence_before();
        const uint32_t r0 = q0[0] + q0[1] + q0[2] + q0[3], r1 = q1[0] + q1[1] + q1[2] + q1[3];
        const int zi = (int)(bf16hi_to_f(pend_sz) - 128.f);
        const int sres = 128 * (int)r0 + (int)r1 - zi * xsum[pkg];
        const float ws = __half2float(__ushort_as_half((unsigned short)(pend_sz & 0xffffu)));
        acc = fmaf((float)sres, ws * xscale[pkg], acc);
      };
      const int first = i0 + ((set - i0) % kSets + kSets) % kSets;
      for (int idx = first; idx < i0 + segn; idx += kSets) {
        const int slot = idx % kSlots, kg = kg0 + (idx - i0);
        long long tc0 = prof ? clock64() : 0;
        bool ok = live && wait_bar(smem_u32(raw_full + slot), (idx / kSlots) & 1, c, 0x500u | slot);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) live = false;
        if (prof) { const long long t = clock64(); t_raw += t - tc0; tc0 = t; }
        uint32_t sz = 0u;
        if (live) {
          const uint8_t* sp = ring + (size_t)slot * kStageBytes;
          const uint4* rp = reinterpret_cast<const uint4*>(sp + row * 64);
          uint4 ch[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) ch[i] = rp[i ^ swz];
          sz = *reinterpret_cast<const uint32_t*>(sp + kWeightBytes + row * 4);
          __syncwarp();
          if (lane == 0) mbar_arrive_local(smem_u32(raw_empty + slot));
          uint32_t a[32];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t wv[4] = {ch[i].x, ch[i].y, ch[i].z, ch[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              a[8 * i + 2 * j] = wv[j] & 0x0f0f0f0fu;
              a[8 * i + 2 * j + 1] = (wv[j] >> 4) & 0x0f0f0f0fu;
            }
          }
          if (prof) { const long long t = clock64(); t_unp += t - tc0; tc0 = t; }
          // the stage two back used the A and D buffers this stage is about to take: read its results first (its MMAs
          // have had a whole iteration to finish)
          if (pend_kg[1] >= 0) epilogue();
          if (prof) { const long long t = clock64(); t_epi += t - tc0; tc0 = t; }
          if (live) {
            tmem_st_x32(lane_base + a_col + 32 * (own & 1), a);
            tmem_st_wait();
            tc_fence_before();
          }
          if (prof) { const long long t = clock64(); t_st += t - tc0; tc0 = t; }
        }
        // the set's stores have landed, the buffers are free: MMA warp, go.  A set that has given up no longer waits for
        // commits, so nothing else would keep it from running ahead of the MMA warp: it then meets the warp at the barrier
        if (live) named_bar_arrive(5 + 2 * set + (own & 1), 128 + 32);
        else named_bar(5 + 2 * set + (own & 1), 128 + 32);
        if (prof) { const long long t = clock64(); t_issue += t - tc0; tc0 = t; }
        // (a set that has given up keeps arriving, so that the MMA warps never wait in vain)
        if (pend_kg[0] < 0) { pend_kg[0] = kg; pend_own[0] = own; pend_szw[0] = sz; }
        else { pend_kg[1] = kg; pend_own[1] = own; pend_szw[1] = sz; }
        ++own;
      }
      while (pend_kg[0] >= 0 && live) epilogue();
      if (!live) { pend_kg[0] = -1; pend_kg[1] = -1; }
      if (tid == 0) tl_mark(p, 4);
      if (prof) {
        unsigned long long* o = p.tl + (size_t)blockIdx.x * 16;
        o[13] = (unsigned long long)t_raw; o[14] = (unsigned long long)t_unp; o[15] = (unsigned long long)t_issue;
        o[7] = (unsigned long long)t_st; o[3] = (unsigned long long)t_epi;
      }
      // ---- the sets' parts of this segment, then the segment's result ----
      if (set > 0) comb[(set - 1) * kRows + row] = acc;
      named_bar(2, kRowThreads);
      if (set == 0) {
#pragma unroll
        for (int s2 = 0; s2 < kSets - 1; ++s2) acc += comb[s2 * kRows + row];
      }
      named_bar(3, kRowThreads);
      if (set == 0) {
        const bool whole = segn == KG;
        float total = acc;
        bool write = true;
        if (!whole) {
          const long fu = (long)b * KG;
          const int c_first = cta_of_unit(fu, T, G), c_last = cta_of_unit(fu + KG - 1, T, G);
          // The finisher is the FIRST CTA of the block: the block's head is that CTA's last segment, and what it waits for
          // are the later CTAs' first (or only) segments, which they reach without waiting for anybody -- no chain of
          // waits across the grid.
          const int ci = (int)blockIdx.x - c_first - 1;
          if ((int)blockIdx.x != c_first) {
            p.partial[((size_t)b * kMaxContrib + ci) * kRows + row] = acc;
            __threadfence();
            named_bar(4, 128);
            if (row == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.flags + (size_t)b * kMaxContrib + ci), "r"(1u) : "memory");
            write = false;
          } else {
            const int others = c_last - c_first;
            for (int cc = 0; cc < others; ++cc) {
              if (row == 0) {
                const unsigned int* f = p.flags + (size_t)b * kMaxContrib + cc;
                bool got = false;
                if (!*s_abort) {
                  for (unsigned int it = 0; it < p.spin; ++it) {
                    unsigned int fv;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(fv) : "l"(f) : "memory");
                    if (fv != 0u) { got = true; break; }
                    if (it > 64u) __nanosleep(32);
                  }
                  if (!got && !*s_abort) { *s_abort = 1; grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x700u | (unsigned int)cc); }
                }
                if (!got) *s_flag_ok = 0;
              }
              named_bar(4, 128);
              if (*s_flag_ok) total += __ldcg(p.partial + ((size_t)b * kMaxContrib + cc) * kRows + row);
            }
            named_bar(4, 128);
            if (row == 0) {
              for (int cc = 0; cc < others; ++cc) p.flags[(size_t)b * kMaxContrib + cc] = 0u;     // ready for the next launch
            }
            write = *s_flag_ok != 0;
          }
        }
        // epilogue of the row
        if (p.epi == 3) {
          const float up = __shfl_down_sync(0xffffffffu, total, 16);
          const int col = b * 64 + (row >> 5) * 16 + lane;
          if (write && lane < 16 && col < p.n_out) reinterpret_cast<bf16*>(p.out)[col] = __float2bfloat16(silu_f(total) * up);
        } else if (write) {
          const int col = b * kRows + row;
          if (col < p.n_out) {
            if (p.epi == 0) reinterpret_cast<bf16*>(p.out)[col] = __float2bfloat16(total);
            else if (p.epi == 1) reinterpret_cast<float*>(p.out)[col] = total;
            else reinterpret_cast<float*>(p.out)[col] += total;
          }
        }
      }
      if (tid == 0) tl_mark(p, 5);
      u += segn;
      i0 += segn;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0) tl_mark(p, 6);
  if (warp == kProducerWarp) {
    tc_fence_after();
    tmem_dealloc(tb, kTmemCols);
  }
}

}  // namespace

// Shared memory of one CTA for a given K.
static size_t tc_smem_bytes(int K) {
  const int KG = K / 128;
  return (size_t)kSlots * kStageBytes + (size_t)K * 2 + 128 + (size_t)KG * 8 + (kSets - 1) * kRows * 4 + 128 + 8 + (2 * kSlots + 2 * kSets + 1) * 8 + 32;
}

// Debug aid: while set, every launch writes 16 clock64 marks per CTA (0 entry, 1 after set-up, 2 activations ready, 3 first
// stage landed, 4 / 5 end of the last segment's stages / of its hand-over, 6 exit; 8 / 9 producer, 10-12 MMA thread).
GRM_API void grm_gemv_w4_tc_set_timeline(void* buf) { g_tc_timeline = (unsigned long long*)buf; }
GRM_API void grm_gemv_w4_tc_set_debug(int bits) { g_tc_dbg = bits; }

// Scratch the caller provides: floats of partial rows and flag words (zeroed once; the kernel leaves them zero).
GRM_API long grm_gemv_w4_tc_scratch_floats(int N) { return (long)((N + kRows - 1) / kRows) * kMaxContrib * kRows; }
GRM_API long grm_gemv_w4_tc_scratch_flags(int N) { return (long)((N + kRows - 1) / kRows) * kMaxContrib; }

// One activation row.  w: row-block records (formats/w4_rowblock.py) of an int4 group-128 weight with N rows (padded to 128
// in the records) and K columns, K % 128 == 0, K <= 20480.  epi: 0 bf16, 1 f32, 2 add_f32, 3 swiglu (gate / up rows
// interleaved per 16; out has N / 2 columns).  h != null: the activations are RMSNorm(h) with weight nw (fp32 [K]).
// Returns -2 on an unsupported shape.
GRM_API int grm_gemv_w4_tc(const void* w, const void* x, const void* h, const void* nw, float eps, float offset, void* out, int N,
                           int K, int epi, void* partial, void* flags, unsigned int spin, void* stream) {
  if (N < 1 || (K % 128) || K < 128 || K > 20480 || epi < 0 || epi > 3 || !partial || !flags || (!h && (!x || ((uintptr_t)x & 7))) ||
      (h && (!nw || ((uintptr_t)h & 15) || ((uintptr_t)nw & 15))) || ((uintptr_t)w & 15) || (epi == 3 && (N & 31)))
    return -2;
  static int sms = 0;
  static bool configured = false;
  if (!configured) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaError_t e = cudaFuncSetAttribute(gemv_w4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tc_smem_bytes(20480));
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  TcParams p;
  p.w = (const uint8_t*)w; p.x = (const bf16*)x; p.h = (const float*)h; p.nw = (const float*)nw; p.eps = eps; p.offset = offset;
  p.out = out; p.n_out = epi == 3 ? N / 2 : N; p.K = K; p.NB = (N + kRows - 1) / kRows; p.KG = K / 128; p.epi = epi;
  p.partial = (float*)partial; p.flags = (unsigned int*)flags; p.status = grm_status_ptr();
  p.spin = spin ? spin : 2000000u;
  p.tl = g_tc_timeline; p.dbg = g_tc_dbg;
  const long T = (long)p.NB * p.KG;
  // contributors of one row block: its KG stages over CTAs of T / grid (or one more) stages each; small problems use fewer
  // CTAs so that a block never has more than kMaxContrib of them
  const long per_min = (p.KG + kMaxContrib - 3) / (kMaxContrib - 2);
  long grid_l = T / per_min;
  if (grid_l > sms) grid_l = sms;
  if (grid_l < 1) grid_l = 1;
  const int grid = (int)grid_l;
  const long per = T / grid;
  if (per < 1 || p.KG / per + 2 > kMaxContrib) return -2;
  gemv_w4_tc_kernel<<<grid, kThreads, tc_smem_bytes(K), (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}
