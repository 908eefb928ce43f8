// flash_prefill_tc: causal attention of a prompt chunk on the 5th-generation tensor cores (head_dim 128).
// Same contract as flash_prefill (attn_prefill.cu): M query rows of ONE sequence at positions q_pos0.. over
// T = q_pos0 + M keys, GQA, optional sliding window; K dense bf16 [T][Hkv*128]; V is consumed TRANSPOSED
// (vt [Hkv*128][ldt], key index contiguous) so both products take K-major operands.
//
// Role in the reference: flash prefill on the matrix unit (flash_fast_impl, src/gemm_fast.cpp:832-1375,
// 17.9 TFLOP/s quoted there).  Design for sm_100a:
//   CTA = 128 query rows of one head, 128 threads (thread = row = TMEM lane), 64-key blocks.
//   S = Q K^T : tcgen05.mma 128x64x128, operands brought by TMA into 128-byte-swizzled shared memory,
//               accumulator in TMEM; each thread reads its row with tcgen05.ld, so the online softmax
//               needs no cross-thread reduction;
//   P (bf16) is written back to shared memory in the same swizzled K-major layout and
//   O += P V    : tcgen05.mma 128x128x64 accumulating in a second TMEM region across all key blocks; a row
//               whose running maximum moved is rescaled in place (tcgen05.ld / st), which is rare after the first
//               few blocks; the accumulator is read once at the end.
//   Software pipeline: S has two TMEM buffers and V two shared-memory buffers, so S(j+1) and PV(j) run on the
//   tensor cores while the CTA computes the softmax of block j+1; K / V tiles are requested a block ahead.
// Two CTAs per SM (96 KB shared memory, 256 TMEM columns each) overlap one CTA's softmax with the other's
// MMAs.  Every mbarrier wait is bounded; on a timeout the CTA records the error, frees its TMEM and returns.
#include "common.cuh"
#include <cuda.h>

namespace {

constexpr int D = 128, BQ = 128, BKV = 64, kThreads = 128;
constexpr int kQBytes = BQ * D * 2, kKBytes = BKV * D * 2, kVBytes = D * BKV * 2, kPBytes = BQ * BKV * 2;
constexpr int kSmem = kQBytes + kKBytes + 2 * kVBytes + kPBytes + 256 + 1024;
constexpr uint32_t kTmemCols = 256;       // S buffer 0: columns [0, 64), O: [64, 192), S buffer 1: [192, 256)

struct TcParams {
  bf16* out; int ld_o;
  const bf16* gate; int ld_g;     // optional [M][Hq*D] gate (output *= sigmoid(gate)); warp-specialised kernel only
  int M, T, Hq, Hkv, q_pos0, window;
  float scale_log2;
  unsigned int* status;
};

// registers -> TMEM: 32 lanes x 32 columns of 32-bit (the mirror of tmem_ld_32x32b_x32)
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
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

__device__ __forceinline__ float ex2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__global__ void __launch_bounds__(kThreads, 2)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                         // 2 boxes of [128 rows][64 dims]
  uint8_t* sK = sQ + kQBytes;                 // 2 boxes of [64 keys][64 dims]
  uint8_t* sV = sK + kKBytes;                 // 2 buffers of [128 dims][64 keys]
  uint8_t* sP = sV + 2 * kVBytes;             // [128 rows][64 keys]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kPBytes);     // 0 Q, 1 K, 2/3 V[0/1], 4/5 S[0/1] done, 6 O done
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // causal: later query blocks have more key blocks; they are launched first so the short ones fill the tail
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;
  const int kvh = h / (p.Hq / p.Hkv);
  const int row = qb * BQ + tid;              // query row of this thread inside the chunk
  const bool row_ok = row < p.M;
  const int q_pos = p.q_pos0 + row;
  const int last_q = p.q_pos0 + min(p.M, (qb + 1) * BQ) - 1;
  const int first_q = p.q_pos0 + qb * BQ;
  const int kb_lo = p.window > 0 ? max(0, first_q - p.window + 1) / BKV : 0;
  const int kb_hi = last_q / BKV;             // inclusive

  if (tid == 0) {
    for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);

  auto load_k = [&](int kb) {
    mbar_expect_tx(&bars[1], kKBytes);
    tma_load_2d(sK, &tmK, &bars[1], kvh * D, kb * BKV);
    tma_load_2d(sK + kKBytes / 2, &tmK, &bars[1], kvh * D + 64, kb * BKV);
  };
  auto load_v = [&](int kb, int buf) {
    mbar_expect_tx(&bars[2 + buf], kVBytes);
    tma_load_2d(sV + buf * kVBytes, &tmV, &bars[2 + buf], kb * BKV, kvh * D);
  };
  if (tid == 0) {
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
    mbar_expect_tx(&bars[0], kQBytes);
    tma_load_2d(sQ, &tmQ, &bars[0], h * D, qb * BQ);
    tma_load_2d(sQ + kQBytes / 2, &tmQ, &bars[0], h * D + 64, qb * BQ);
    load_k(kb_lo);
    load_v(kb_lo, 0);
  }

  float m_run = -INFINITY, l_run = 0.f;
  constexpr uint32_t idesc_s = make_idesc(BQ, BKV, 1, 1);
  constexpr uint32_t idesc_o = make_idesc(BQ, D, 1, 1);
  bool ok = true;
  const int nblk = kb_hi - kb_lo + 1;

  // S(j) = Q K(j)^T into S buffer (j & 1); issued by thread 0 once K(j) has landed
  auto issue_s = [&](int j) -> bool {
    if (!mbar_wait(&bars[1], (uint32_t)j & 1u, p.status, 0x801u)) return false;
    tc_fence_after();
    const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK);
    const uint32_t td = tmem_base + ((j & 1) ? 192u : 0u);
#pragma unroll
    for (int k = 0; k < D / 16; ++k) {
      const uint64_t da = make_sw128_kmajor_desc(qa + (k >> 2) * (kQBytes / 2)) + (uint64_t)((k & 3) * 2);
      const uint64_t db = make_sw128_kmajor_desc(ka + (k >> 2) * (kKBytes / 2)) + (uint64_t)((k & 3) * 2);
      tc_mma_f16(td, da, db, idesc_s, k != 0 ? 1u : 0u);
    }
    tc_commit(&bars[4 + (j & 1)]);
    return true;
  };
  if (tid == 0) {
    if (!mbar_wait(&bars[0], 0u, p.status, 0x800u) || !issue_s(0)) *s_abort = 1;
  }

  // Software pipeline over the key blocks j = 0 .. nblk-1 (kb = kb_lo + j):
  //   top     : S(j) is ready; K(j+1) is requested (the K buffer is free)
  //   softmax : this thread's row of S(j); then PV(j-1) is awaited, V(j+1) requested, O rescaled if needed, P(j) stored
  //   barrier : thread 0 issues S(j+1) and PV(j); both run while the CTA does the softmax of the next block
  for (int j = 0; j < nblk && ok; ++j) {
    const int kb = kb_lo + j, b = j & 1;
    if (!mbar_wait(&bars[4 + b], (uint32_t)(j >> 1) & 1u, p.status, 0x803u)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && j + 1 < nblk) load_k(kb + 1);            // the S(j) MMAs have read K
    // ---- softmax of this thread's row ----
    float sv[BKV];
    {
      const uint32_t ts = t_row + (b ? 192u : 0u);
      uint32_t r[32];
      tmem_ld_32x32b_x32(ts, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) sv[i] = __uint_as_float(r[i]);
      tmem_ld_32x32b_x32(ts + 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) sv[32 + i] = __uint_as_float(r[i]);
    }
    float mx = -INFINITY;
    const int key0 = kb * BKV;
    const bool need_mask = (key0 + BKV - 1 > first_q) || (p.window > 0) || !row_ok;
#pragma unroll
    for (int i = 0; i < BKV; ++i) {
      float sc = sv[i] * p.scale_log2;
      if (need_mask) {
        const int kp = key0 + i;
        const bool vis = row_ok && kp <= q_pos && (p.window <= 0 || kp > q_pos - p.window);
        sc = vis ? sc : -INFINITY;
      }
      sv[i] = sc;
      mx = fmaxf(mx, sc);
    }
    const float m_new = fmaxf(m_run, mx);
    const float alpha = (m_new == -INFINITY) ? 1.f : ex2(m_run - m_new);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    float psum = 0.f;
    uint32_t pk[BKV / 2];
#pragma unroll
    for (int i = 0; i < BKV; i += 2) {
      const float p0 = ex2(sv[i] - m_use), p1 = ex2(sv[i + 1] - m_use);
      psum += p0 + p1;
      pk[i >> 1] = pack_bf16x2(p0, p1);
    }
    m_run = m_new;
    l_run = l_run * alpha + psum;
    // PV(j-1) must have finished before O is rescaled, P is overwritten and its V buffer is refilled
    if (j > 0) {
      if (!mbar_wait(&bars[6], (uint32_t)(j - 1) & 1u, p.status, 0x804u)) { ok = false; break; }
      tc_fence_after();
    }
    if (tid == 0 && j + 1 < nblk) load_v(kb + 1, b ^ 1);
    // O stays in TMEM across blocks; a row whose running maximum moved is rescaled in place.  After the first few
    // blocks of a row this is rare, so the branch is taken per warp only when one of its rows needs it.
    if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + 64 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
        tmem_st_32x32b_x32(t_row + 64 + c * 32, r);
      }
      tmem_st_wait();
    }
    // P -> shared memory, K-major rows of 128 bytes with the 16-byte chunks XOR-swizzled by (row & 7)
    {
      uint8_t* prow = sP + tid * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow + ((c ^ (tid & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      bool good = !*s_abort;
      // S(j+1) first: the next block's softmax waits for it; its TMEM buffer was last read before this barrier
      if (good && j + 1 < nblk) good = issue_s(j + 1);
      if (good) good = mbar_wait(&bars[2 + b], (uint32_t)(j >> 1) & 1u, p.status, 0x802u);
      if (good) {
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + b * kVBytes);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
          tc_mma_f16(tmem_base + 64, make_sw128_kmajor_desc(pa) + (uint64_t)(k * 2), make_sw128_kmajor_desc(va) + (uint64_t)(k * 2), idesc_o,
                     (k != 0 || j != 0) ? 1u : 0u);
        tc_commit(&bars[6]);
      } else {
        *s_abort = 1;
      }
    }
  }
  if (ok) {
    if (!mbar_wait(&bars[6], (uint32_t)(nblk - 1) & 1u, p.status, 0x805u)) ok = false;
    tc_fence_after();
  }

  if (ok) {
    const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
    bf16* dst = p.out + (size_t)row * p.ld_o + (size_t)h * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_row + 64 + c * 32, r);          // warp-wide: every lane takes part, rows beyond M skip the store
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
          v.y = pack_bf16x2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
          v.z = pack_bf16x2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
          v.w = pack_bf16x2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
        }
      }
    }
  }
  if (!ok && tid == 0) {
    // let copies in flight land before the shared memory is handed to another CTA (bounded)
    for (int b = 1; b <= 3; ++b)
      for (int i = 0; i < 200000 && !mbar_try_wait(&bars[b], 0u) && !mbar_try_wait(&bars[b], 1u); ++i) __nanosleep(64);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

// Warp-specialised form of the same kernel: warps 0-3 are the 128 softmax rows, warp 4 owns every TMA request and every
// tcgen05.mma.  The row threads never issue or wait for a copy, and S(j+1) is issued as soon as S(j) has left the K buffer
// -- while the rows are still in the softmax of block j -- instead of after it, so the S product's latency is off the
// critical path.  Hand-overs: bars[4/5] S(j) complete (rows and the MMA warp wait), bars[7] P(j) stored (128 arrivals, the
// MMA warp waits), bars[6] PV(j) complete (rows wait before touching O / P, the MMA warp before refilling V).
// Templated on the head dimension: 128 (two CTAs per SM) or 256 (one CTA per SM: 176 KB of tiles, 384 TMEM columns); an
// optional gate multiplies the output by sigmoid(gate) in the epilogue (gated attention of the hybrid family).
constexpr int kThreadsWs = 160;
template <int DH> struct WsGeom {
  static constexpr int kQB = BQ * DH * 2, kKB = BKV * DH * 2, kVB = DH * BKV * 2;
  static constexpr int kQBox = BQ * 128, kKBox = BKV * 128;            // one 64-dim box of the Q / K tile
  static constexpr int kSmemBytes = kQB + kKB + 2 * kVB + kPBytes + 256 + 1024;
  static constexpr uint32_t kCols = DH == 128 ? 256u : 512u;           // S0 [0, 64), O [64, 64 + DH), S1 [64 + DH, 128 + DH)
  static constexpr uint32_t kS1 = 64u + DH;
};

template <int DH>
__global__ void __launch_bounds__(kThreadsWs, DH == 128 ? 2 : 1)
flash_prefill_tc_ws_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                           const __grid_constant__ CUtensorMap tmV, const TcParams p) {
  using G = WsGeom<DH>;
  constexpr int D = DH;                        // shadows the file-wide 128 inside this kernel
  constexpr int kQBytes = G::kQB, kKBytes = G::kKB, kVBytes = G::kVB;
  constexpr uint32_t kTmemCols = G::kCols;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kQBytes;
  uint8_t* sV = sK + kKBytes;
  uint8_t* sP = sV + 2 * kVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + kPBytes);     // 0 Q, 1 K, 2/3 V[0/1], 4/5 S[0/1] done, 6 PV done, 7 P stored
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qb = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y;
  const int kvh = h / (p.Hq / p.Hkv);
  const int row = qb * BQ + tid;
  const bool row_ok = warp < 4 && row < p.M;
  const int q_pos = p.q_pos0 + row;
  const int last_q = p.q_pos0 + min(p.M, (qb + 1) * BQ) - 1;
  const int first_q = p.q_pos0 + qb * BQ;
  const int kb_lo = p.window > 0 ? max(0, first_q - p.window + 1) / BKV : 0;
  const int kb_hi = last_q / BKV;
  const int nblk = kb_hi - kb_lo + 1;

  if (tid == 0) {
    for (int i = 0; i < 7; ++i) mbar_init(&bars[i], 1);
    mbar_init(&bars[7], 128);
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_holder, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  constexpr uint32_t idesc_s = make_idesc(BQ, BKV, 1, 1);
  constexpr uint32_t idesc_o = make_idesc(BQ, D, 1, 1);

  if (warp == 4) {
    if (lane == 0) {
      auto load_k = [&](int kb) {
        mbar_expect_tx(&bars[1], kKBytes);
#pragma unroll
        for (int bx = 0; bx < D / 64; ++bx) tma_load_2d(sK + bx * G::kKBox, &tmK, &bars[1], kvh * D + 64 * bx, kb * BKV);
      };
      auto load_v = [&](int kb, int buf) {
        mbar_expect_tx(&bars[2 + buf], kVBytes);
        tma_load_2d(sV + buf * kVBytes, &tmV, &bars[2 + buf], kb * BKV, kvh * D);
      };
      auto issue_s = [&](int j) -> bool {
        if (!mbar_wait(&bars[1], (uint32_t)j & 1u, p.status, 0x811u)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK);
        const uint32_t td = tmem_base + ((j & 1) ? G::kS1 : 0u);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t da = make_sw128_kmajor_desc(qa + (k >> 2) * G::kQBox) + (uint64_t)((k & 3) * 2);
          const uint64_t db = make_sw128_kmajor_desc(ka + (k >> 2) * G::kKBox) + (uint64_t)((k & 3) * 2);
          tc_mma_f16(td, da, db, idesc_s, k != 0 ? 1u : 0u);
        }
        tc_commit(&bars[4 + (j & 1)]);
        return true;
      };
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(&bars[0], kQBytes);
#pragma unroll
      for (int bx = 0; bx < D / 64; ++bx) tma_load_2d(sQ + bx * G::kQBox, &tmQ, &bars[0], h * D + 64 * bx, qb * BQ);
      load_k(kb_lo);
      load_v(kb_lo, 0);
      bool good = mbar_wait(&bars[0], 0u, p.status, 0x810u) && issue_s(0);
      for (int j = 0; j < nblk && good; ++j) {
        const int kb = kb_lo + j, b = j & 1;
        // S(j) has left the K buffer: fetch K(j+1) and issue S(j+1) at once.  Its TMEM buffer was last read by the rows'
        // softmax of block j-1, which all of them finished before they reported P(j-1) -- awaited below one round ago.
        good = mbar_wait(&bars[4 + b], (uint32_t)(j >> 1) & 1u, p.status, 0x813u);
        if (!good) break;
        if (j + 1 < nblk) {
          load_k(kb + 1);
          good = issue_s(j + 1);
          if (!good) break;
        }
        // PV(j-1) done: its V buffer can take V(j+1)
        if (j > 0) {
          good = mbar_wait(&bars[6], (uint32_t)(j - 1) & 1u, p.status, 0x814u);
          if (!good) break;
        }
        if (j + 1 < nblk) load_v(kb + 1, b ^ 1);
        good = mbar_wait(&bars[7], (uint32_t)j & 1u, p.status, 0x815u) && mbar_wait(&bars[2 + b], (uint32_t)(j >> 1) & 1u, p.status, 0x812u);
        if (!good) break;
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + b * kVBytes);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)
          tc_mma_f16(tmem_base + 64, make_sw128_kmajor_desc(pa) + (uint64_t)(k * 2), make_sw128_kmajor_desc(va) + (uint64_t)(k * 2), idesc_o,
                     (k != 0 || j != 0) ? 1u : 0u);
        tc_commit(&bars[6]);
      }
      if (!good) {
        *s_abort = 1;
        // let copies in flight land before the shared memory is handed to another CTA (bounded)
        for (int b = 1; b <= 3; ++b)
          for (int i = 0; i < 200000 && !mbar_try_wait(&bars[b], 0u) && !mbar_try_wait(&bars[b], 1u); ++i) __nanosleep(64);
      }
    }
  } else {
    const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      const int kb = kb_lo + j, b = j & 1;
      if (!mbar_wait(&bars[4 + b], (uint32_t)(j >> 1) & 1u, p.status, 0x803u)) { ok = false; break; }
      tc_fence_after();
      float sv[BKV];
      {
        const uint32_t ts = t_row + (b ? G::kS1 : 0u);
        uint32_t r[32];
        tmem_ld_32x32b_x32(ts, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[i] = __uint_as_float(r[i]);
        tmem_ld_32x32b_x32(ts + 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[32 + i] = __uint_as_float(r[i]);
      }
      // The raw scores stay unscaled: the scale is positive, so the maximum commutes with it and the scaling rides in the
      // multiply-add in front of each exp2.  Four independent maxima / sums keep the dependent chains short.
      const int key0 = kb * BKV;
      const bool need_mask = (key0 + BKV - 1 > first_q) || (p.window > 0) || !row_ok;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < BKV; ++i) {
          const int kp = key0 + i;
          const bool vis = row_ok && kp <= q_pos && (p.window <= 0 || kp > q_pos - p.window);
          sv[i] = vis ? sv[i] : -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < BKV; i += 4) {
        mx4[0] = fmaxf(mx4[0], sv[i]); mx4[1] = fmaxf(mx4[1], sv[i + 1]);
        mx4[2] = fmaxf(mx4[2], sv[i + 2]); mx4[3] = fmaxf(mx4[3], sv[i + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      const float m_new = fmaxf(m_run, mx);
      const float alpha = (m_new == -INFINITY) ? 1.f : ex2(m_run - m_new);
      const float m_neg = (m_new == -INFINITY) ? 0.f : -m_new;
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[BKV / 2];
#pragma unroll
      for (int i = 0; i < BKV; i += 4) {
        const float p0 = ex2(fmaf(sv[i], p.scale_log2, m_neg)), p1 = ex2(fmaf(sv[i + 1], p.scale_log2, m_neg));
        const float p2 = ex2(fmaf(sv[i + 2], p.scale_log2, m_neg)), p3 = ex2(fmaf(sv[i + 3], p.scale_log2, m_neg));
        ps4[0] += p0; ps4[1] += p1; ps4[2] += p2; ps4[3] += p3;
        pk[i >> 1] = pack_bf16x2(p0, p1);
        pk[(i >> 1) + 1] = pack_bf16x2(p2, p3);
      }
      m_run = m_new;
      l_run = l_run * alpha + ((ps4[0] + ps4[1]) + (ps4[2] + ps4[3]));
      // PV(j-1) must have finished before O is rescaled and P is overwritten
      if (j > 0) {
        if (!mbar_wait(&bars[6], (uint32_t)(j - 1) & 1u, p.status, 0x804u)) { ok = false; break; }
        tc_fence_after();
      }
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_row + 64 + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x32(t_row + 64 + c * 32, r);
        }
        tmem_st_wait();
      }
      {
        uint8_t* prow = sP + tid * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(prow + ((c ^ (tid & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_before();
      mbar_arrive(&bars[7]);
    }
    if (ok) {
      if (!mbar_wait(&bars[6], (uint32_t)(nblk - 1) & 1u, p.status, 0x805u)) ok = false;
      tc_fence_after();
    }
    if (ok) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      bf16* dst = p.out + (size_t)row * p.ld_o + (size_t)h * D;
      const bf16* gsrc = p.gate ? p.gate + (size_t)row * p.ld_g + (size_t)h * D : nullptr;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + 64 + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[i + e]) * inv;
            if (gsrc) {                                      // gated attention: o *= sigmoid(gate)
              const uint4 gv = *reinterpret_cast<const uint4*>(gsrc + c * 32 + i);
              const float gf[8] = {bf16lo_to_f(gv.x), bf16hi_to_f(gv.x), bf16lo_to_f(gv.y), bf16hi_to_f(gv.y),
                                   bf16lo_to_f(gv.z), bf16hi_to_f(gv.z), bf16lo_to_f(gv.w), bf16hi_to_f(gv.w)};
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] *= 1.f / (1.f + __expf(-gf[e]));
            }
            uint4 v;
            v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
            v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

// v [T][ld] (this kv head block of 128 columns at col0) -> vt [128][ldt]: 32x32 tiles through shared memory
__global__ void __launch_bounds__(256) kv_transpose_kernel(const bf16* __restrict__ v, int ld, bf16* __restrict__ vt, int ldt, int T, int cols) {
  __shared__ bf16 tile[32][33];
  const int t0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const int t = t0 + r, c = c0 + tx;
    tile[r][tx] = (t < T && c < cols) ? v[(size_t)t * ld + c] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int c = c0 + r, t = t0 + tx;
    if (c < cols && t < ldt) vt[(size_t)c * ldt + t] = tile[tx][r];
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}
// 2-D bf16 row-major [rows][cols], box = box_rows x 64 columns, 128-byte swizzle, zero fill outside
int make_map(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -3;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {64u, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

}  // namespace

// vt: scratch bf16 [Hkv*Dh][ldt] with ldt >= T rounded up to 64 (filled here from v).  head_dim 128, or 256 with the
// warp-specialised kernel; gate (optional, [M][Hq*Dh] bf16 with row pitch ld_g): output *= sigmoid(gate), warp-specialised
// kernel only.  Returns -2 for anything else (the caller then takes the warp-MMA kernel).
GRM_API int grm_flash_prefill_tc_gated(const void* q, int ld_q, const void* k, const void* v, int ld_kv, void* vt, int ldt, const void* gate,
                                       int ld_g, void* out, int ld_o, int M, int T, int Hq, int Hkv, int Dh, int q_pos0, int window,
                                       float scale, void* stream) {
  if ((Dh != 128 && Dh != 256) || M < 1 || T < M || Hq % Hkv || (ld_o & 7) || (ldt & 63) || ldt < ((T + 63) / 64) * 64 ||
      (gate && ((ld_g & 7) || ((uintptr_t)gate & 15))))
    return -2;
  static int ws = -1;
  if (ws < 0) {
    const char* ev = getenv("GRIMOIRE_FLASH_WS");
    ws = (ev && ev[0] == '0') ? 0 : 1;
    if (ws && (cudaFuncSetAttribute(flash_prefill_tc_ws_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, WsGeom<128>::kSmemBytes) != cudaSuccess ||
               cudaFuncSetAttribute(flash_prefill_tc_ws_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, WsGeom<256>::kSmemBytes) != cudaSuccess))
      ws = 0;
  }
  if (!ws && (Dh != 128 || gate)) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  kv_transpose_kernel<<<dim3((ldt + 31) / 32, (Hkv * Dh + 31) / 32), 256, 0, st>>>((const bf16*)v, ld_kv, (bf16*)vt, ldt, T, Hkv * Dh);
  CUtensorMap tq, tk, tv;
  int e = make_map(&tq, q, (uint64_t)M, (uint64_t)Hq * Dh, (uint64_t)ld_q, BQ);
  if (e) return e;
  e = make_map(&tk, k, (uint64_t)T, (uint64_t)Hkv * Dh, (uint64_t)ld_kv, BKV);
  if (e) return e;
  e = make_map(&tv, vt, (uint64_t)Hkv * Dh, (uint64_t)ldt, (uint64_t)ldt, (uint32_t)Dh);
  if (e) return e;
  TcParams p;
  p.out = (bf16*)out; p.ld_o = ld_o; p.gate = (const bf16*)gate; p.ld_g = ld_g; p.M = M; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.q_pos0 = q_pos0;
  p.window = window; p.scale_log2 = scale * 1.4426950408889634f; p.status = grm_status_ptr();
  const dim3 grid((M + BQ - 1) / BQ, Hq);
  if (ws) {
    if (Dh == 128) flash_prefill_tc_ws_kernel<128><<<grid, kThreadsWs, WsGeom<128>::kSmemBytes, st>>>(tq, tk, tv, p);
    else flash_prefill_tc_ws_kernel<256><<<grid, kThreadsWs, WsGeom<256>::kSmemBytes, st>>>(tq, tk, tv, p);
    GRM_LAUNCH_RET();
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t ce = cudaFuncSetAttribute(flash_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (ce != cudaSuccess) return (int)ce;
    configured = true;
  }
  flash_prefill_tc_kernel<<<grid, kThreads, kSmem, st>>>(tq, tk, tv, p);
  GRM_LAUNCH_RET();
}

GRM_API int grm_flash_prefill_tc(const void* q, int ld_q, const void* k, const void* v, int ld_kv, void* vt, int ldt, void* out, int ld_o,
                                 int M, int T, int Hq, int Hkv, int Dh, int q_pos0, int window, float scale, void* stream) {
  return grm_flash_prefill_tc_gated(q, ld_q, k, v, ld_kv, vt, ldt, nullptr, 0, out, ld_o, M, T, Hq, Hkv, Dh, q_pos0, window, scale, stream);
}
