// gemm_tcgen05: C[M][N] = A[M][K] . B[N][K]^T for the compute-bound (prefill / large verify) shapes.
// bf16 operands, both K-major; fp32 accumulation in TMEM on the 5th-generation tensor cores.
//
// Role in the reference: gemm_bf16_vnni / launch_gemm_fast(+_residual,+_swiglu)
// (src/gemm_fast.cpp:138-720) and the oneDNN prompt GEMMs (src/onednn_gemm.cpp).  Design here:
//
//   * persistent kernel, one CTA per SM, tiles of 128 x BN (BN = 256 or 128) walked m-fastest so
//     the 148 resident CTAs share a handful of B (weight) panels through the 126 MB L2 while A
//     stays L2-resident;
//   * warp-specialised: warp 0 = TMA producer (one elected lane issues cp.async.bulk.tensor for
//     the A and B k-slabs, 128-byte swizzle, no multicast), warp 1 = MMA issuer (one elected lane
//     issues tcgen05.mma kind::f16 128xBNx16, 4 per 64-wide k slab, and tcgen05.commit to release
//     the stage), warps 2-5 = epilogue (tcgen05.ld 32 lanes x 32 columns -> registers -> global);
//   * a ring of kStages shared-memory stages between producer and MMA, and two TMEM accumulator
//     buffers (2 x BN columns of the 512) between MMA and epilogue so tile i+1's main loop runs
//     under tile i's epilogue;
//   * epilogues: bf16 store, fp32 store, fp32 accumulate (residual stream h += y), SwiGLU over the
//     gate/up row interleave used by the int4 layout (16 gate rows then 16 up rows), and -- for
//     tensor parallelism -- a reduce-scatter push of bf16 partial tiles into the owning rank's
//     receive buffer (peer stores over NVLink; see tp_fused.cu for the consumer side);
//   * every mbarrier wait is bounded; a timeout raises the CTA's abort flag, all roles drain, the
//     producer waits (bounded) for TMA copies still in flight, TMEM is freed, the kernel returns
//     and the host finds GRM_ERR_MBAR_TIMEOUT in the status block.
#include <cuda.h>
#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int kThreads = 192;          // 6 warps
constexpr int kEpiWarps = 4;

enum GemmEpi : int { G_BF16 = 0, G_F32 = 1, G_ADD_F32 = 2, G_SWIGLU = 3, G_RS_PUSH = 4 };

struct GemmParams {
  int M, N, K;
  void* out; int ldo;
  unsigned int* status;
  // reduce-scatter push (G_RS_PUSH): rows [r*rows_per_rank, (r+1)*rows_per_rank) of the output
  // belong to rank r; this rank's bf16 partial of those rows is stored into rank r's buffer
  // peer_out[r] at slot `my_rank`: peer_out[r] + ((my_rank * rows_per_rank + local_row) * ldo + n)
  void* peer_out[8];
  int world, my_rank, rows_per_rank;
  // tile arrival counters of the reduce-scatter: after a tile is stored into rank r's buffer, the
  // CTA adds 1 (release, system scope) to peer_cnt[r][(local m tile) * world + my_rank]; the
  // consumer waits for epoch * (N / BN) arrivals per (m tile, source)
  unsigned int* peer_cnt[8];
  // all-gather wait (consumer side of a fused all-gather -> GEMM): before the A rows of m tile t are
  // loaded, the producer warp waits until ag_cnt[t] >= ag_expect (rows pushed by their owners into
  // this rank's own copy of A); null disables the wait
  const unsigned int* ag_cnt;
  unsigned int ag_expect;
  unsigned int spin;
  int vec_ok;   // output base and row pitch are 16-byte aligned: the epilogue may use 128-bit stores
};

__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <int BN>
struct SmemLayout {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // + barriers + alignment slack
};

template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using L = SmemLayout<BN>;
  constexpr int kStages = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty = full + kStages;
  uint64_t* tfull = empty + kStages;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* s_abort = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull[a], 1); mbar_init(&tempty[a], kEpiWarps); }
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------------------
    if (elect_one()) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t stage = 0, phase = 0;
      uint32_t armed = 0, armed_par = 0;   // bit s: full[s] armed at least once / parity of its last arming
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m_blk = t % num_m, n_blk = t / num_m;
        if (p.ag_cnt) {
          // rows of this m tile were written by their owner ranks over NVLink (generic proxy); once
          // the count is seen with acquire semantics, order the async-proxy (TMA) reads after it
          bool seen = false;
          for (unsigned int i = 0; i < p.spin; ++i) {
            if ((int)(ld_acquire_sys_u32(p.ag_cnt + m_blk) - p.ag_expect) >= 0) { seen = true; break; }
            __nanosleep(64);
          }
          if (!seen) { grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x20000u | (unsigned)m_blk); ok = false; break; }
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (*s_abort || !mbar_wait(&empty[stage], phase ^ 1, p.status, 0x100u | stage)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::kStageBytes;
          mbar_expect_tx(&full[stage], L::kStageBytes);
          tma_load_2d(sa, &tmA, &full[stage], kb * BK, m_blk * BM);
          tma_load_2d(sa + L::kABytes, &tmB, &full[stage], kb * BK, n_blk * BN);
          armed |= 1u << stage;
          armed_par = (armed_par & ~(1u << stage)) | (phase << stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        *s_abort = 1;
        // let copies in flight land before the CTA's shared memory is handed to another CTA
        for (int s = 0; s < kStages; ++s)
          if (armed & (1u << s)) {
            for (int i = 0; i < 200000 && !mbar_try_wait(&full[s], (armed_par >> s) & 1u); ++i) __nanosleep(64);
          }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer ---------------------------------------------
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc(BM, BN, 1, 1);
      uint32_t stage = 0, phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (*s_abort || !mbar_wait(&tempty[acc], acc_phase ^ 1, p.status, 0x200u | acc)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (*s_abort || !mbar_wait(&full[stage], phase, p.status, 0x300u | stage)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint64_t da = make_sw128_kmajor_desc(sa);
          const uint64_t db = make_sw128_kmajor_desc(sa + L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // advancing 16 bf16 = 32 bytes along K inside the swizzle row: +2 in the >>4 address field
            tc_mma_f16(tmem_d, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(&empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (ok) tc_commit(&tfull[acc]);
      }
      if (!ok) *s_abort = 1;
    }
  } else {
    // ------------------------------- epilogue warps 2..5 -------------------------------------
    const int q = warp & 3;                 // TMEM lane quarter this warp may touch
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      const int m_blk = t % num_m, n_blk = t / num_m;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (*s_abort || !mbar_wait(&tfull[acc], acc_phase, p.status, 0x400u | acc)) { ok = false; break; }
      tc_fence_after();
      const int row = m_blk * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col = n_blk * BN + c * 32;
        if (!row_ok || col >= p.N) continue;
        if (EPI == G_BF16 || EPI == G_RS_PUSH) {
          bf16* dst;
          if (EPI == G_RS_PUSH) {
            const int owner = row / p.rows_per_rank, lrow = row % p.rows_per_rank;
            dst = reinterpret_cast<bf16*>(p.peer_out[owner]) + ((size_t)p.my_rank * p.rows_per_rank + lrow) * p.ldo + col;
          } else {
            dst = reinterpret_cast<bf16*>(p.out) + (size_t)row * p.ldo + col;
          }
          if (col + 32 <= p.N && p.vec_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              reinterpret_cast<uint4*>(dst)[v] = o;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.N) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
          }
        } else if (EPI == G_F32 || EPI == G_ADD_F32) {
          float* dst = reinterpret_cast<float*>(p.out) + (size_t)row * p.ldo + col;
          if (col + 32 <= p.N && p.vec_ok) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float4 o = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]), __uint_as_float(r[4 * v + 2]),
                                     __uint_as_float(r[4 * v + 3]));
              if (EPI == G_ADD_F32) {
                const float4 h = reinterpret_cast<const float4*>(dst)[v];
                o.x += h.x; o.y += h.y; o.z += h.z; o.w += h.w;
              }
              reinterpret_cast<float4*>(dst)[v] = o;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (col + i < p.N) {
                const float a = __uint_as_float(r[i]);
                dst[i] = (EPI == G_ADD_F32) ? dst[i] + a : a;
              }
          }
        } else {  // G_SWIGLU: columns [0,16) of the chunk = gate, [16,32) = up -> 16 outputs
          bf16* dst = reinterpret_cast<bf16*>(p.out) + (size_t)row * p.ldo + (col >> 1);
          uint32_t o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float g0 = __uint_as_float(r[2 * i]), g1 = __uint_as_float(r[2 * i + 1]);
            const float u0 = __uint_as_float(r[16 + 2 * i]), u1 = __uint_as_float(r[16 + 2 * i + 1]);
            o[i] = pack_bf16x2(silu_f(g0) * u0, silu_f(g1) * u1);
          }
          reinterpret_cast<uint4*>(dst)[0] = make_uint4(o[0], o[1], o[2], o[3]);
          reinterpret_cast<uint4*>(dst)[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
      if (EPI == G_RS_PUSH) {
        // the 32 rows this warp stored belong to one owner (rows_per_rank is a multiple of 128):
        // publish them, then count one arrival per warp quarter (4 per tile)
        __threadfence_system();
        __syncwarp();
        if (lane == 0 && m_blk * BM + q * 32 < p.M) {
          const int r0 = m_blk * BM + q * 32;
          const int owner = r0 / p.rows_per_rank, ltile = (r0 % p.rows_per_rank) / BM;
          red_release_sys_add(p.peer_cnt[owner] + (size_t)ltile * p.world + p.my_rank, 1u);
        }
      }
    }
    if (!ok) *s_abort = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// --------------------------------------------------------------------------------------------
// host side
// --------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
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

// 2-D bf16 row-major [rows][cols] (ld elements between rows), box = box_rows x 64, 128-byte swizzle.
int make_tmap_bf16(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -3;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return -2;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

template <int BN, int EPI>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int sms, cudaStream_t st) {
  using L = SmemLayout<BN>;
  auto kfn = gemm_tcgen05_kernel<BN, EPI>;
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  const int num_tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = num_tiles < sms ? num_tiles : sms;
  kfn<<<grid, kThreads, L::kTotal, st>>>(ta, tb, p);
  GRM_LAUNCH_RET();
}

template <int BN>
int launch_epi(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int epi, int sms, cudaStream_t st) {
  switch (epi) {
    case G_BF16: return launch<BN, G_BF16>(ta, tb, p, sms, st);
    case G_F32: return launch<BN, G_F32>(ta, tb, p, sms, st);
    case G_ADD_F32: return launch<BN, G_ADD_F32>(ta, tb, p, sms, st);
    case G_SWIGLU: return launch<BN, G_SWIGLU>(ta, tb, p, sms, st);
    case G_RS_PUSH: return launch<BN, G_RS_PUSH>(ta, tb, p, sms, st);
    default: return -1;
  }
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

// A: bf16 [M][lda], B: bf16 [N][ldb] (both K contiguous).  epi: 0 bf16 out, 1 fp32 out, 2 fp32 +=,
// 3 SwiGLU (B rows interleaved 16 gate / 16 up; out bf16 [M][N/2]), 4 reduce-scatter push (peer_out
// = array of `world` device pointers, rows_per_rank = M / world).  K % 8 == 0; K tails and M/N tails
// are zero-filled by TMA.  bn: 0 = auto, else 128 or 256.  max_ctas: 0 = one per SM.
static int gemm_bf16_impl(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K, int epi,
                          int bn, int max_ctas, const void* const* peer_out, const void* const* peer_cnt, int world, int my_rank,
                          const void* ag_cnt, unsigned int ag_expect, void* stream) {
  if (M < 1 || N < 1 || K < 8 || (K & 7)) return -2;
  if (epi == G_SWIGLU && (N & 31)) return -2;
  if (epi == G_RS_PUSH && (!peer_out || !peer_cnt || world < 1 || world > 8 || (M % (world * BM)))) return -2;
  if (bn == 0) bn = (N >= 2048 && (N % 256 == 0 || N > 8192)) ? 256 : 128;
  if (bn != 128 && bn != 256) return -2;
  CUtensorMap ta, tb;
  int e = make_tmap_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM);
  if (e) return e;
  e = make_tmap_bf16(&tb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)bn);
  if (e) return e;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.out = out; p.ldo = ldo; p.status = grm_status_ptr();
  p.world = world; p.my_rank = my_rank; p.rows_per_rank = world > 0 ? M / world : M;
  for (int i = 0; i < 8; ++i) {
    p.peer_out[i] = (peer_out && i < world) ? const_cast<void*>(peer_out[i]) : nullptr;
    p.peer_cnt[i] = (peer_cnt && i < world) ? (unsigned int*)const_cast<void*>(peer_cnt[i]) : nullptr;
  }
  p.ag_cnt = (const unsigned int*)ag_cnt; p.ag_expect = ag_expect; p.spin = 4000000u;
  {
    const size_t esz = (epi == G_F32 || epi == G_ADD_F32) ? 4 : 2;
    bool ok = (reinterpret_cast<uintptr_t>(out) % 16 == 0) && (((size_t)ldo * esz) % 16 == 0);
    for (int i = 0; i < 8 && ok; ++i) if (p.peer_out[i] && reinterpret_cast<uintptr_t>(p.peer_out[i]) % 16) ok = false;
    p.vec_ok = ok ? 1 : 0;
  }
  int sms = sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  cudaStream_t st = (cudaStream_t)stream;
  return bn == 256 ? launch_epi<256>(ta, tb, p, epi, sms, st) : launch_epi<128>(ta, tb, p, epi, sms, st);
}

GRM_API int grm_gemm_bf16(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K, int epi,
                          int bn, int max_ctas, const void* const* peer_out, int world, int my_rank, void* stream) {
  if (epi == G_RS_PUSH) return -1;   // use grm_gemm_bf16_tp
  return gemm_bf16_impl(A, lda, B, ldb, out, ldo, M, N, K, epi, bn, max_ctas, peer_out, nullptr, world, my_rank, nullptr, 0u, stream);
}

// Tensor-parallel variants.  epi 4 (reduce-scatter push): bf16 partial tiles go to the owner rank's
// buffer peer_out[r] (slot my_rank; [world][M/world][ldo]) and every stored 32-row slab adds 1 to
// peer_cnt[r][(local m tile)*world + my_rank], so a complete (m tile, source) pair reads
// 4 * ceil(N/BN) per launch.  ag_cnt != null (all-gather wait): rows of A are pushed into this rank's
// copy by their owners; m tile t is loaded once ag_cnt[t] >= ag_expect.  M must be a multiple of
// world*128 for epi 4.  The block-column count this launch uses is returned through n_tiles_out.
GRM_API int grm_gemm_bf16_tp(const void* A, int lda, const void* B, int ldb, void* out, int ldo, int M, int N, int K, int epi,
                             int bn, const void* const* peer_out, const void* const* peer_cnt, int world, int my_rank,
                             const void* ag_cnt, unsigned int ag_expect, int* n_tiles_out, void* stream) {
  int use_bn = bn ? bn : ((N >= 2048 && (N % 256 == 0 || N > 8192)) ? 256 : 128);
  if (n_tiles_out) *n_tiles_out = (N + use_bn - 1) / use_bn;
  return gemm_bf16_impl(A, lda, B, ldb, out, ldo, M, N, K, epi, use_bn, 0, peer_out, peer_cnt, world, my_rank, ag_cnt, ag_expect, stream);
}
