// Sequence-parallel glue between the fused tensor-parallel GEMMs of a prefill chunk:
//
//   GEMM (row-parallel, epilogue pushes bf16 partial tiles to the row owner)      gemm_tcgen05.cu, epi 4
//     -> rs_reduce_norm_ag (this file): the owner waits for the W partials of a row's tile, sums them
//        in rank order into its token shard of the fp32 residual stream, applies RMSNorm on the
//        shard and pushes the normalised row into EVERY rank's copy of the activation matrix
//     -> GEMM (column-parallel, producer warp waits per m tile for the pushed rows)   epi 0/3 + ag_cnt
//
// i.e. GEMM -> reduce-scatter and all-gather -> GEMM with the norm / residual work done on M/W rows
// (sequence parallelism), every byte moved by plain peer stores over NVLink and every hand-off a
// counter with release / acquire at system scope.  The reference exchanges these activations through
// host memory (tp_shm_allreduce / tp_pipe_allreduce / wavefront prefill, grimoire.cpp:5671-6366,
// :21584-21703).  All waits are bounded and report GRM_ERR_FLAG_TIMEOUT through the status block.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 8;      // H <= 256 * 4 * 8

struct RsParams {
  float* h;                     // [R][ldh] fp32 token shard of the residual stream (in/out)
  const bf16* recv;             // this rank's receive region [W][R][H] (null: no reduce, e.g. first layer)
  const unsigned int* rs_cnt;   // [R/128][W] arrivals
  unsigned int rs_expect;
  const float* norm_w;          // null: no norm / all-gather (last layer)
  float eps, offset;
  bf16* x_peer[8];              // every rank's activation copy [M][H]
  unsigned int* ag_peer[8];     // every rank's per-m-tile row counters [M/128]
  unsigned int* status;
  int R, H, ldh, W, rank;
  unsigned int spin;
};

__device__ __forceinline__ unsigned int ld_acq(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_rel_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kThreads) rs_reduce_norm_ag_kernel(const RsParams p) {
  __shared__ float sh[32];
  __shared__ int s_fail;
  const int row = blockIdx.x, tid = threadIdx.x;
  const int tile = row >> 7;
  if (tid == 0) s_fail = 0;
  __syncthreads();
  if (p.recv) {
    if (tid < p.W) {
      const unsigned int* c = p.rs_cnt + (size_t)tile * p.W + tid;
      bool ok = false;
      for (unsigned int i = 0; i < p.spin; ++i) {
        if ((int)(ld_acq(c) - p.rs_expect) >= 0) { ok = true; break; }
        __nanosleep(100);
      }
      if (!ok) { s_fail = 1; grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x30000u | (tid << 12) | (tile & 0xfff)); }
    }
    __syncthreads();
    if (s_fail) return;
  }
  float* hr = p.h + (size_t)row * p.ldh;
  const int nvec = p.H >> 2;
  float4 v[kMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = tid + i * kThreads;
    if (c < nvec) {
      float4 a = reinterpret_cast<const float4*>(hr)[c];
      if (p.recv) {
        for (int s = 0; s < p.W; ++s) {     // rank order: every owner adds the same numbers in the same order
          const uint2 d = __ldcg(reinterpret_cast<const uint2*>(p.recv + ((size_t)s * p.R + row) * p.H) + c);
          a.x += bf16lo_to_f(d.x); a.y += bf16hi_to_f(d.x); a.z += bf16lo_to_f(d.y); a.w += bf16hi_to_f(d.y);
        }
        reinterpret_cast<float4*>(hr)[c] = a;
      }
      v[i] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  if (!p.norm_w) return;
  ss = warp_sum(ss);
  if ((tid & 31) == 0) sh[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) tot += sh[w];
  const float r = rsqrtf(tot / (float)p.H + p.eps);
  const size_t grow = (size_t)p.rank * p.R + row;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = tid + i * kThreads;
    if (c < nvec) {
      const float4 g = reinterpret_cast<const float4*>(p.norm_w)[c];
      uint2 o;
      o.x = pack_bf16x2(v[i].x * r * (p.offset + g.x), v[i].y * r * (p.offset + g.y));
      o.y = pack_bf16x2(v[i].z * r * (p.offset + g.z), v[i].w * r * (p.offset + g.w));
      for (int s = 0; s < p.W; ++s) reinterpret_cast<uint2*>(p.x_peer[s] + grow * p.H)[c] = o;   // all-gather push
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.W) red_rel_add(p.ag_peer[tid] + (grow >> 7), 1u);
}

}  // namespace

// One CTA per local row.  recv may be null (no partials to add), norm_w may be null (no norm and no
// all-gather).  x_peer / ag_peer: arrays of `world` peer-mapped pointers.
GRM_API int grm_rs_reduce_norm_ag(void* h, int ldh, const void* recv, const void* rs_cnt, unsigned int rs_expect,
                                  const void* norm_w, float eps, float offset, const void* const* x_peer,
                                  const void* const* ag_peer, int R, int H, int world, int rank, unsigned int spin,
                                  void* stream) {
  if (R < 1 || (R & 127) || (H & 3) || H > kThreads * 4 * kMaxVec || world < 1 || world > 8) return -2;
  RsParams p;
  p.h = (float*)h; p.ldh = ldh; p.recv = (const bf16*)recv; p.rs_cnt = (const unsigned int*)rs_cnt; p.rs_expect = rs_expect;
  p.norm_w = (const float*)norm_w; p.eps = eps; p.offset = offset;
  for (int i = 0; i < 8; ++i) {
    p.x_peer[i] = (x_peer && i < world) ? (bf16*)const_cast<void*>(x_peer[i]) : nullptr;
    p.ag_peer[i] = (ag_peer && i < world) ? (unsigned int*)const_cast<void*>(ag_peer[i]) : nullptr;
  }
  p.status = grm_status_ptr(); p.R = R; p.H = H; p.W = world; p.rank = rank; p.spin = spin ? spin : 2000000u;
  rs_reduce_norm_ag_kernel<<<R, kThreads, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}

// ---------------------------------------------------------------------------------------------
// Context-parallel exchange of a prefill chunk's fresh k | v rows (parallel/cp.py): every rank pushes the rows it projected
// into each peer's receive buffer with plain peer stores, counts its arrival there, waits (bounded) until the rows of all
// ranks have arrived in its own buffer and copies them into its q|k|v matrix.  One launch; the grid is at most one CTA per
// SM so that CTAs waiting for remote rows never keep CTAs that still have rows to push off the machine.
// ---------------------------------------------------------------------------------------------
namespace {

struct CpParams {
  bf16* qkv; int ld, qsz, width, a, b, M;
  bf16* peer_buf[8];            // every rank's receive buffer [2 parity][rows_cap][width]
  unsigned int* peer_cnt[8];    // every rank's arrival counters [source rank], monotonic
  int parity;
  unsigned int target;          // arrivals per source expected after this launch
  int rows_cap, world, rank;
  unsigned int spin;
  unsigned int* status;
};

__global__ void __launch_bounds__(256) cp_push_rows_kernel(const CpParams p) {
  __shared__ int s_fail;
  const int tid = threadIdx.x;
  const int vec = p.width / 8;                                  // 16-byte vectors per row
  if (tid == 0) s_fail = 0;
  for (int row = p.a + blockIdx.x; row < p.b; row += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(p.qkv + (size_t)row * p.ld + p.qsz);
    for (int r = 0; r < p.world; ++r) {
      if (r == p.rank) continue;
      uint4* dst = reinterpret_cast<uint4*>(p.peer_buf[r] + ((size_t)p.parity * p.rows_cap + row) * p.width);
      for (int i = tid; i < vec; i += 256) dst[i] = src[i];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid < p.world && tid != p.rank) red_rel_add(p.peer_cnt[tid] + p.rank, 1u);
  if (tid < p.world && tid != p.rank) {
    const unsigned int* c = p.peer_cnt[p.rank] + tid;
    bool ok = false;
    for (unsigned int i = 0; i < p.spin; ++i) {
      if ((int)(ld_acq(c) - p.target) >= 0) { ok = true; break; }
      __nanosleep(100);
    }
    if (!ok) { s_fail = 1; grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x80000u | ((unsigned int)tid << 12)); }
  }
  __syncthreads();
  if (s_fail) return;
  const bf16* mine = p.peer_buf[p.rank] + (size_t)p.parity * p.rows_cap * p.width;
  for (int row = blockIdx.x; row < p.M; row += gridDim.x) {
    if (row >= p.a && row < p.b) continue;
    const uint4* src = reinterpret_cast<const uint4*>(mine + (size_t)row * p.width);
    uint4* dst = reinterpret_cast<uint4*>(p.qkv + (size_t)row * p.ld + p.qsz);
    for (int i = tid; i < vec; i += 256) dst[i] = __ldcg(src + i);
  }
}

}  // namespace

// Number of CTAs grm_cp_push_rows launches for `rows_local` rows per rank (every rank must use the same value: the
// arrival target counts them).
GRM_API int grm_cp_push_grid(int rows_local) { return rows_local < 128 ? (rows_local < 1 ? 1 : rows_local) : 128; }

// qkv: this rank's [M][ld] bf16 matrix whose rows [a, b) hold fresh k | v columns [qsz, qsz + width); on return (in stream
// order) all M rows do.  peer_buf / peer_cnt: `world` peer-mapped pointers; target: total arrivals per source after this
// launch (the caller adds grm_cp_push_grid(b - a) per exchange).  width and ld * 2 must be multiples of 16 bytes.
GRM_API int grm_cp_push_rows(void* qkv, int ld, int qsz, int width, int a, int b, int M, const void* const* peer_buf,
                             const void* const* peer_cnt, int parity, unsigned int target, int rows_cap, int world, int rank,
                             unsigned int spin, void* stream) {
  if (world < 2 || world > 8 || rank < 0 || rank >= world || (width & 7) || (ld & 7) || (qsz & 7) || a < 0 || b <= a || b > M ||
      M > rows_cap || !peer_buf || !peer_cnt)
    return -2;
  CpParams p;
  p.qkv = (bf16*)qkv; p.ld = ld; p.qsz = qsz; p.width = width; p.a = a; p.b = b; p.M = M;
  for (int i = 0; i < 8; ++i) {
    p.peer_buf[i] = i < world ? (bf16*)const_cast<void*>(peer_buf[i]) : nullptr;
    p.peer_cnt[i] = i < world ? (unsigned int*)const_cast<void*>(peer_cnt[i]) : nullptr;
  }
  p.parity = parity & 1; p.target = target; p.rows_cap = rows_cap; p.world = world; p.rank = rank;
  p.spin = spin ? spin : 20000000u;
  p.status = grm_status_ptr();
  cp_push_rows_kernel<<<grm_cp_push_grid(b - a), 256, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}
