// Expert-parallel MoE: token all-to-all dispatch and combine over NVLink peer memory, fused with the
// grouped expert GEMM (moe.cu, MODE 4) and the weighted top-k sum.
//
// Every rank owns E/W experts and a contiguous shard of the step's rows.  One MoE layer is
//
//   route (moe.cu)                                 top-k ids / weights / per-expert counts of MY rows
//   ep_prefix    per-expert offsets inside each owner's region; group descriptors -> owners (peer stores)
//   ep_dispatch  one warp per (row, choice): copies the bf16 activation row straight into the owner's
//                receive region and records where the result has to come back; the last CTA raises a
//                per-source flag on every owner (release at system scope)
//   ep_plan      owner: waits (bounded) for the W source flags, turns the W x E_local group descriptors
//                into 32-row tiles (expert-major, so an expert's weights stay hot in L2)
//   grouped GEMM gate|up + SwiGLU on the received rows, then the down projection whose epilogue stores
//                each fp32 result row into the SOURCE rank's return buffer and bumps its arrival counter
//   ep_combine   source: waits (bounded) for all its rows, h += sum_j w_j * y_j in fixed slot order
//                (+ shared expert), pushes the updated rows to every peer's gather buffer, flags them
//   ep_apply     every rank: waits for the owners' flags and copies the other shards' rows into h
//
// The reference moves expert inputs/outputs through host memory between two cards
// (tp_small_allreduce / tm_* tiered MoE, grimoire.cpp:6499-6679, :13800-14400).  Here each receive
// region is private to one source, so no remote atomics are needed; all epochs and expected counts
// live in device memory and are advanced by the kernels themselves, which keeps the whole layer
// replayable from a CUDA graph.  Every wait is bounded and reports GRM_ERR_FLAG_TIMEOUT.
#include "common.cuh"

namespace {

__device__ __forceinline__ unsigned int ld_acq_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_rel_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool wait_ge(const unsigned int* p, unsigned int want, unsigned int spin) {
  for (unsigned int i = 0; i < spin; ++i) {
    if ((int)(ld_acq_sys(p) - want) >= 0) return true;
    __nanosleep(64);
  }
  return false;
}

// state words (device, per rank): 0 dispatch epoch, 1 plan epoch, 2 expected arrivals, 3 combine epoch,
// 4 apply epoch, 8.. finish counters of the multi-CTA kernels
enum { ST_DISPATCH = 0, ST_PLAN = 1, ST_DONE = 2, ST_COMBINE = 3, ST_APPLY = 4, ST_FIN_DISPATCH = 8, ST_FIN_COMBINE = 9, ST_FIN_APPLY = 10 };

// ---------------------------------------------------------------------------------------------
struct PrefixParams {
  const int* counts;          // [E] rows of this rank per (global) expert
  int* ebase;                 // [E] offset of the expert inside its owner's region for this source
  int* cursors;               // [E] zeroed here, claimed by ep_dispatch
  int* peer_groups[8];        // owner o: [W * E_loc][2] (first row, rows), index src * E_loc + e_loc
  int E, E_loc, W, rank, cap;
};

__global__ void __launch_bounds__(1024) ep_prefix_kernel(const PrefixParams p) {
  __shared__ int excl[1024];
  __shared__ int wsum[32];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  const int c = e < p.E ? p.counts[e] : 0;
  int v = c;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, v, off);
    if (lane >= off) v += n;
  }
  if (lane == 31) wsum[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int w = wsum[lane];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, w, off);
      if (lane >= off) w += n;
    }
    wsum[lane] = w;
  }
  __syncthreads();
  excl[e] = v - c + (warp ? wsum[warp - 1] : 0);
  __syncthreads();
  if (e < p.E) {
    const int o = e / p.E_loc, el = e - o * p.E_loc;
    const int base = excl[e] - excl[o * p.E_loc];
    p.ebase[e] = base;
    p.cursors[e] = 0;
    int2* g = reinterpret_cast<int2*>(p.peer_groups[o]) + (size_t)p.rank * p.E_loc + el;
    *g = make_int2(p.rank * p.cap + base, c);
  }
}

// ---------------------------------------------------------------------------------------------
struct DispatchParams {
  const bf16* x; int ldx;     // this rank's rows [M_loc][H]
  const int* ids; int ld_ids; // [M_loc][k] global expert ids
  const int* ebase; int* cursors;
  bf16* peer_x[8];            // owner o: receive rows [W * cap][H]
  int* peer_rowdst[8];        // owner o: [W * cap] return row on the source
  unsigned int* peer_flags[8];// owner o: [W] dispatch epoch per source
  unsigned int* state;
  int M_loc, k, H, E_loc, W, rank, cap;
};

__global__ void __launch_bounds__(128) ep_dispatch_kernel(const DispatchParams p) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pair = blockIdx.x * 4 + warp;
  if (pair < p.M_loc * p.k) {
    const int m = pair / p.k, j = pair - m * p.k;
    const int e = p.ids[(size_t)m * p.ld_ids + j];
    int r = 0;
    if (lane == 0) r = atomicAdd(&p.cursors[e], 1);
    r = __shfl_sync(0xffffffffu, r, 0);
    const int o = e / p.E_loc;
    const int dst = p.rank * p.cap + p.ebase[e] + r;
    const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)m * p.ldx);
    uint4* out = reinterpret_cast<uint4*>(p.peer_x[o] + (size_t)dst * p.H);
    for (int c = lane; c < p.H / 8; c += 32) out[c] = src[c];
    if (lane == 0) p.peer_rowdst[o][dst] = pair;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(&p.state[ST_FIN_DISPATCH], 1u);
    if (prev == gridDim.x - 1) {
      p.state[ST_FIN_DISPATCH] = 0;
      const unsigned int epoch = p.state[ST_DISPATCH] + 1;
      p.state[ST_DISPATCH] = epoch;
      __threadfence_system();
      for (int o = 0; o < p.W; ++o) st_rel_sys(p.peer_flags[o] + p.rank, epoch);
    }
  }
}

// ---------------------------------------------------------------------------------------------
constexpr int kPlanRows = 32;      // rows per tile: the grouped kernel's tile height (moe.cu: kTileRows)

struct PlanParams {
  const unsigned int* flags;  // [W] (local)
  const int* groups;          // [W * E_loc][2] (local)
  int* tile_expert; int* tile_row0; int* tile_rows; int* tile_src; int* n_tiles;
  unsigned int* state; unsigned int* status;
  int E_loc, W, max_tiles;
  unsigned int spin;
};

__global__ void __launch_bounds__(512) ep_plan_kernel(const PlanParams p) {
  __shared__ int s_fail, s_base, wsum[16];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned int epoch = p.state[ST_PLAN] + 1;
  if (tid == 0) { s_fail = 0; s_base = 0; }
  __syncthreads();
  if (tid < p.W && !wait_ge(p.flags + tid, epoch, p.spin)) {
    s_fail = 1;
    grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x50000u | tid);
  }
  __syncthreads();
  __threadfence_system();
  const int G = p.W * p.E_loc;
  for (int g0 = 0; g0 < G && !s_fail; g0 += 512) {
    const int gi = g0 + tid;
    int el = 0, s = 0, row0 = 0, cnt = 0;
    if (gi < G) {
      el = gi / p.W; s = gi - el * p.W;
      const int2 g = reinterpret_cast<const int2*>(p.groups)[(size_t)s * p.E_loc + el];
      row0 = g.x; cnt = g.y;
    }
    const int nt = (cnt + kPlanRows - 1) / kPlanRows;
    int v = nt;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, v, off);
      if (lane >= off) v += n;
    }
    if (lane == 31) wsum[warp] = v;
    __syncthreads();
    int before = s_base;
    for (int w = 0; w < warp; ++w) before += wsum[w];
    int off = before + v - nt;
    for (int t = 0; t < nt; ++t, ++off) {
      if (off >= p.max_tiles) break;
      p.tile_expert[off] = el; p.tile_row0[off] = row0 + kPlanRows * t; p.tile_rows[off] = min(kPlanRows, cnt - kPlanRows * t);
      p.tile_src[off] = s;
    }
    __syncthreads();
    if (tid == 511) s_base = before + v;
    __syncthreads();
  }
  if (tid == 0) {
    *p.n_tiles = s_fail ? 0 : min(s_base, p.max_tiles);
    p.state[ST_PLAN] = epoch;
  }
}

// ---------------------------------------------------------------------------------------------
struct CombineParams {
  float* h; int ldh;          // this rank's rows of the residual stream [M_loc][H] (in/out)
  const float* y; int ldy;    // return buffer: rows m*k+j (routed), M_loc*k + m (shared expert)
  const float* wts; int ld_w; // [M_loc][k (+1)]
  const unsigned int* done;   // arrivals (rows x column blocks)
  float* peer_gather[8];      // rank o: [2][M_total][H] fp32
  unsigned int* peer_hflags[8];
  unsigned int* state; unsigned int* status;
  int M_loc, k, H, has_shared, nblk, W, rank, row_base, M_total;
  unsigned int spin;
};

__global__ void __launch_bounds__(256) ep_combine_kernel(const CombineParams p) {
  __shared__ int s_fail;
  const int m = blockIdx.x, tid = threadIdx.x;
  const unsigned int want = p.state[ST_DONE] + (unsigned)(p.M_loc * p.k * p.nblk);
  const unsigned int par = p.state[ST_COMBINE] & 1u;
  if (tid == 0) {
    s_fail = 0;
    if (!wait_ge(p.done, want, p.spin)) { s_fail = 1; grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x60000u | (m & 0xffff)); }
  }
  __syncthreads();
  __threadfence_system();
  if (m < p.M_loc && !s_fail) {
    float* hr = p.h + (size_t)m * p.ldh;
    const size_t grow = (size_t)par * p.M_total + p.row_base + m;
    for (int c = tid * 4; c < p.H; c += 256 * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < p.k + p.has_shared; ++j) {
        const size_t yr = j < p.k ? (size_t)m * p.k + j : (size_t)p.M_loc * p.k + m;
        const float w = p.wts[(size_t)m * p.ld_w + j];
        const float4 v = *reinterpret_cast<const float4*>(p.y + yr * p.ldy + c);
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
      }
      float4 o = *reinterpret_cast<const float4*>(hr + c);
      o.x += acc.x; o.y += acc.y; o.z += acc.z; o.w += acc.w;
      *reinterpret_cast<float4*>(hr + c) = o;
      for (int r = 0; r < p.W; ++r)
        if (r != p.rank) *reinterpret_cast<float4*>(p.peer_gather[r] + grow * p.H + c) = o;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const unsigned int prev = atomicAdd(&p.state[ST_FIN_COMBINE], 1u);
    if (prev == gridDim.x - 1) {
      p.state[ST_FIN_COMBINE] = 0;
      p.state[ST_DONE] = want;
      const unsigned int epoch = p.state[ST_COMBINE] + 1;
      p.state[ST_COMBINE] = epoch;
      __threadfence_system();
      for (int r = 0; r < p.W; ++r)
        if (r != p.rank) st_rel_sys(p.peer_hflags[r] + p.rank, epoch);
    }
  }
}

// ---------------------------------------------------------------------------------------------
struct ApplyParams {
  float* h; int ldh;          // all rows [M_total][H]
  const float* gather;        // [2][M_total][H] (local)
  const unsigned int* hflags; // [W] (local)
  unsigned int* state; unsigned int* status;
  int M_total, H, Mq, rank;
  unsigned int spin;
};

__global__ void __launch_bounds__(256) ep_apply_kernel(const ApplyParams p) {
  __shared__ int s_fail;
  const int row = blockIdx.x, tid = threadIdx.x;
  const unsigned int epoch = p.state[ST_APPLY] + 1;
  const unsigned int par = p.state[ST_APPLY] & 1u;
  const int owner = row / p.Mq;
  if (owner != p.rank) {
    if (tid == 0) {
      s_fail = 0;
      if (!wait_ge(p.hflags + owner, epoch, p.spin)) { s_fail = 1; grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x70000u | owner); }
    }
    __syncthreads();
    __threadfence_system();
    if (!s_fail) {
      const float4* src = reinterpret_cast<const float4*>(p.gather + ((size_t)par * p.M_total + row) * p.H);
      float4* dst = reinterpret_cast<float4*>(p.h + (size_t)row * p.ldh);
      for (int c = tid; c < p.H / 4; c += 256) dst[c] = src[c];
    }
  }
  __syncthreads();
  if (tid == 0) {
    const unsigned int prev = atomicAdd(&p.state[ST_FIN_APPLY], 1u);
    if (prev == gridDim.x - 1) { p.state[ST_FIN_APPLY] = 0; p.state[ST_APPLY] = epoch; }
  }
}

template <typename T>
void fill_peers(T* (&dst)[8], void* const* src, int world) {
  for (int i = 0; i < 8; ++i) dst[i] = (src && i < world) ? (T*)src[i] : nullptr;
}

}  // namespace

GRM_API int grm_ep_prefix(const void* counts, void* ebase, void* cursors, void* const* peer_groups, int E, int E_loc, int world,
                          int rank, int cap, void* stream) {
  if (E < 1 || E > 1024 || E_loc * world != E || world < 1 || world > 8) return -2;
  PrefixParams p;
  p.counts = (const int*)counts; p.ebase = (int*)ebase; p.cursors = (int*)cursors; fill_peers(p.peer_groups, peer_groups, world);
  p.E = E; p.E_loc = E_loc; p.W = world; p.rank = rank; p.cap = cap;
  ep_prefix_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}

GRM_API int grm_ep_dispatch(const void* x, int ldx, const void* ids, int ld_ids, const void* ebase, void* cursors, void* const* peer_x,
                            void* const* peer_rowdst, void* const* peer_flags, void* state, int M_loc, int k, int H, int E_loc,
                            int world, int rank, int cap, void* stream) {
  if ((H & 7) || (ldx & 7) || M_loc < 0 || M_loc * k > cap || world < 1 || world > 8) return -2;
  DispatchParams p;
  p.x = (const bf16*)x; p.ldx = ldx; p.ids = (const int*)ids; p.ld_ids = ld_ids; p.ebase = (const int*)ebase; p.cursors = (int*)cursors;
  fill_peers(p.peer_x, peer_x, world); fill_peers(p.peer_rowdst, peer_rowdst, world); fill_peers(p.peer_flags, peer_flags, world);
  p.state = (unsigned int*)state; p.M_loc = M_loc; p.k = k; p.H = H; p.E_loc = E_loc; p.W = world; p.rank = rank; p.cap = cap;
  const int blocks = (M_loc * k + 3) / 4;
  ep_dispatch_kernel<<<blocks < 1 ? 1 : blocks, 128, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}

GRM_API int grm_ep_plan(const void* flags, const void* groups, void* tile_expert, void* tile_row0, void* tile_rows, void* tile_src,
                        void* n_tiles, void* state, int E_loc, int world, int max_tiles, unsigned int spin, void* stream) {
  if (world < 1 || world > 8 || E_loc < 1 || max_tiles < 1) return -2;
  PlanParams p;
  p.flags = (const unsigned int*)flags; p.groups = (const int*)groups; p.tile_expert = (int*)tile_expert; p.tile_row0 = (int*)tile_row0;
  p.tile_rows = (int*)tile_rows; p.tile_src = (int*)tile_src; p.n_tiles = (int*)n_tiles; p.state = (unsigned int*)state;
  p.status = grm_status_ptr(); p.E_loc = E_loc; p.W = world; p.max_tiles = max_tiles; p.spin = spin ? spin : 2000000u;
  ep_plan_kernel<<<1, 512, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}

GRM_API int grm_ep_combine(void* h, int ldh, const void* y, int ldy, const void* wts, int ld_w, const void* done,
                           void* const* peer_gather, void* const* peer_hflags, void* state, int M_loc, int k, int H, int has_shared,
                           int nblk, int world, int rank, int row_base, int M_total, unsigned int spin, void* stream) {
  if ((H & 3) || (ldh & 3) || (ldy & 3) || world < 1 || world > 8 || M_loc < 0) return -2;
  CombineParams p;
  p.h = (float*)h; p.ldh = ldh; p.y = (const float*)y; p.ldy = ldy; p.wts = (const float*)wts; p.ld_w = ld_w;
  p.done = (const unsigned int*)done; fill_peers(p.peer_gather, peer_gather, world); fill_peers(p.peer_hflags, peer_hflags, world);
  p.state = (unsigned int*)state; p.status = grm_status_ptr(); p.M_loc = M_loc; p.k = k; p.H = H; p.has_shared = has_shared;
  p.nblk = nblk; p.W = world; p.rank = rank; p.row_base = row_base; p.M_total = M_total; p.spin = spin ? spin : 2000000u;
  ep_combine_kernel<<<M_loc < 1 ? 1 : M_loc, 256, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}

GRM_API int grm_ep_apply(void* h, int ldh, const void* gather, const void* hflags, void* state, int M_total, int H, int Mq, int rank,
                         unsigned int spin, void* stream) {
  if ((H & 3) || (ldh & 3) || M_total < 1 || Mq < 1) return -2;
  ApplyParams p;
  p.h = (float*)h; p.ldh = ldh; p.gather = (const float*)gather; p.hflags = (const unsigned int*)hflags; p.state = (unsigned int*)state;
  p.status = grm_status_ptr(); p.M_total = M_total; p.H = H; p.Mq = Mq; p.rank = rank; p.spin = spin ? spin : 2000000u;
  ep_apply_kernel<<<M_total, 256, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}

// ---------------------------------------------------------------------------------------------
// Expert-parallel decode (a handful of rows): activations and routing are replicated, every rank runs the chosen
// experts it owns as one-row tiles, and the weighted sum over choices is all-reduced in the combine kernel itself.
// The exchange is the fence-free one of the tensor-parallel decode path: every partial value travels as one 8-byte
// {value, epoch} store into each peer's receive region and the receiver polls the data slot; partials are added in
// rank order, so all ranks hold the same bits.  (The reference's expert parallelism is this scheme with a host
// all-reduce: grimoire.cpp:6263-6366.)
// ---------------------------------------------------------------------------------------------
namespace {

__global__ void ep_decode_prep_kernel(const int* __restrict__ ids, int ld_ids, int M, int k, int e0, int e1, int owns_shared,
                                      int* __restrict__ te, int* __restrict__ nr, int* __restrict__ pos) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx < M * k) {
    const int m = idx / k, j = idx - m * k;
    const int id = ids[(size_t)m * ld_ids + j];
    const bool local = id >= e0 && id < e1;
    te[idx] = local ? id - e0 : 0;
    nr[idx] = local ? 1 : 0;
    pos[(size_t)m * (k + 1) + j] = local ? idx : -1;
  }
  if (idx < M) pos[(size_t)idx * (k + 1) + k] = owns_shared ? M * k + idx : -1;
}

struct CombineArParams {
  float* h; int ldh;
  const float* y; int ldy;
  const int* pos; const float* wts;
  int M, slots, H;
  float* recv[8];            // per rank: {value, epoch} pairs [2 parity][world][cap]
  unsigned int* epochs;      // [blocks], local
  unsigned int* status;
  size_t cap;                // pairs per (parity, source): fixed for the buffer
  int W, rank;
  unsigned int spin;
};

__global__ void __launch_bounds__(256) ep_combine_allreduce_kernel(const CombineArParams p) {
  const int idx = blockIdx.x * 256 + threadIdx.x;
  const unsigned int e = p.epochs[blockIdx.x] + 1u;
  const size_t par = e & 1u;
  if (idx < p.M * p.H) {
    const int row = idx / p.H, c = idx - row * p.H;
    float acc = 0.f;
    for (int j = 0; j < p.slots; ++j) {
      const int ps = p.pos[(size_t)row * p.slots + j];
      if (ps >= 0) acc = fmaf(p.wts[(size_t)row * p.slots + j], p.y[(size_t)ps * p.ldy + c], acc);
    }
    const size_t slot = (par * p.W + p.rank) * p.cap + idx;
    for (int r = 0; r < p.W; ++r) {
      if (r == p.rank) continue;
      uint2* dst = reinterpret_cast<uint2*>(p.recv[r]) + slot;
      asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(acc)), "r"(e) : "memory");
    }
    const uint2* mine = reinterpret_cast<const uint2*>(p.recv[p.rank]);
    float s = 0.f;
    bool ok = true;
    for (int r = 0; r < p.W && ok; ++r) {
      if (r == p.rank) { s += acc; continue; }
      const uint2* src = mine + (par * p.W + r) * p.cap + idx;
      uint32_t vx = 0u, vy = 0u;
      ok = false;
      for (unsigned int i = 0; i < p.spin; ++i) {
        asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(vx), "=r"(vy) : "l"(src) : "memory");
        if (vy == e) { ok = true; break; }
        if (i > 64) __nanosleep(20);
      }
      if (!ok) grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x30000u | (r << 12) | (blockIdx.x & 0xfff));
      s += __uint_as_float(vx);
    }
    if (ok) p.h[(size_t)row * p.ldh + c] += s;
  }
  __syncthreads();
  if (threadIdx.x == 0) p.epochs[blockIdx.x] = e;   // advance even after a timeout so later launches stay aligned
}

}  // namespace

// ids [M][ld_ids] global expert choices -> one-row tiles over this rank's experts [e0, e1): te (local expert or 0), nr (1 if
// the choice is local else 0), pos [M][k + 1] (grouped row m * k + j of a local choice, -1 otherwise; column k = the shared
// expert's row M * k + m on the rank that owns it).
GRM_API int grm_ep_decode_prep(const void* ids, int ld_ids, int M, int k, int e0, int e1, int owns_shared, void* te, void* nr,
                               void* pos, void* stream) {
  if (M < 1 || k < 1) return -2;
  const int n = M * k;
  ep_decode_prep_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>((const int*)ids, ld_ids, M, k, e0, e1, owns_shared, (int*)te,
                                                                          (int*)nr, (int*)pos);
  GRM_LAUNCH_RET();
}

// h[M][ldh] += sum over ranks of (sum_j wts[m][j] * y[pos[m][j]]).  recv: `world` peer-mapped receive regions of
// 2 * world * cap {value, epoch} pairs (zero before first use), cap >= M * H; epochs: ceil(cap / 256) local counters (zero
// before first use).  Every rank issues the same sequence of calls with the same M.  The grid (M * H / 256 CTAs) must be
// resident at once, which holds for the few rows this path is used for (-2 otherwise).
GRM_API int grm_ep_combine_allreduce(void* h, int ldh, const void* y, int ldy, const void* pos, const void* wts, int M, int slots, int H,
                                     void* const* recv, long cap, void* epochs, int world, int rank, unsigned int spin, void* stream) {
  if (M < 1 || world < 1 || world > 8 || rank < 0 || rank >= world || (long)M * H > cap) return -2;
  const int blocks = (M * H + 255) / 256;
  if (blocks > 148 * 4) return -2;
  CombineArParams p;
  p.h = (float*)h; p.ldh = ldh; p.y = (const float*)y; p.ldy = ldy; p.pos = (const int*)pos; p.wts = (const float*)wts;
  p.M = M; p.slots = slots; p.H = H;
  for (int i = 0; i < 8; ++i) p.recv[i] = i < world ? (float*)recv[i] : nullptr;
  p.epochs = (unsigned int*)epochs; p.status = grm_status_ptr(); p.cap = (size_t)cap; p.W = world; p.rank = rank;
  p.spin = spin ? spin : 2000000u;
  ep_combine_allreduce_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}
