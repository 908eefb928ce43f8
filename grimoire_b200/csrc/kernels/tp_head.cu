// tp_head_pick: the greedy token of a vocabulary-split lm_head.
//
// Under tensor parallelism every rank holds the lm_head rows [v0, v0 + vn) and computes only those logits.  One kernel
// then (1) finds the best (value, index) of its slice per row -- highest value, lowest index on a tie, the rule of the
// whole-vocabulary arg-max (misc.cu) --, (2) stores the candidate into every peer's receive slots over NVLink as two
// self-validating 8-byte words {value bits, epoch} and {global index, epoch}, (3) polls its own slots (bounded) until the
// W - 1 peer candidates of this epoch are there and (4) takes the same decision on every rank.  The reference does the
// same exchange through sockets on the host (tp_head_pick_at, src/grimoire.cpp:5421-5449): best value, lowest index on a
// tie, an index of INT_MAX (no candidate: all logits -inf / NaN) stays INT_MAX.
//
// The epoch is a per-row counter in device memory advanced by the kernel itself, so a captured graph can replay the
// launch; slots are double-buffered by epoch parity (a rank can be at most one launch ahead of a peer, because it needs
// the peer's candidate of launch n to finish launch n).  Waits are bounded and report GRM_ERR_FLAG_TIMEOUT.
#include "common.cuh"

namespace {

constexpr int kThreads = 1024;
constexpr int kNone = 0x7fffffff;

struct PickParams {
  const float* logits; int ld;      // [M][ld], columns 0..vn of this pointer are the local slice
  int vn, v0;
  uint2* recv[8];                   // every rank's slots [2 parity][W src][max_rows][2 words]
  int* epochs;                      // [max_rows] device counters
  int* out;                         // [M] tokens
  float* out_val;                   // [M] winning logit, or null
  unsigned int* status;
  int world, rank, max_rows;
  unsigned int spin;
};

__device__ __forceinline__ bool cand_better(float av, int ai, float bv, int bi) {   // is a better than b
  return av > bv || (av == bv && ai < bi);
}

__global__ void __launch_bounds__(kThreads) tp_head_pick_kernel(const PickParams p) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cv[8];
  __shared__ int ci[8];
  __shared__ int s_fail;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  grm_pdl_trigger();
  grm_pdl_wait();        // the logits come from the launch before this one
  const float* lg = p.logits + (size_t)row * p.ld;
  float bv = -INFINITY;
  int bi = kNone;
  for (int i = tid; i < p.vn; i += kThreads) {
    const float v = __ldcs(lg + i);
    if (v > bv || (v == bv && v > -INFINITY && i < bi)) { bv = v; bi = i; }     // NaN and -inf never become candidates
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  if (tid == 0) s_fail = 0;
  __syncthreads();
  if (warp == 0) {
    bv = sv[lane]; bi = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (cand_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int gi = bi == kNone ? kNone : bi + p.v0;
    const unsigned int ep = (unsigned int)p.epochs[row] + 1u;
    const size_t par = (size_t)(ep & 1u) * p.world * p.max_rows;
    if (lane < p.world) {
      if (lane == p.rank) {
        cv[lane] = bv; ci[lane] = gi;
      } else {
        uint2* dst = p.recv[lane] + (par + (size_t)p.rank * p.max_rows + row) * 2;
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(bv)), "r"(ep) : "memory");
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst + 1), "r"((unsigned int)gi), "r"(ep) : "memory");
        const uint2* src = p.recv[p.rank] + (par + (size_t)lane * p.max_rows + row) * 2;
        unsigned int a0 = 0u, a1 = 0u, b0 = 0u, b1 = 0u;
        bool got = false;
        for (unsigned int i = 0; i < p.spin; ++i) {
          asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(a0), "=r"(a1) : "l"(src) : "memory");
          asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "l"(src + 1) : "memory");
          if (a1 == ep && b1 == ep) { got = true; break; }
          if (i > 64) __nanosleep(40);
        }
        if (!got) { s_fail = 1; grm_set_error(p.status, GRM_ERR_FLAG_TIMEOUT, 0x60000u | ((unsigned int)lane << 12) | (unsigned int)(row & 0xfff)); }
        cv[lane] = __uint_as_float(a0); ci[lane] = (int)b0;
      }
    }
    __syncwarp();
    if (lane == 0) {
      p.epochs[row] = (int)ep;
      if (!s_fail) {
        float wv = cv[0];
        int wi = ci[0];
        for (int r = 1; r < p.world; ++r)
          if (cand_better(cv[r], ci[r], wv, wi)) { wv = cv[r]; wi = ci[r]; }
        p.out[row] = wi;
        if (p.out_val) p.out_val[row] = wv;
      }
    }
  }
}

}  // namespace

// logits: fp32 [M][ld] with this rank's vn columns starting at the pointer; v0: global index of column 0.
// recv: `world` peer-mapped pointers to each rank's slot array (2 * world * max_rows * 2 uint2 words, zero before the first
// use); epochs: max_rows zeroed ints on this device.  Every rank must make the same sequence of calls.
GRM_API int grm_tp_head_pick(const void* logits, int ld, int M, int vn, int v0, const void* const* recv, void* epochs, void* out,
                             void* out_val, int world, int rank, int max_rows, unsigned int spin, void* stream) {
  if (M <= 0) return 0;
  if (world < 2 || world > 8 || rank < 0 || rank >= world || M > max_rows || vn <= 0 || !recv || !epochs || !out) return -2;
  PickParams p;
  p.logits = (const float*)logits; p.ld = ld; p.vn = vn; p.v0 = v0;
  for (int i = 0; i < 8; ++i) p.recv[i] = i < world ? (uint2*)const_cast<void*>(recv[i]) : nullptr;
  p.epochs = (int*)epochs; p.out = (int*)out; p.out_val = (float*)out_val;
  p.status = grm_status_ptr();
  p.world = world; p.rank = rank; p.max_rows = max_rows;
  p.spin = spin ? spin : 4000000u;
  cudaError_t e = grm_launch_pdl(GRM_PDL_MISC, tp_head_pick_kernel, dim3(M), dim3(kThreads), 0, (cudaStream_t)stream, p);
  if (e != cudaSuccess) return (int)e;
  GRM_LAUNCH_RET();
}
