// paged_decode_attn_i8kv: attention of M independent query rows over the pooled int8 KV cache.
// A row is (sequence, position): one decode token of some conversation, or one row of a
// speculative verify block (row r of a block sees keys 0..pos_r, which is the causal rule inside
// the block).  Covers the reference's launch_flash_decode* / _rows / _batched + launch_flash_merge*
// (src/attention.cpp:109-1547) and the verify-attention entry point (src/attn_verify.hpp:40-69).
//
// Design (bandwidth-bound, int8 K and V with one fp32 scale per token and kv head):
//   grid = (splits, kv heads, rows); the G = Hq/Hkv query heads of a group share every K/V byte;
//   a warp owns whole 16-token pages and runs both products on the tensor cores (int8 QK^T straight
//   from the cached bytes, f16 PV), with the online softmax on the accumulator fragments;
//   the 4 warps merge in shared memory, split partials go to a scratch buffer and the last CTA to
//   arrive for a (row, kv head) merges the splits in split order (deterministic) and applies the
//   optional sigmoid output gate of gated attention.
#include "common.cuh"
#include "attn_mma.cuh"

namespace {

using namespace attn_mma;

constexpr int kPage = 16;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxSplits = 64;

struct DecParams {
  const bf16* q; int ld_q;
  const int* row_seq; const int* row_pos;
  const int* block_table; int max_pages;
  const int8_t* k_pages; const int8_t* v_pages; const float* k_scale; const float* v_scale;
  const bf16* gate;           // [M][Hq*D] or null
  bf16* out; int ld_o;
  float* part_o;              // [M][Hkv][splits][G][D]
  float* part_ml;             // [M][Hkv][splits][G][2]
  unsigned int* counters;     // [M*Hkv]
  int M, Hq, Hkv, window;
  float scale;
  // fused q/k norm + RoPE + KV append (qkv != null; one row per sequence in the launch): q is read from the raw fused
  // projection output and the CTA whose split holds the row's last page appends this token's K / V before it reads it
  const bf16* qkv; int ld_qkv;     // [M][(Hq + 2 Hkv) * D]
  const float* inv_freq;           // [rot / 2]
  const float* q_norm_w;           // [D] or null
  const float* k_norm_w;           // [D] or null
  float norm_eps, norm_offset;
  int rot;
  int prefetch;                    // 1: the kernel before this one in the stream writes only the qkv rows (see the kernel)
  unsigned int* status;            // device status block (bounded waits report here)
  int cluster;                     // 1: the splits of a (row, kv head) are one thread-block cluster and merge through DSMEM
  unsigned long long* tl;          // optional per-CTA timeline (8 words per CTA, thread 0: clock64 at the marks below)
};

constexpr int kMaxCluster = 16;   // splits merged through distributed shared memory (8 is the portable cluster size)

// Distributed shared memory helpers (thread-block cluster).  Addresses are 32-bit shared-window addresses of the LOCAL
// copy of a variable; mapa turns them into the address of the same variable in CTA ``cta`` of the cluster.
__device__ __forceinline__ uint32_t dsmem_addr(uint32_t local_addr, int cta) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(cta));
  return ra;
}
__device__ __forceinline__ void st_dsmem_f1(uint32_t remote_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_dsmem_f2(uint32_t remote_addr, float a, float b) {
  asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote_addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_remote(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0u;
}

unsigned long long* g_attn_timeline = nullptr;   // host-side: copied into DecParams::tl of every launch while set

__device__ __forceinline__ void tl_mark(const DecParams& p, int slot) {
  if (p.tl && threadIdx.x == 0) {
    const size_t cta = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    unsigned long long v;
    if (slot == 0 || slot == 7) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(v));
    else v = (unsigned long long)clock64();
    p.tl[cta * 8 + slot] = v;
  }
}

// Per-head RMSNorm (optional) and rotary embedding of one head held as v[i] = x[lane + 32 i] -- the arithmetic of
// rope_kv.cu, so the fused and the two-kernel paths produce the same bits.
template <int D>
__device__ __forceinline__ void head_norm_rope(float (&v)[D / 32], const float* nw, float eps, float offset, const float* inv_freq,
                                               int rot, float pos, int lane) {
  constexpr int per = D / 32;
  if (nw) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < per; ++i) ss += v[i] * v[i];
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)D + eps);
#pragma unroll
    for (int i = 0; i < per; ++i) v[i] = v[i] * r * (offset + nw[lane + 32 * i]);
  }
  const int hreg = rot >> 6;   // registers per rotary half
#pragma unroll
  for (int i = 0; i < per / 2; ++i) {
    if (i < hreg) {
      const float ang = pos * inv_freq[lane + 32 * i];
      float sn, cs;
      sincosf(ang, &sn, &cs);
      const float a = v[i], b = v[i + hreg];
      v[i] = a * cs - b * sn;
      v[i + hreg] = b * cs + a * sn;
    }
  }
}

// Tensor-core formulation.  Per 16-token page and warp:
//   S[head][token] = Q K^T with the G query heads of the group as MMA rows (8 of 16 rows used), the page's
//     tokens as two n8 tiles and int8 operands: K bytes go from global memory straight into the B
//     fragments (lane t of a quad owns 16 contiguous dims of a 64-dim half; A and B use the same
//     dim -> k-slot mapping, so no shuffling is needed), q is quantised once per CTA to 15 bits as
//     128*hi + lo with int8 hi / lo and both levels are accumulated in int32;
//   online softmax on the C fragments (a head's 16 scores live in one quad: 2 shuffles per reduction);
//   O[head][dim] += P V with P (f16, the token's V scale folded in) reused from the C fragments as the A
//     operand and V bytes expanded to f16 by byte permutes as 1152 + v; the constant is removed at
//     the end with the running sum of the rounded P values (exact in fp32).
__device__ __forceinline__ int bt_page(const DecParams& p, int seq, int page_index) {
  return p.block_table[(size_t)seq * p.max_pages + page_index];
}

template <int D, int G>
__global__ void __launch_bounds__(kThreads) decode_attn_kernel(const DecParams p) {
  static_assert(G <= 8 && (D == 64 || D == 128 || D == 256), "unsupported geometry");
  constexpr int NH = D / 64;       // 64-dim halves of the QK contraction
  constexpr int DT = D / 8;        // dims per row group g in the PV product = number of n8 tiles
  constexpr int VW = DT / 4;       // 32-bit words of V per token row and lane
  __shared__ __align__(16) int8_t q_hi[8][D];
  __shared__ __align__(16) int8_t q_lo[8][D];
  __shared__ float q_delta[8];
  __shared__ float sm_ml[kWarps][G][2];
  __shared__ __align__(16) float sm_o[kWarps][G][D];
  __shared__ int s_last;
  // cluster merge: CTA r owns outputs [r * per, (r + 1) * per) of the G x D block and receives every split's partial values
  // of that slice (cl_recv[source][j]) and (max, sum) pairs (cl_rml[source][head]) by remote shared-memory stores
  __shared__ __align__(16) float cl_recv[G * D + kMaxCluster];
  __shared__ __align__(16) float cl_rml[kMaxCluster][G][2];
  __shared__ __align__(16) float cl_ml[G][2];
  __shared__ __align__(8) uint64_t cl_bar;

  const int split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int nsplit = gridDim.x;
  tl_mark(p, 0);
  tl_mark(p, 1);
  if (p.cluster) {
    // arrival barrier of the merge: one arrival per split.  Its initialisation is published to the cluster by the
    // arrive half of a cluster barrier here; the wait half sits right before the first remote store.
    if (threadIdx.x == 0) {
      mbar_init(&cl_bar, (uint32_t)gridDim.x);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    cluster_arrive();
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int seq = p.row_seq[row];
  const int len = p.row_pos[row] + 1;
  const int first = (p.window > 0 && len > p.window) ? (len - p.window) : 0;
  const int page_lo = first / kPage;
  const int page_hi = (len + kPage - 1) / kPage;       // exclusive
  const int npages = page_hi - page_lo;
  const int pps = (npages + nsplit - 1) / nsplit;
  const int pbeg = page_lo + split * pps;
  const int pend = min(pbeg + pps, page_hi);

  const bool fused = p.qkv != nullptr;
  const int* bt = p.block_table + (size_t)seq * p.max_pages;

  // ---- per-warp ring of whole pages in shared memory, filled by cp.async STAGES-1 pages ahead ----
  // stage = K page [16][D] | V page [16][D] | K scales [16] | V scales [16]; 16-byte chunks are XOR-swizzled
  // so the fragment reads below are bank-conflict free.
  constexpr int STAGES = (D == 256) ? 3 : 4;
  constexpr int STAGE_BYTES = 2 * kPage * D + 128;
  constexpr int CPR = D / 16;                           // 16-byte chunks per token row
  extern __shared__ __align__(128) uint8_t ring_raw[];
  uint8_t* ring = ring_raw + (size_t)warp * STAGES * STAGE_BYTES;
  auto k_off = [](int r, int c) { return r * D + 16 * (D >= 128 ? (c ^ (4 * (r & 1))) : c); };
  auto v_off = [](int r, int c) {
    const int x = (r >> 1) & 3;
    const int sw = D == 128 ? 2 * x : (D == 256 ? ((x & 1) | ((x & 2) << 1)) : 0);
    return kPage * D + r * D + 16 * (c ^ sw);
  };
  auto issue = [&](int page, int st) {
    if (page < pend) {
      const size_t pb = ((size_t)bt[page] * p.Hkv + kvh) * kPage;
      const uint32_t sb = smem_u32(ring + st * STAGE_BYTES);
      const int8_t* ksrc = p.k_pages + pb * D;
      const int8_t* vsrc = p.v_pages + pb * D;
#pragma unroll
      for (int i = 0; i < D / 32; ++i) {
        const int idx = lane + 32 * i, r = idx / CPR, c = idx % CPR;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sb + k_off(r, c)), "l"(ksrc + 16 * idx) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sb + v_off(r, c)), "l"(vsrc + 16 * idx) : "memory");
      }
      if (lane < 8) {
        const float* ssrc = (lane < 4 ? p.k_scale : p.v_scale) + pb + 4 * (lane & 3);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sb + 2 * kPage * D + 16 * lane), "l"(ssrc) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  // Programmatic dependent launch: this kernel may start while its predecessor (the q|k|v projection) is still running.
  // Everything the predecessor does not write -- the row tables, the block table, the pages of earlier tokens -- may be
  // read before grm_pdl_wait(): with p.prefetch every warp requests its first STAGES-1 pages here, so they are in shared
  // memory by the time the projection has finished.  The one page that receives this step's K / V (the last page, in
  // the CTA that appends to it) is requested after the append.  Without PDL (or with p.prefetch 0) the loads start
  // after the q prologue: requesting them right before it in the same kernel was measured and does not pay, the
  // prologue's own global loads then return behind the page traffic.
  grm_pdl_trigger();
  const int hot_page = (fused && pbeg < pend && pend == page_hi) ? (len - 1) / kPage : -1;
  int pg = pbeg + warp;
  bool late = false;                 // this warp owns the page that is loaded after the append
  if (p.prefetch) {
#pragma unroll
    for (int s0 = 0; s0 < STAGES - 1; ++s0) {
      const int pgs = pg + s0 * kWarps;
      const bool defer = pgs == hot_page;
      late = late || defer;
      issue(defer ? pend : pgs, s0);           // a page index >= pend commits an empty group
    }
  }
  grm_pdl_wait();
  if (fused && pbeg < pend && pend == page_hi && warp < 2) {
    // This CTA's split holds the last page: append the row's K (warp 0: norm, RoPE) and V (warp 1) to it -- int8 with a
    // scale per (token, head) -- before the barrier below; the page loads start after it.
    const int pos = len - 1;
    const int page = bt_page(p, seq, pos / kPage);
    if (page >= 0) {
      const bf16* src = p.qkv + (size_t)row * p.ld_qkv + (size_t)p.Hq * D + (size_t)((warp == 0 ? 0 : p.Hkv) + kvh) * D;
      float v[D / 32];
#pragma unroll
      for (int i = 0; i < D / 32; ++i) v[i] = __bfloat162float(src[lane + 32 * i]);
      if (warp == 0) head_norm_rope<D>(v, p.k_norm_w, p.norm_eps, p.norm_offset, p.inv_freq, p.rot, (float)pos, lane);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < D / 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
      amax = warp_max(amax);
      const float sc = amax > 0.f ? amax / 127.f : 1.f;
      const float inv = 1.f / sc;
      const size_t base = ((size_t)page * p.Hkv + kvh) * kPage + (pos % kPage);
      int8_t* dst = const_cast<int8_t*>(warp == 0 ? p.k_pages : p.v_pages) + base * D;
#pragma unroll
      for (int i = 0; i < D / 32; ++i) dst[lane + 32 * i] = (int8_t)max(-127, min(127, __float2int_rn(v[i] * inv)));
      if (lane == 0) const_cast<float*>(warp == 0 ? p.k_scale : p.v_scale)[base] = sc;
    }
  }
  // ---- q -> two int8 levels per head (warp w quantises heads w, w + 4; both heads' loads are in flight together) ----
  float qv[8 / kWarps][D / 32];
#pragma unroll
  for (int it = 0; it < 8 / kWarps; ++it) {
    const int h = warp + kWarps * it;
    if (h < G) {
      const bf16* src = fused ? p.qkv + (size_t)row * p.ld_qkv + (size_t)(kvh * G + h) * D
                              : p.q + (size_t)row * p.ld_q + (size_t)(kvh * G + h) * D;
#pragma unroll
      for (int i = 0; i < D / 32; ++i) qv[it][i] = __bfloat162float(src[lane + 32 * i]);
    } else {
#pragma unroll
      for (int i = 0; i < D / 32; ++i) qv[it][i] = 0.f;
    }
  }
#pragma unroll
  for (int it = 0; it < 8 / kWarps; ++it) {
    const int h = warp + kWarps * it;
    float (&v)[D / 32] = qv[it];
    float mx = 0.f;
    if (fused && h < G) {
      head_norm_rope<D>(v, p.q_norm_w, p.norm_eps, p.norm_offset, p.inv_freq, p.rot, (float)(len - 1), lane);
#pragma unroll
      for (int i = 0; i < D / 32; ++i) v[i] = __bfloat162float(__float2bfloat16(v[i]));     // the two-kernel path rounds q to bf16
    }
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      v[i] *= p.scale;
      mx = fmaxf(mx, fabsf(v[i]));
    }
    mx = warp_max(mx);
    const float delta = mx > 0.f ? mx / 16256.f : 1.f;
    const float inv = 1.f / delta;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const int qi = __float2int_rn(v[i] * inv);
      const int hi = (qi + 64) >> 7;
      q_hi[h][lane + 32 * i] = (int8_t)hi;
      q_lo[h][lane + 32 * i] = (int8_t)(qi - 128 * hi);
    }
    if (lane == 0) q_delta[h] = h < G ? delta : 0.f;
  }
  __syncthreads();
  tl_mark(p, 2);
  uint32_t qa_hi[NH][4], qa_lo[NH][4];
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    const uint4 a = *reinterpret_cast<const uint4*>(&q_hi[g][64 * h + 16 * t]);
    const uint4 b = *reinterpret_cast<const uint4*>(&q_lo[g][64 * h + 16 * t]);
    qa_hi[h][0] = a.x; qa_hi[h][1] = a.y; qa_hi[h][2] = a.z; qa_hi[h][3] = a.w;
    qa_lo[h][0] = b.x; qa_lo[h][1] = b.y; qa_lo[h][2] = b.z; qa_lo[h][3] = b.w;
  }
  const float qd = q_delta[g];

  float m_run = -INFINITY, l_part = 0.f, lv_part = 0.f;   // head g: running max, this lane's share of sum p and of sum f16(p*vs)
  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
  if (!p.prefetch) {
#pragma unroll
    for (int s0 = 0; s0 < STAGES - 1; ++s0) issue(pg + s0 * kWarps, s0);
  } else if (late) {
    // the appended page is this warp's last one and is visible now (barrier above): one more group; the loop then
    // waits for all groups instead of all but the newest ones
    issue(hot_page, ((hot_page - pg) / kWarps) % STAGES);
  }
  int st = 0;
  for (; pg < pend; pg += kWarps) {
    if (late) asm volatile("cp.async.wait_group 0;" ::: "memory");
    else asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncwarp();
    issue(pg + (STAGES - 1) * kWarps, (st + STAGES - 1) % STAGES);
    const uint8_t* sb = ring + st * STAGE_BYTES;
    st = (st + 1 == STAGES) ? 0 : st + 1;
    uint4 kreg[2][NH];                 // K rows of tokens g and g + 8, this lane's 16 dims per 64-dim half
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int h = 0; h < NH; ++h) kreg[nt][h] = *reinterpret_cast<const uint4*>(sb + k_off(8 * nt + g, 4 * h + t));
    float2 ksc[2], vsc[2];             // scales of tokens (2t, 2t+1) and (2t+8, 2t+9)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      ksc[nt] = *reinterpret_cast<const float2*>(sb + 2 * kPage * D + 4 * (8 * nt + 2 * t));
      vsc[nt] = *reinterpret_cast<const float2*>(sb + 2 * kPage * D + 64 + 4 * (8 * nt + 2 * t));
    }
    // V rows 2t, 2t+1, 2t+8, 2t+9: this lane's DT contiguous dims [DT*g, DT*g + DT)
    uint32_t vraw[4][VW];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int vr = 2 * t + (r & 1) + 8 * (r >> 1);
      if (VW == 2) {
        const uint2 w = *reinterpret_cast<const uint2*>(sb + v_off(vr, g >> 1) + 8 * (g & 1));
        vraw[r][0] = w.x; vraw[r][VW - 1] = w.y;
      } else {
#pragma unroll
        for (int q4 = 0; q4 < VW / 4; ++q4) {
          const uint4 w = *reinterpret_cast<const uint4*>(sb + v_off(vr, (VW / 4) * g + q4));
          vraw[r][4 * q4] = w.x; vraw[r][4 * q4 + 1] = w.y; vraw[r][4 * q4 + 2] = w.z; vraw[r][4 * q4 + 3] = w.w;
        }
      }
    }
    // ---- S = Q K^T (int8, two levels) ----
    int s_hi[2][4], s_lo[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) { s_hi[nt][c] = 0; s_lo[nt][c] = 0; }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int h = 0; h < NH; ++h) {
        const uint32_t kw[4] = {kreg[nt][h].x, kreg[nt][h].y, kreg[nt][h].z, kreg[nt][h].w};
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          mma_s8_16832(s_hi[nt], qa_hi[h][2 * s], 0u, qa_hi[h][2 * s + 1], 0u, kw[2 * s], kw[2 * s + 1]);
          mma_s8_16832(s_lo[nt], qa_lo[h][2 * s], 0u, qa_lo[h][2 * s + 1], 0u, kw[2 * s], kw[2 * s + 1]);
        }
      }
    const float2 ksc_c[2] = {ksc[0], ksc[1]}, vsc_c[2] = {vsc[0], vsc[1]};
    // ---- online softmax for head g over this lane's 4 tokens, quad reductions ----
    float sc[4];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int nt = i >> 1, c = i & 1;
      const int tok = pg * kPage + 8 * nt + 2 * t + c;
      const float ks = c ? ksc_c[nt].y : ksc_c[nt].x;
      const float sv = (float)(128 * s_hi[nt][c] + s_lo[nt][c]) * qd * ks;
      sc[i] = (tok < len && tok >= first) ? sv : -INFINITY;
      mx = fmaxf(mx, sc[i]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mnew = fmaxf(m_run, mx);
    const float alpha = (m_run == -INFINITY) ? 0.f : __expf(m_run - mnew);
    m_run = mnew;
    float pv[4];
    float psum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float pr = (sc[i] == -INFINITY) ? 0.f : __expf(sc[i] - mnew);
      psum += pr;
      pv[i] = pr * ((i & 1) ? vsc_c[i >> 1].y : vsc_c[i >> 1].x) * 1024.f;   // lifted out of the f16 subnormal range
    }
    const uint32_t pa0 = pack_f16x2(pv[0], pv[1]), pa2 = pack_f16x2(pv[2], pv[3]);
    const float2 r0 = __half22float2(*reinterpret_cast<const __half2*>(&pa0));
    const float2 r2 = __half22float2(*reinterpret_cast<const __half2*>(&pa2));
    l_part = l_part * alpha + psum;
    lv_part = lv_part * alpha + (r0.x + r0.y + r2.x + r2.y);
    // ---- O = alpha O + P V ----
#pragma unroll
    for (int w = 0; w < VW; ++w) {
      // bytes of rows (2t, 2t+1) and (2t+8, 2t+9), interleaved per dim, biased to unsigned
      const uint32_t lo01 = prmt(vraw[0][w], vraw[1][w], 0x5140u) ^ 0x80808080u, hi01 = prmt(vraw[0][w], vraw[1][w], 0x7362u) ^ 0x80808080u;
      const uint32_t lo89 = prmt(vraw[2][w], vraw[3][w], 0x5140u) ^ 0x80808080u, hi89 = prmt(vraw[2][w], vraw[3][w], 0x7362u) ^ 0x80808080u;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = 4 * w + e;
        const uint32_t src01 = e < 2 ? lo01 : hi01, src89 = e < 2 ? lo89 : hi89;
        const uint32_t sel = (e & 1) ? 0x4342u : 0x4140u;
        const uint32_t b0 = prmt(src01, 0x64646464u, sel), b1 = prmt(src89, 0x64646464u, sel);
        o[j][0] *= alpha; o[j][1] *= alpha;
        mma_f16_16816(o[j], pa0, 0u, pa2, 0u, b0, b1);
      }
    }
  }

  asm volatile("cp.async.wait_group 0;" ::: "memory");
  tl_mark(p, 3);
  // ---- this warp's result for head g: quad-reduce the sums, remove the 1152 bias, stage for the CTA merge ----
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 1);
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 2);
  lv_part += __shfl_xor_sync(0xffffffffu, lv_part, 1);
  lv_part += __shfl_xor_sync(0xffffffffu, lv_part, 2);
  if (g < G) {
    if (t == 0) { sm_ml[warp][g][0] = m_run; sm_ml[warp][g][1] = l_part; }
    const float bias = 1152.f * lv_part;
    // lane (g, t) owns the D/4 contiguous dims [t * D/4, (t + 1) * D/4) of head g: o[j][0] is dim 2t*DT + j and o[j][1]
    // dim (2t+1)*DT + j.  They are stored as float4 chunks whose position inside the lane's window is rotated by
    // so_rot(g, t), so that the eight lanes of a store phase hit eight different groups of four banks (unrotated, every
    // lane of the warp would start at bank 0).  so_index() is the matching read mapping.
    float* dst = &sm_o[warp][g][t * (D / 4)];
    const int rot = so_rot<D>(g, t);
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      const int c = i / (DT / 4), j0 = 4 * (i % (DT / 4));       // chunk i = dims 4i..4i+3 of the window
      float4 v4;
      v4.x = (o[j0][c] - bias) * (1.f / 1024.f); v4.y = (o[j0 + 1][c] - bias) * (1.f / 1024.f);
      v4.z = (o[j0 + 2][c] - bias) * (1.f / 1024.f); v4.w = (o[j0 + 3][c] - bias) * (1.f / 1024.f);
      *reinterpret_cast<float4*>(dst + 4 * ((i + rot) & (D / 16 - 1))) = v4;
    }
  }
  __syncthreads();

  if (p.cluster) cluster_wait();        // every CTA of the cluster has initialised its arrival barrier
  const size_t pidx = ((size_t)row * p.Hkv + kvh) * nsplit + split;
  for (int i = tid; i < G * D; i += kThreads) {
    const int g = i / D, d = i % D;
    float M_ = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M_ = fmaxf(M_, sm_ml[w][g][0]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = sm_ml[w][g][0];
      const float f = (mw == -INFINITY) ? 0.f : __expf(mw - M_);
      L += sm_ml[w][g][1] * f;
      O += sm_o[w][g][so_index<D>(g, d)] * f;
    }
    if (nsplit == 1) {
      float r = L > 0.f ? O / L : 0.f;
      const size_t oi = (size_t)row * p.ld_o + (size_t)(kvh * G + g) * D + d;
      if (p.gate) r *= sigmoid_f(__bfloat162float(p.gate[oi]));
      p.out[oi] = __float2bfloat16(r);
    } else if (p.cluster) {
      const int per = (G * D + nsplit - 1) / nsplit;
      const int r = i / per, j = i - r * per;
      st_dsmem_f1(dsmem_addr(smem_u32(&cl_recv[split * per + j]), r), O);
      if (d == 0) { cl_ml[g][0] = M_; cl_ml[g][1] = L; }
    } else {
      p.part_o[(pidx * G + g) * D + d] = O;
      if (d == 0) { p.part_ml[(pidx * G + g) * 2] = M_; p.part_ml[(pidx * G + g) * 2 + 1] = L; }
    }
  }
  if (nsplit == 1) return;
  tl_mark(p, 4);
  if (p.cluster) {
    // The splits of this (row, kv head) are the CTAs of one cluster.  Every CTA has pushed slice r of its un-normalised
    // output into CTA r's shared memory (above); it now pushes its (max, sum) pairs to every CTA, makes the stores
    // visible and arrives on every CTA's barrier.  CTA r waits (bounded) for the nsplit arrivals on its own barrier and
    // combines its slice in split order with the arithmetic of the last-CTA merge below.  Nobody reads another CTA's
    // memory, so a CTA may exit as soon as its own slice is written.
    __syncthreads();
    for (int idx = tid; idx < nsplit * G; idx += kThreads) {
      const int r = idx / G, g = idx - r * G;
      st_dsmem_f2(dsmem_addr(smem_u32(&cl_rml[split][g][0]), r), cl_ml[g][0], cl_ml[g][1]);
    }
    __syncthreads();
    if (tid < nsplit) {
      asm volatile("fence.acq_rel.cluster;" ::: "memory");
      mbar_arrive_remote(dsmem_addr(smem_u32(&cl_bar), tid));
    }
    tl_mark(p, 5);
    {
      const uint32_t bar = smem_u32(&cl_bar);
      bool ok = mbar_try_wait_cluster(bar, 0u);
      for (unsigned int it = 0; !ok && it < 4000000u; ++it) {
        __nanosleep(32);
        ok = mbar_try_wait_cluster(bar, 0u);
      }
      if (!ok) {
        if (tid == 0) grm_set_error(p.status, GRM_ERR_MBAR_TIMEOUT, 0x70000u | (unsigned int)split);
        return;
      }
    }
    const int per = (G * D + nsplit - 1) / nsplit;
    for (int j = tid; j < per; j += kThreads) {
      const int e = split * per + j;
      if (e >= G * D) break;
      const int g = e / D, d = e % D;
      float M_ = -INFINITY;
#pragma unroll
      for (int sp = 0; sp < kMaxCluster; ++sp) if (sp < nsplit) M_ = fmaxf(M_, cl_rml[sp][g][0]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int sp = 0; sp < kMaxCluster; ++sp) {
        if (sp < nsplit) {
          const float ms = cl_rml[sp][g][0];
          const float f = (ms == -INFINITY) ? 0.f : __expf(ms - M_);
          L += cl_rml[sp][g][1] * f;
          O = fmaf(cl_recv[sp * per + j], f, O);
        }
      }
      float r = O * (L > 0.f ? 1.f / L : 0.f);
      const size_t oi = (size_t)row * p.ld_o + (size_t)(kvh * G + g) * D + d;
      if (p.gate) r *= sigmoid_f(__bfloat162float(p.gate[oi]));
      p.out[oi] = __float2bfloat16(r);
    }
    tl_mark(p, 6);
    tl_mark(p, 7);
    return;
  }

  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int prev = atomicAdd(&p.counters[row * p.Hkv + kvh], 1u);
    s_last = (prev == (unsigned int)nsplit - 1u);
    if (s_last) p.counters[row * p.Hkv + kvh] = 0u;
  }
  __syncthreads();
  tl_mark(p, 5);
  if (!s_last) { tl_mark(p, 7); return; }
  __threadfence();
  // Last CTA of this (row, kv head): merge the splits in split order.  The per-split (max, sum) pairs
  // are staged in shared memory first so the long loop only carries independent loads.
  const size_t base = ((size_t)row * p.Hkv + kvh) * nsplit;
  float* wts = &sm_o[0][0][0];            // reuse: [G][kMaxSplits] weights
  for (int i = tid; i < G * nsplit; i += kThreads) {
    const int g = i / nsplit, sp = i % nsplit;
    wts[g * kMaxSplits + sp] = __ldcg(&p.part_ml[((base + sp) * G + g) * 2]);
  }
  __syncthreads();
  if (tid < G) {
    float M_ = -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) M_ = fmaxf(M_, wts[tid * kMaxSplits + sp]);
    float L = 0.f;
    for (int sp = 0; sp < nsplit; ++sp) {
      const float ms = wts[tid * kMaxSplits + sp];
      const float f = (ms == -INFINITY) ? 0.f : __expf(ms - M_);
      wts[tid * kMaxSplits + sp] = f;
      L += __ldcg(&p.part_ml[((base + sp) * G + tid) * 2 + 1]) * f;
    }
    sm_ml[0][tid][0] = L;
  }
  __syncthreads();
  for (int i = tid; i < G * D / 4; i += kThreads) {
    const int g = i / (D / 4), d = 4 * (i % (D / 4));
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 16
    for (int sp = 0; sp < nsplit; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(&p.part_o[((base + sp) * G + g) * D + d]));
      const float w = wts[g * kMaxSplits + sp];
      O.x = fmaf(v.x, w, O.x); O.y = fmaf(v.y, w, O.y); O.z = fmaf(v.z, w, O.z); O.w = fmaf(v.w, w, O.w);
    }
    const float L = sm_ml[0][g][0];
    const float inv = L > 0.f ? 1.f / L : 0.f;
    float r[4] = {O.x * inv, O.y * inv, O.z * inv, O.w * inv};
    const size_t oi = (size_t)row * p.ld_o + (size_t)(kvh * G + g) * D + d;
    if (p.gate) {
#pragma unroll
      for (int c = 0; c < 4; ++c) r[c] *= sigmoid_f(__bfloat162float(p.gate[oi + c]));
    }
    uint2 o2;
    o2.x = pack_bf16x2(r[0], r[1]); o2.y = pack_bf16x2(r[2], r[3]);
    *reinterpret_cast<uint2*>(p.out + oi) = o2;
  }
  tl_mark(p, 6);
  tl_mark(p, 7);
}

int g_attn_cluster = 1;     // 0: always merge the splits through global scratch and the last-arriving CTA

template <int D, int G>
int launch(const DecParams& p_in, int splits, cudaStream_t st) {
  dim3 grid(splits, p_in.Hkv, p_in.M);
  constexpr int kRing = kWarps * ((D == 256) ? 3 : 4) * (2 * kPage * D + 128);
  // per template instance: 0 = not configured, 1 = clusters of up to 8, 2 = clusters of up to 16, -1 = no clusters
  static int configured = 0;
  if (configured == 0) {
    cudaError_t e = cudaFuncSetAttribute(decode_attn_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing);
    if (e != cudaSuccess) return (int)e;
    configured = 1;
    if (cudaFuncSetAttribute(decode_attn_kernel<D, G>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
      // a cluster of 16 must fit one GPC with this kernel's shared memory: ask the occupancy calculator
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(16, 1, 1); cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kRing;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 16; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      int nclusters = 0;
      if (cudaOccupancyMaxActiveClusters(&nclusters, decode_attn_kernel<D, G>, &cfg) == cudaSuccess && nclusters >= 1) configured = 2;
    }
    (void)cudaGetLastError();
  }
  DecParams p = p_in;
  p.status = grm_status_ptr();
  const int max_cl = configured == 2 ? 16 : 8;
  // clusters of 16 only while the whole grid is co-resident: with more CTAs than SMs the wait for a GPC with 16 free SMs
  // delays the launch of the later clusters by more than the merge saves (measured: 8 rows x 8 kv heads x 16 splits)
  const long ctas = (long)splits * p.Hkv * p.M;
  p.cluster = (g_attn_cluster && splits >= 2 && splits <= max_cl && (splits <= 8 || ctas <= 148)) ? 1 : 0;
  if (p.cluster) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = kRing; cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)splits; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = (grm_pdl_enabled() & GRM_PDL_ATTN) ? 1 : 0;
    cfg.attrs = at; cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_attn_kernel<D, G>, p);
    if (e != cudaSuccess) return (int)e;
    GRM_LAUNCH_RET();
  }
  cudaError_t e = grm_launch_pdl(GRM_PDL_ATTN, decode_attn_kernel<D, G>, grid, dim3(kThreads), (size_t)kRing, st, p);
  if (e != cudaSuccess) return (int)e;
  GRM_LAUNCH_RET();
}

template <int D>
int launch_g(const DecParams& p, int G, int splits, cudaStream_t st) {
  switch (G) {
    case 1: return launch<D, 1>(p, splits, st);
    case 2: return launch<D, 2>(p, splits, st);
    case 4: return launch<D, 4>(p, splits, st);
    case 5: return launch<D, 5>(p, splits, st);
    case 6: return launch<D, 6>(p, splits, st);
    case 8: return launch<D, 8>(p, splits, st);
    default: return -2;
  }
}

}  // namespace

// Debug aid: while set, every decode-attention launch writes 8 words per CTA (marks 0 and 7: %globaltimer at entry and
// exit; 1..6: clock64 at entry, after the q prologue, after the page loop, after the CTA merge, after the arrival
// counter, after the split merge of the last CTA).  The buffer must hold 8 * grid words; null switches it off.
GRM_API void grm_attn_set_timeline(void* buf) { g_attn_timeline = (unsigned long long*)buf; }

// 1 (default): splits of up to 16 CTAs merge through cluster shared memory; 0: through global scratch.
GRM_API void grm_attn_set_cluster(int on) { g_attn_cluster = on; }

// part_o: fp32 M*Hq*splits*D, part_ml: fp32 M*Hq*splits*2, counters: M*Hkv zeroed uints (only read
// when splits > 1).  window <= 0 disables the sliding window.
GRM_API int grm_paged_decode_attn(const void* q, int ld_q, const void* row_seq, const void* row_pos, const void* block_table,
                                  int max_pages, const void* k_pages, const void* v_pages, const void* k_scale,
                                  const void* v_scale, const void* gate, void* out, int ld_o, void* part_o, void* part_ml,
                                  void* counters, int M, int Hq, int Hkv, int D, int splits, int window, float scale,
                                  void* stream) {
  if (M < 1 || Hkv < 1 || Hq % Hkv || splits < 1 || splits > kMaxSplits || (ld_o & 3)) return -2;
  if (splits > 1 && (!part_o || !part_ml || !counters)) return -2;
  DecParams p;
  p.q = (const bf16*)q; p.ld_q = ld_q; p.row_seq = (const int*)row_seq; p.row_pos = (const int*)row_pos;
  p.block_table = (const int*)block_table; p.max_pages = max_pages;
  p.k_pages = (const int8_t*)k_pages; p.v_pages = (const int8_t*)v_pages; p.k_scale = (const float*)k_scale; p.v_scale = (const float*)v_scale;
  p.gate = (const bf16*)gate; p.out = (bf16*)out; p.ld_o = ld_o; p.part_o = (float*)part_o; p.part_ml = (float*)part_ml;
  p.counters = (unsigned int*)counters; p.M = M; p.Hq = Hq; p.Hkv = Hkv; p.window = window; p.scale = scale;
  p.qkv = nullptr; p.ld_qkv = 0; p.inv_freq = nullptr; p.q_norm_w = p.k_norm_w = nullptr; p.norm_eps = p.norm_offset = 0.f; p.rot = 0;
  p.tl = g_attn_timeline; p.prefetch = 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int G = Hq / Hkv;
  switch (D) {
    case 64: return launch_g<64>(p, G, splits, st);
    case 128: return launch_g<128>(p, G, splits, st);
    case 256: return launch_g<256>(p, G, splits, st);
    default: return -2;
  }
}

// The same attention with the q/k norm, RoPE and the KV append of the rows' own tokens folded in (the work of
// grm_rope_kvwrite): qkv is the raw fused projection output [M][(Hq + 2 Hkv) * D] (ungated q).  Valid when no row
// attends to a token that another row of the same launch appends, i.e. every row is a different sequence.
// prefetch != 0 promises that the kernel launched before this one in the stream writes nothing this kernel reads except
// the qkv rows (it is the q|k|v projection): the pages of earlier tokens are then requested while that kernel is still
// running (programmatic dependent launch).
GRM_API int grm_paged_decode_attn_fused(const void* qkv, int ld_qkv, const void* inv_freq, const void* q_norm_w, const void* k_norm_w,
                                        float norm_eps, float norm_offset, int rot, const void* row_seq, const void* row_pos,
                                        const void* block_table, int max_pages, void* k_pages, void* v_pages, void* k_scale,
                                        void* v_scale, void* out, int ld_o, void* part_o, void* part_ml, void* counters, int M,
                                        int Hq, int Hkv, int D, int splits, int window, float scale, int prefetch, void* stream) {
  if (M < 1 || Hkv < 1 || Hq % Hkv || splits < 1 || splits > kMaxSplits || (ld_o & 3) || !qkv || !inv_freq || (rot & 63) || rot > D ||
      rot < 64)
    return -2;
  if (splits > 1 && (!part_o || !part_ml || !counters)) return -2;
  DecParams p;
  p.q = nullptr; p.ld_q = 0; p.row_seq = (const int*)row_seq; p.row_pos = (const int*)row_pos;
  p.block_table = (const int*)block_table; p.max_pages = max_pages;
  p.k_pages = (const int8_t*)k_pages; p.v_pages = (const int8_t*)v_pages; p.k_scale = (const float*)k_scale; p.v_scale = (const float*)v_scale;
  p.gate = nullptr; p.out = (bf16*)out; p.ld_o = ld_o; p.part_o = (float*)part_o; p.part_ml = (float*)part_ml;
  p.counters = (unsigned int*)counters; p.M = M; p.Hq = Hq; p.Hkv = Hkv; p.window = window; p.scale = scale;
  p.qkv = (const bf16*)qkv; p.ld_qkv = ld_qkv; p.inv_freq = (const float*)inv_freq; p.q_norm_w = (const float*)q_norm_w;
  p.k_norm_w = (const float*)k_norm_w; p.norm_eps = norm_eps; p.norm_offset = norm_offset; p.rot = rot;
  p.tl = g_attn_timeline; p.prefetch = (prefetch && (grm_pdl_enabled() & GRM_PDL_ATTN) && (grm_pdl_enabled() & GRM_PDL_ATTN_PREFETCH)) ? 1 : 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int G = Hq / Hkv;
  switch (D) {
    case 64: return launch_g<64>(p, G, splits, st);
    case 128: return launch_g<128>(p, G, splits, st);
    case 256: return launch_g<256>(p, G, splits, st);
    default: return -2;
  }
}
