// paged_verify_attn_i8kv: attention of a speculative VERIFY BLOCK -- several consecutive positions of one sequence --
// over the pooled int8 KV cache in one pass over the pages.
//
// The decode kernel (attn_decode.cu) puts the G = Hq / Hkv query heads of a KV head into the rows of a 16-row MMA tile and
// leaves rows 8..15 empty; run on a verify block it reads the cache once per row.  Here the MMA rows are (block row, query
// head) PAIRS: pair p = r * G + h for block row r and head h, up to 16 pairs per CTA (floor(16 / G) rows: 3 rows for the
// 40 / 8 head split, 4 rows for 32 / 8, 16 rows for MQA-style G = 1), so every K / V byte of the context is read once per
// group of rows instead of once per row.  Row r of the block sits at position pos0 + r and sees keys 0 .. pos0 + r: the
// causal rule inside the block is a per-pair length applied to the scores (only the last page or two differ).  Blocks
// taller than one group run as several z entries of the grid (the caller's block table lists them).  Everything else is
// the decode kernel's formulation: per-warp cp.async ring of whole pages, int8 QK^T with q in two int8 levels, online
// softmax on the accumulator fragments, f16 PV with the V scale folded into P, 4-warp merge in shared memory, split-KV
// with a deterministic last-CTA merge.  K / V of the block's own tokens are appended before this kernel runs
// (rope_kv.cu).  Reference: launch_verify_attn_dpas / launch_verify_merge (src/attn_verify.hpp:48-69), which put
// (draft rows x q heads of a KV head) into the matrix unit's M dimension for the same reason.
#include "common.cuh"
#include "attn_mma.cuh"

namespace {

using namespace attn_mma;

constexpr int kPage = 16;
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxSplits = 64;
constexpr int kPairs = 16;

struct VerParams {
  const bf16* q; int ld_q;                 // [rows][Hq * D], already normed / rotated
  const int* blk_seq;                      // per grid z: sequence slot,
  const int* blk_row0;                     //   first row in q / out,
  const int* blk_nrows;                    //   rows of this group (<= 16 / G),
  const int* blk_pos0;                     //   position of its first row
  const int* block_table; int max_pages;
  const int8_t* k_pages; const int8_t* v_pages; const float* k_scale; const float* v_scale;
  const bf16* gate;                        // [rows][Hq * D] or null
  bf16* out; int ld_o;
  float* part_o;                           // [blocks][Hkv][splits][16][D]
  float* part_ml;                          // [blocks][Hkv][splits][16][2]
  unsigned int* counters;                  // [blocks * Hkv], zero between launches
  int Hq, Hkv, G, window;
  float scale;
};

template <int D>
__global__ void __launch_bounds__(kThreads) verify_attn_kernel(const VerParams p) {
  static_assert(D == 64 || D == 128 || D == 256, "unsupported head size");
  constexpr int NH = D / 64;
  constexpr int DT = D / 8;
  constexpr int VW = DT / 4;
  __shared__ __align__(16) int8_t q_hi[kPairs][D];
  __shared__ __align__(16) int8_t q_lo[kPairs][D];
  __shared__ float q_delta[kPairs];
  __shared__ float sm_ml[kWarps][kPairs][2];
  __shared__ float sm_L[kPairs];
  __shared__ int s_last;

  const int split = blockIdx.x, kvh = blockIdx.y, blk = blockIdx.z;
  const int nsplit = gridDim.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int G = p.G;
  const int seq = p.blk_seq[blk], row0 = p.blk_row0[blk], nrows = p.blk_nrows[blk], pos0 = p.blk_pos0[blk];
  const int npairs = nrows * G;                                   // <= 16
  const int len_max = pos0 + nrows;                               // keys seen by the block's last row
  const int first_min = (p.window > 0 && pos0 + 1 > p.window) ? (pos0 + 1 - p.window) : 0;   // first key of the first row
  const int page_lo = first_min / kPage;
  const int page_hi = (len_max + kPage - 1) / kPage;
  const int npages = page_hi - page_lo;
  const int pps = (npages + nsplit - 1) / nsplit;
  const int pbeg = page_lo + split * pps;
  const int pend = min(pbeg + pps, page_hi);
  const int* bt = p.block_table + (size_t)seq * p.max_pages;

  constexpr int STAGES = (D == 256) ? 3 : 4;
  constexpr int STAGE_BYTES = 2 * kPage * D + 128;
  constexpr int CPR = D / 16;
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

  // ---- q of every pair -> two int8 levels (warp w quantises pairs w, w + 4, w + 8, w + 12) ----
  for (int pr = warp; pr < kPairs; pr += kWarps) {
    float v[D / 32];
    float mx = 0.f;
    const bool valid = pr < npairs;
    const int r = pr / G, h = pr - r * G;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      v[i] = valid ? __bfloat162float(p.q[(size_t)(row0 + r) * p.ld_q + (size_t)(kvh * G + h) * D + lane + 32 * i]) * p.scale : 0.f;
      mx = fmaxf(mx, fabsf(v[i]));
    }
    mx = warp_max(mx);
    const float delta = mx > 0.f ? mx / 16256.f : 1.f;
    const float inv = 1.f / delta;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const int qi = __float2int_rn(v[i] * inv);
      const int hi = (qi + 64) >> 7;
      q_hi[pr][lane + 32 * i] = (int8_t)hi;
      q_lo[pr][lane + 32 * i] = (int8_t)(qi - 128 * hi);
    }
    if (lane == 0) q_delta[pr] = valid ? delta : 0.f;
  }
  __syncthreads();
  // A fragments: pair g in MMA rows 0..7, pair g + 8 in rows 8..15
  uint32_t qa_hi[NH][4], qa_lo[NH][4], qb_hi[NH][4], qb_lo[NH][4];
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    const uint4 a = *reinterpret_cast<const uint4*>(&q_hi[g][64 * h + 16 * t]);
    const uint4 b = *reinterpret_cast<const uint4*>(&q_lo[g][64 * h + 16 * t]);
    const uint4 c = *reinterpret_cast<const uint4*>(&q_hi[g + 8][64 * h + 16 * t]);
    const uint4 d = *reinterpret_cast<const uint4*>(&q_lo[g + 8][64 * h + 16 * t]);
    qa_hi[h][0] = a.x; qa_hi[h][1] = a.y; qa_hi[h][2] = a.z; qa_hi[h][3] = a.w;
    qa_lo[h][0] = b.x; qa_lo[h][1] = b.y; qa_lo[h][2] = b.z; qa_lo[h][3] = b.w;
    qb_hi[h][0] = c.x; qb_hi[h][1] = c.y; qb_hi[h][2] = c.z; qb_hi[h][3] = c.w;
    qb_lo[h][0] = d.x; qb_lo[h][1] = d.y; qb_lo[h][2] = d.z; qb_lo[h][3] = d.w;
  }
  // per pair: its scale, the keys it may see [first, len)
  float qd[2];
  int plen[2], pfirst[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int pr = g + 8 * u;
    const int r = pr / G;
    qd[u] = q_delta[pr];
    plen[u] = pr < npairs ? pos0 + r + 1 : 0;
    pfirst[u] = (p.window > 0 && plen[u] > p.window) ? plen[u] - p.window : 0;
  }

  float m_run[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f}, lv_part[2] = {0.f, 0.f};
  float o[DT][4];
#pragma unroll
  for (int j = 0; j < DT; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
  int pg = pbeg + warp;
#pragma unroll
  for (int s0 = 0; s0 < STAGES - 1; ++s0) issue(pg + s0 * kWarps, s0);
  int st = 0;
  for (; pg < pend; pg += kWarps) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncwarp();
    issue(pg + (STAGES - 1) * kWarps, (st + STAGES - 1) % STAGES);
    const uint8_t* sb = ring + st * STAGE_BYTES;
    st = (st + 1 == STAGES) ? 0 : st + 1;
    uint4 kreg[2][NH];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int h = 0; h < NH; ++h) kreg[nt][h] = *reinterpret_cast<const uint4*>(sb + k_off(8 * nt + g, 4 * h + t));
    float2 ksc[2], vsc[2];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      ksc[nt] = *reinterpret_cast<const float2*>(sb + 2 * kPage * D + 4 * (8 * nt + 2 * t));
      vsc[nt] = *reinterpret_cast<const float2*>(sb + 2 * kPage * D + 64 + 4 * (8 * nt + 2 * t));
    }
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
    // ---- S = Q K^T: c0, c1 = pair g x tokens (2t, 2t + 1) of the n8 tile, c2, c3 = pair g + 8 ----
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
          mma_s8_16832(s_hi[nt], qa_hi[h][2 * s], qb_hi[h][2 * s], qa_hi[h][2 * s + 1], qb_hi[h][2 * s + 1], kw[2 * s], kw[2 * s + 1]);
          mma_s8_16832(s_lo[nt], qa_lo[h][2 * s], qb_lo[h][2 * s], qa_lo[h][2 * s + 1], qb_lo[h][2 * s + 1], kw[2 * s], kw[2 * s + 1]);
        }
      }
    // ---- online softmax per pair over this lane's 4 tokens, quad reductions ----
    uint32_t pa[4];            // P as the A operand of PV: a0 / a2 = pair g (tokens 2t.., 2t + 8..), a1 / a3 = pair g + 8
    float alpha[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float sc[4];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int nt = i >> 1, c = i & 1;
        const int tok = pg * kPage + 8 * nt + 2 * t + c;
        const float ks = c ? ksc[nt].y : ksc[nt].x;
        const float sv = (float)(128 * s_hi[nt][2 * u + c] + s_lo[nt][2 * u + c]) * qd[u] * ks;
        sc[i] = (tok < plen[u] && tok >= pfirst[u]) ? sv : -INFINITY;
        mx = fmaxf(mx, sc[i]);
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mnew = fmaxf(m_run[u], mx);
      alpha[u] = (m_run[u] == -INFINITY) ? 0.f : __expf(m_run[u] - mnew);
      m_run[u] = mnew;
      float pv[4];
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pr = (sc[i] == -INFINITY) ? 0.f : __expf(sc[i] - mnew);
        psum += pr;
        pv[i] = pr * ((i & 1) ? vsc[i >> 1].y : vsc[i >> 1].x) * 1024.f;
      }
      pa[u] = pack_f16x2(pv[0], pv[1]);
      pa[2 + u] = pack_f16x2(pv[2], pv[3]);
      const float2 r0 = __half22float2(*reinterpret_cast<const __half2*>(&pa[u]));
      const float2 r2 = __half22float2(*reinterpret_cast<const __half2*>(&pa[2 + u]));
      l_part[u] = l_part[u] * alpha[u] + psum;
      lv_part[u] = lv_part[u] * alpha[u] + (r0.x + r0.y + r2.x + r2.y);
    }
    // ---- O = alpha O + P V ----
#pragma unroll
    for (int w = 0; w < VW; ++w) {
      const uint32_t lo01 = prmt(vraw[0][w], vraw[1][w], 0x5140u) ^ 0x80808080u, hi01 = prmt(vraw[0][w], vraw[1][w], 0x7362u) ^ 0x80808080u;
      const uint32_t lo89 = prmt(vraw[2][w], vraw[3][w], 0x5140u) ^ 0x80808080u, hi89 = prmt(vraw[2][w], vraw[3][w], 0x7362u) ^ 0x80808080u;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = 4 * w + e;
        const uint32_t src01 = e < 2 ? lo01 : hi01, src89 = e < 2 ? lo89 : hi89;
        const uint32_t sel = (e & 1) ? 0x4342u : 0x4140u;
        const uint32_t b0 = prmt(src01, 0x64646464u, sel), b1 = prmt(src89, 0x64646464u, sel);
        o[j][0] *= alpha[0]; o[j][1] *= alpha[0]; o[j][2] *= alpha[1]; o[j][3] *= alpha[1];
        mma_f16_16816(o[j], pa[0], pa[1], pa[2], pa[3], b0, b1);
      }
    }
  }

  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncwarp();
  // ---- this warp's result per pair: quad-reduce the sums, remove the 1152 bias, stage in the warp's own (now idle) ring ----
  float* so = reinterpret_cast<float*>(ring);              // [16 pairs][D]
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    l_part[u] += __shfl_xor_sync(0xffffffffu, l_part[u], 1);
    l_part[u] += __shfl_xor_sync(0xffffffffu, l_part[u], 2);
    lv_part[u] += __shfl_xor_sync(0xffffffffu, lv_part[u], 1);
    lv_part[u] += __shfl_xor_sync(0xffffffffu, lv_part[u], 2);
    const int pr = g + 8 * u;
    if (t == 0) { sm_ml[warp][pr][0] = m_run[u]; sm_ml[warp][pr][1] = l_part[u]; }
    const float bias = 1152.f * lv_part[u];
    float* dst = so + pr * D + t * (D / 4);
    const int rot = so_rot<D>(g, t);
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
      const int c = i / (DT / 4), j0 = 4 * (i % (DT / 4));
      float4 v4;
      v4.x = (o[j0][2 * u + c] - bias) * (1.f / 1024.f); v4.y = (o[j0 + 1][2 * u + c] - bias) * (1.f / 1024.f);
      v4.z = (o[j0 + 2][2 * u + c] - bias) * (1.f / 1024.f); v4.w = (o[j0 + 3][2 * u + c] - bias) * (1.f / 1024.f);
      *reinterpret_cast<float4*>(dst + 4 * ((i + rot) & (D / 16 - 1))) = v4;
    }
  }
  __syncthreads();

  const size_t pidx = ((size_t)blk * p.Hkv + kvh) * nsplit + split;
  for (int i = tid; i < npairs * D; i += kThreads) {
    const int pr = i / D, d = i % D;
    float M_ = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M_ = fmaxf(M_, sm_ml[w][pr][0]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float mw = sm_ml[w][pr][0];
      const float f = (mw == -INFINITY) ? 0.f : __expf(mw - M_);
      L += sm_ml[w][pr][1] * f;
      const float* wso = reinterpret_cast<const float*>(ring_raw + (size_t)w * STAGES * STAGE_BYTES);
      O += wso[pr * D + so_index<D>(pr & 7, d)] * f;
    }
    if (nsplit == 1) {
      float rv = L > 0.f ? O / L : 0.f;
      const int r = pr / G, h = pr - r * G;
      const size_t oi = (size_t)(row0 + r) * p.ld_o + (size_t)(kvh * G + h) * D + d;
      if (p.gate) rv *= sigmoid_f(__bfloat162float(p.gate[oi]));
      p.out[oi] = __float2bfloat16(rv);
    } else {
      p.part_o[(pidx * kPairs + pr) * D + d] = O;
      if (d == 0) { p.part_ml[(pidx * kPairs + pr) * 2] = M_; p.part_ml[(pidx * kPairs + pr) * 2 + 1] = L; }
    }
  }
  if (nsplit == 1) return;

  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int prev = atomicAdd(&p.counters[blk * p.Hkv + kvh], 1u);
    s_last = (prev == (unsigned int)nsplit - 1u);
    if (s_last) p.counters[blk * p.Hkv + kvh] = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // last CTA of this (block, kv head): merge the splits in split order
  const size_t base = ((size_t)blk * p.Hkv + kvh) * nsplit;
  float* wts = reinterpret_cast<float*>(ring_raw);        // [16][kMaxSplits]; every warp's staging has been consumed
  for (int i = tid; i < npairs * nsplit; i += kThreads) {
    const int pr = i / nsplit, sp = i % nsplit;
    wts[pr * kMaxSplits + sp] = __ldcg(&p.part_ml[((base + sp) * kPairs + pr) * 2]);
  }
  __syncthreads();
  if (tid < npairs) {
    float M_ = -INFINITY;
    for (int sp = 0; sp < nsplit; ++sp) M_ = fmaxf(M_, wts[tid * kMaxSplits + sp]);
    float L = 0.f;
    for (int sp = 0; sp < nsplit; ++sp) {
      const float ms = wts[tid * kMaxSplits + sp];
      const float f = (ms == -INFINITY) ? 0.f : __expf(ms - M_);
      wts[tid * kMaxSplits + sp] = f;
      L += __ldcg(&p.part_ml[((base + sp) * kPairs + tid) * 2 + 1]) * f;
    }
    sm_L[tid] = L;
  }
  __syncthreads();
  for (int i = tid; i < npairs * D / 4; i += kThreads) {
    const int pr = i / (D / 4), d = 4 * (i % (D / 4));
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int sp = 0; sp < nsplit; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(&p.part_o[((base + sp) * kPairs + pr) * D + d]));
      const float w = wts[pr * kMaxSplits + sp];
      O.x = fmaf(v.x, w, O.x); O.y = fmaf(v.y, w, O.y); O.z = fmaf(v.z, w, O.z); O.w = fmaf(v.w, w, O.w);
    }
    const float L = sm_L[pr];
    const float inv = L > 0.f ? 1.f / L : 0.f;
    float rv[4] = {O.x * inv, O.y * inv, O.z * inv, O.w * inv};
    const int r = pr / G, h = pr - r * G;
    const size_t oi = (size_t)(row0 + r) * p.ld_o + (size_t)(kvh * G + h) * D + d;
    if (p.gate) {
#pragma unroll
      for (int c = 0; c < 4; ++c) rv[c] *= sigmoid_f(__bfloat162float(p.gate[oi + c]));
    }
    uint2 o2;
    o2.x = pack_bf16x2(rv[0], rv[1]); o2.y = pack_bf16x2(rv[2], rv[3]);
    *reinterpret_cast<uint2*>(p.out + oi) = o2;
  }
}

template <int D>
int launch(const VerParams& p, int splits, int blocks, cudaStream_t st) {
  dim3 grid(splits, p.Hkv, blocks);
  constexpr int kRing = kWarps * ((D == 256) ? 3 : 4) * (2 * kPage * D + 128);
  static_assert(kRing / kWarps >= kPairs * D * 4, "a warp's ring must hold its 16 x D staging");
  static_assert(kRing >= kPairs * kMaxSplits * 4, "the ring must hold the merge weights");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(verify_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  verify_attn_kernel<D><<<grid, kThreads, kRing, st>>>(p);
  GRM_LAUNCH_RET();
}

}  // namespace

// Rows per grid entry for a head split (floor(16 / G)).
GRM_API int grm_verify_attn_rows_per_group(int Hq, int Hkv) {
  if (Hkv < 1 || Hq % Hkv) return 0;
  const int G = Hq / Hkv;
  return G > 16 ? 0 : 16 / G;
}

// blocks groups of rows (blk_* arrays on the device, one entry per group): rows blk_row0 .. + blk_nrows of q / out are the
// consecutive positions blk_pos0 .. of sequence blk_seq; blk_nrows <= grm_verify_attn_rows_per_group().  K / V of those
// positions must already be in the cache.  part_o: blocks * Hkv * splits * 16 * D floats, part_ml: ... * 16 * 2 floats,
// counters: blocks * Hkv zeroed uints (only used when splits > 1).
GRM_API int grm_paged_verify_attn(const void* q, int ld_q, const void* blk_seq, const void* blk_row0, const void* blk_nrows,
                                  const void* blk_pos0, int blocks, const void* block_table, int max_pages, const void* k_pages,
                                  const void* v_pages, const void* k_scale, const void* v_scale, const void* gate, void* out, int ld_o,
                                  void* part_o, void* part_ml, void* counters, int Hq, int Hkv, int D, int splits, int window,
                                  float scale, void* stream) {
  if (blocks < 1 || Hkv < 1 || Hq % Hkv || Hq / Hkv > 16 || splits < 1 || splits > kMaxSplits || (ld_o & 3)) return -2;
  if (splits > 1 && (!part_o || !part_ml || !counters)) return -2;
  VerParams p;
  p.q = (const bf16*)q; p.ld_q = ld_q;
  p.blk_seq = (const int*)blk_seq; p.blk_row0 = (const int*)blk_row0; p.blk_nrows = (const int*)blk_nrows; p.blk_pos0 = (const int*)blk_pos0;
  p.block_table = (const int*)block_table; p.max_pages = max_pages;
  p.k_pages = (const int8_t*)k_pages; p.v_pages = (const int8_t*)v_pages; p.k_scale = (const float*)k_scale; p.v_scale = (const float*)v_scale;
  p.gate = (const bf16*)gate; p.out = (bf16*)out; p.ld_o = ld_o;
  p.part_o = (float*)part_o; p.part_ml = (float*)part_ml; p.counters = (unsigned int*)counters;
  p.Hq = Hq; p.Hkv = Hkv; p.G = Hq / Hkv; p.window = window; p.scale = scale;
  cudaStream_t st = (cudaStream_t)stream;
  switch (D) {
    case 64: return launch<64>(p, splits, blocks, st);
    case 128: return launch<128>(p, splits, blocks, st);
    case 256: return launch<256>(p, splits, blocks, st);
    default: return -2;
  }
}
