// qk_norm_rope_kvwrite_i8: one pass over the fused q|k|v projection output that
//   * splits q (and the per-head output gate of gated attention: q_proj rows are [q | gate] per head),
//   * applies the optional per-head RMSNorm to q and k BEFORE RoPE,
//   * applies NeoX half-split RoPE over the first `rot` dims (partial rotary),
//   * writes q (bf16) for the attention kernel, optionally roped k / v in bf16 for prefill attention,
//   * quantizes k and v to int8 with one fp32 scale per (token, kv head) = max|x|/127 and stores them
//     in 16-token pages through the block table.
// Replaces the reference's launch_split_qgate + launch_qk_norm_rope(_batched) + launch_kv_append* +
// kv_append_k8 chain (src/ops.cpp:870-941,996,1551; src/prefill.cpp:1262-1533; src/kv_k8.hpp:19-59).
// Unlike the reference's opt-in int8 K, both K and V are int8 here.
//
// Page layout (per layer):  k_pages/v_pages int8 [pages][Hkv][16][D];  k_scale/v_scale fp32 [pages][Hkv][16].
// One warp per (row, head); D <= 256, D % 32 == 0, rot % 64 == 0 so a rotation pair lives in one lane.
#include "common.cuh"

namespace {

struct RopeKvParams {
  const bf16* qkv; int ld_qkv;
  const int* row_pos;        // [M] absolute position of each row
  const int* row_seq;        // [M] sequence index into the block table (null: no cache write)
  const int* block_table;    // [S][max_pages]
  int max_pages;
  const float* inv_freq;     // [rot/2]
  const float* q_norm_w;     // [D] or null
  const float* k_norm_w;     // [D] or null
  float norm_eps, norm_offset;
  bf16* q_out; int ld_q;     // [M][Hq*D]
  bf16* gate_out;            // [M][Hq*D] or null (q_gated)
  bf16* k_out; bf16* v_out; int ld_kv;   // [M][Hkv*D] or null
  int8_t* k_pages; int8_t* v_pages; float* k_scale; float* v_scale;
  int M, Hq, Hkv, D, rot, q_gated;
  int dense_pos0;            // >= 0: dense k / v rows are indexed by row_pos[row] - dense_pos0 instead of by row
  int q_row0, q_rows;        // q (and gate) are produced for rows [q_row0, q_row0 + q_rows) only (q_rows < 0: every row)
};

constexpr int kPage = 16;

__global__ void __launch_bounds__(256) rope_kv_kernel(const RopeKvParams p) {
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int heads = p.Hq + 2 * p.Hkv;
  if (wid >= p.M * heads) return;
  const int row = wid / heads, hd = wid % heads;
  const int D = p.D, per = D >> 5;
  const int qstride = p.q_gated ? 2 * D : D;
  const bf16* src;
  int kind;  // 0 q, 1 k, 2 v
  int h;
  if (hd < p.Hq && p.q_rows >= 0 && (row < p.q_row0 || row >= p.q_row0 + p.q_rows)) return;
  if (hd < p.Hq) { kind = 0; h = hd; src = p.qkv + (size_t)row * p.ld_qkv + (size_t)h * qstride; }
  else if (hd < p.Hq + p.Hkv) { kind = 1; h = hd - p.Hq; src = p.qkv + (size_t)row * p.ld_qkv + (size_t)p.Hq * qstride + (size_t)h * D; }
  else { kind = 2; h = hd - p.Hq - p.Hkv; src = p.qkv + (size_t)row * p.ld_qkv + (size_t)p.Hq * qstride + (size_t)(p.Hkv + h) * D; }

  float v[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = (i < per) ? __bfloat162float(src[lane + 32 * i]) : 0.f;

  if (kind == 0 && p.q_gated && p.gate_out) {
    for (int i = 0; i < per; ++i)
      p.gate_out[(size_t)row * p.ld_q + (size_t)h * D + lane + 32 * i] = src[D + lane + 32 * i];
  }

  if (kind != 2) {
    const float* nw = kind == 0 ? p.q_norm_w : p.k_norm_w;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)D + p.norm_eps);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < per) {
          // the reference norms in fp32 and rounds once at the end; keep that
          v[i] = v[i] * r * (p.norm_offset + nw[lane + 32 * i]);
        }
    }
    const int half = p.rot >> 1, hreg = half >> 5;   // registers per half
    const float pos = (float)p.row_pos[row];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (i < hreg) {
        const float ang = pos * p.inv_freq[lane + 32 * i];
        float sn, cs;
        sincosf(ang, &sn, &cs);
        const float a = v[i], b = v[i + hreg];
        v[i] = a * cs - b * sn;
        v[i + hreg] = b * cs + a * sn;
      }
    }
  }

  if (kind == 0) {
    for (int i = 0; i < per; ++i) p.q_out[(size_t)row * p.ld_q + (size_t)h * D + lane + 32 * i] = __float2bfloat16(v[i]);
    return;
  }
  bf16* dense = kind == 1 ? p.k_out : p.v_out;
  if (dense) {
    const int drow = p.dense_pos0 >= 0 ? p.row_pos[row] - p.dense_pos0 : row;
    if (drow >= 0)
      for (int i = 0; i < per; ++i) dense[(size_t)drow * p.ld_kv + (size_t)h * D + lane + 32 * i] = __float2bfloat16(v[i]);
  }
  if (!p.row_seq || !p.k_pages) return;
  const int seq = p.row_seq[row];
  if (seq < 0) return;
  const int pos = p.row_pos[row];
  const int page = p.block_table[(size_t)seq * p.max_pages + pos / kPage];
  if (page < 0) return;
  const int slot = pos % kPage;
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax / 127.f : 1.f;
  const float inv = 1.f / scale;
  int8_t* dst = (kind == 1 ? p.k_pages : p.v_pages) + (((size_t)page * p.Hkv + h) * kPage + slot) * D;
  for (int i = 0; i < per; ++i) {
    const int q = max(-127, min(127, __float2int_rn(v[i] * inv)));
    dst[lane + 32 * i] = (int8_t)q;
  }
  if (lane == 0) (kind == 1 ? p.k_scale : p.v_scale)[((size_t)page * p.Hkv + h) * kPage + slot] = scale;
}

// pages -> contiguous bf16 [T][Hkv][D] for one sequence (earlier chunks of a chunked prefill are
// re-read through this pre-pass, as the reference converts its FP8 cache to bf16 operands before
// flash prefill: src/gemm_fast.cpp flash pre-pass).
__global__ void kv_gather_dequant_kernel(const int8_t* __restrict__ pages, const float* __restrict__ scales,
                                         const int* __restrict__ block_table, bf16* __restrict__ out, int T, int Hkv, int D,
                                         int ld_out) {
  const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (wid >= T * Hkv) return;
  const int tok = wid / Hkv, h = wid % Hkv;
  const int page = block_table[tok / kPage], slot = tok % kPage;
  const size_t base = ((size_t)page * Hkv + h) * kPage + slot;
  const float s = scales[base];
  const int8_t* src = pages + base * D;
  for (int d = lane; d < D; d += 32) out[(size_t)tok * ld_out + h * D + d] = __float2bfloat16((float)src[d] * s);
}

}  // namespace

// Extended form: dense_pos0 >= 0 writes the dense k / v row of a token at index row_pos - dense_pos0 (rows may then come in any
// order; the caller guarantees row_pos - dense_pos0 < the dense buffers' height); q_rows >= 0 limits q / gate to rows
// [q_row0, q_row0 + q_rows) (context-parallel prefill: the other rows' queries belong to other ranks).
GRM_API int grm_rope_kvwrite_ex(const void* qkv, int ld_qkv, const void* row_pos, const void* row_seq, const void* block_table,
                             int max_pages, const void* inv_freq, const void* q_norm_w, const void* k_norm_w, float norm_eps,
                             float norm_offset, void* q_out, int ld_q, void* gate_out, void* k_out, void* v_out, int ld_kv,
                             void* k_pages, void* v_pages, void* k_scale, void* v_scale, int M, int Hq, int Hkv, int D, int rot,
                             int q_gated, int dense_pos0, int q_row0, int q_rows, void* stream) {
  if ((D & 31) || D > 256 || (rot & 63) || rot > D || M < 1) return -2;
  RopeKvParams p;
  p.qkv = (const bf16*)qkv; p.ld_qkv = ld_qkv; p.row_pos = (const int*)row_pos; p.row_seq = (const int*)row_seq;
  p.block_table = (const int*)block_table; p.max_pages = max_pages; p.inv_freq = (const float*)inv_freq;
  p.q_norm_w = (const float*)q_norm_w; p.k_norm_w = (const float*)k_norm_w; p.norm_eps = norm_eps; p.norm_offset = norm_offset;
  p.q_out = (bf16*)q_out; p.ld_q = ld_q; p.gate_out = (bf16*)gate_out; p.k_out = (bf16*)k_out; p.v_out = (bf16*)v_out; p.ld_kv = ld_kv;
  p.k_pages = (int8_t*)k_pages; p.v_pages = (int8_t*)v_pages; p.k_scale = (float*)k_scale; p.v_scale = (float*)v_scale;
  p.M = M; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.rot = rot; p.q_gated = q_gated;
  p.dense_pos0 = dense_pos0; p.q_row0 = q_row0; p.q_rows = q_rows;
  const long warps = (long)M * (Hq + 2 * Hkv);
  const int threads = 256;
  const long blocks = (warps * 32 + threads - 1) / threads;
  rope_kv_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(p);
  GRM_LAUNCH_RET();
}

GRM_API int grm_rope_kvwrite(const void* qkv, int ld_qkv, const void* row_pos, const void* row_seq, const void* block_table,
                             int max_pages, const void* inv_freq, const void* q_norm_w, const void* k_norm_w, float norm_eps,
                             float norm_offset, void* q_out, int ld_q, void* gate_out, void* k_out, void* v_out, int ld_kv,
                             void* k_pages, void* v_pages, void* k_scale, void* v_scale, int M, int Hq, int Hkv, int D, int rot,
                             int q_gated, void* stream) {
  return grm_rope_kvwrite_ex(qkv, ld_qkv, row_pos, row_seq, block_table, max_pages, inv_freq, q_norm_w, k_norm_w, norm_eps, norm_offset,
                             q_out, ld_q, gate_out, k_out, v_out, ld_kv, k_pages, v_pages, k_scale, v_scale, M, Hq, Hkv, D, rot, q_gated,
                             -1, 0, -1, stream);
}

GRM_API int grm_kv_gather_dequant(const void* pages, const void* scales, const void* block_table, void* out, int T, int Hkv,
                                  int D, int ld_out, void* stream) {
  if (T < 1) return 0;
  const long warps = (long)T * Hkv;
  const int threads = 256;
  const long blocks = (warps * 32 + threads - 1) / threads;
  kv_gather_dequant_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>((const int8_t*)pages, (const float*)scales,
                                                                                 (const int*)block_table, (bf16*)out, T, Hkv, D, ld_out);
  GRM_LAUNCH_RET();
}
