"""Python wrappers of the non-GEMM kernels: norms, RoPE + paged int8 KV write, paged decode /
verify attention, flash prefill, embedding, arg-max.  Each function runs the sm_100a kernel for
CUDA tensors and the fp32 PyTorch reference (``ops.ref``) for CPU tensors; on a CUDA tensor a
missing native library raises instead of falling back.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import _native
from . import ref
from .workspace import Workspace

PAGE = 16
# tcgen05 flash prefill for head_dim 128 (GRIMOIRE_FLASH_TC=0 selects the warp-MMA kernel)
FLASH_TC = os.environ.get("GRIMOIRE_FLASH_TC", "1") != "0"


def _c(v):
    return ctypes.c_int(int(v))


def _f(v):
    return ctypes.c_float(float(v))


# ---------------------------------------------------------------------------------------------
# norms
# ---------------------------------------------------------------------------------------------
def add_rmsnorm(h: torch.Tensor, w: torch.Tensor, x_out: torch.Tensor, eps: float, offset: float,
                delta: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``h += delta`` (optional, fp32 or bf16); ``x_out = rms(h) * (offset + w)`` as bf16.

    h: fp32 [M][H] residual stream, updated in place.  Reference: launch_rmsnorm_residual*
    (src/ops.cpp:205-313)."""
    M, H = h.shape
    if not h.is_cuda:
        if delta is not None:
            h.add_(delta.float())
        x_out.copy_(ref.rmsnorm(h, w, eps, offset).to(x_out.dtype))
        return x_out
    dd = 0 if delta is None else (1 if delta.dtype == torch.float32 else 2)
    x16 = x_out if x_out.dtype == torch.bfloat16 else None
    x32 = x_out if x_out.dtype == torch.float32 else None
    code = _native.cuda().grm_add_rmsnorm(_native.ptr(h), _native.ptr(delta), _c(dd), _native.ptr(w), _native.ptr(x16),
                                          _native.ptr(x32), _c(M), _c(H), _c(h.stride(0)),
                                          _c(delta.stride(0) if delta is not None else 0), _c(x_out.stride(0)), _f(eps),
                                          _f(offset), _native.stream_ptr())
    _native.check(code, "add_rmsnorm")
    return x_out


def rmsnorm_heads(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, heads: int, D: int, eps: float, offset: float,
                  z: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Per-head RMSNorm (fp32 in, bf16 out) with optional ``* silu(z)`` (GDN gated output norm)."""
    rows = x.shape[0]
    if not x.is_cuda:
        y = ref.head_rmsnorm(x.float().reshape(rows, heads, D), w, eps, offset)
        if z is not None:
            y = y * torch.nn.functional.silu(z.float().reshape(rows, heads, D))
        out.copy_(y.reshape(rows, heads * D).to(out.dtype))
        return out
    code = _native.cuda().grm_rmsnorm_heads(_native.ptr(x), _native.ptr(z), _native.ptr(w), _native.ptr(out), _c(rows),
                                            _c(heads), _c(D), _c(x.stride(0)), _c(z.stride(0) if z is not None else 0),
                                            _c(out.stride(0)), _f(eps), _f(offset), _native.stream_ptr())
    _native.check(code, "rmsnorm_heads")
    return out


# ---------------------------------------------------------------------------------------------
# paged int8 KV cache (one layer)
# ---------------------------------------------------------------------------------------------
@dataclass
class KvLayer:
    """int8 K/V pages of one layer: pages [P][Hkv][16][D] int8, scales [P][Hkv][16] fp32."""

    k: torch.Tensor
    v: torch.Tensor
    ks: torch.Tensor
    vs: torch.Tensor

    @staticmethod
    def alloc(pages: int, Hkv: int, D: int, device) -> "KvLayer":
        mk = lambda *s, dt: torch.zeros(*s, dtype=dt, device=device)
        return KvLayer(mk(pages, Hkv, PAGE, D, dt=torch.int8), mk(pages, Hkv, PAGE, D, dt=torch.int8),
                       mk(pages, Hkv, PAGE, dt=torch.float32), mk(pages, Hkv, PAGE, dt=torch.float32))

    def bytes_per_token(self) -> int:
        Hkv, D = self.k.shape[1], self.k.shape[3]
        return 2 * Hkv * D + 2 * Hkv * 4


@dataclass
class AttnGeom:
    Hq: int
    Hkv: int
    D: int
    rot: int
    scale: float
    q_gated: bool = False
    window: int = 0
    norm_eps: float = 1e-6
    norm_offset: float = 0.0


def rope_kvwrite(qkv: torch.Tensor, row_pos: torch.Tensor, row_seq: Optional[torch.Tensor],
                 block_table: Optional[torch.Tensor], inv_freq: torch.Tensor, geom: AttnGeom, q_out: torch.Tensor,
                 kv: Optional[KvLayer], q_norm_w=None, k_norm_w=None, gate_out=None, k_out=None, v_out=None,
                 dense_pos0: int = -1, q_rows: Optional[tuple] = None):
    """Split the fused q|k|v rows, q/k norm, RoPE, write q (bf16) and int8 K/V pages (+ dense bf16
    K/V for the prefill attention of the current chunk).  See rope_kv.cu.  ``dense_pos0`` >= 0: the dense K / V row of a
    token lands at index ``row_pos - dense_pos0`` (rows in any order); ``q_rows`` = (first, count): q / gate are produced
    for those rows only (the other rows of ``q_out`` are left as they are)."""
    M = qkv.shape[0]
    Hq, Hkv, D = geom.Hq, geom.Hkv, geom.D
    if not qkv.is_cuda:
        qs = 2 * D if geom.q_gated else D
        x = qkv.float()
        qg = x[:, : Hq * qs].reshape(M, Hq, qs)
        q = qg[..., :D]
        if geom.q_gated and gate_out is not None:
            gate_out.copy_(qg[..., D:].reshape(M, Hq * D).to(gate_out.dtype))
        k = x[:, Hq * qs: Hq * qs + Hkv * D].reshape(M, Hkv, D)
        v = x[:, Hq * qs + Hkv * D:].reshape(M, Hkv, D)
        q = ref.head_rmsnorm(q, q_norm_w, geom.norm_eps, geom.norm_offset)
        k = ref.head_rmsnorm(k, k_norm_w, geom.norm_eps, geom.norm_offset)
        q = ref.apply_rope(q, row_pos, inv_freq, geom.rot)
        k = ref.apply_rope(k, row_pos, inv_freq, geom.rot)
        q_out.copy_(q.reshape(M, Hq * D).to(q_out.dtype))
        if k_out is not None and dense_pos0 >= 0:
            idx = (row_pos.long() - dense_pos0)
            k_out[idx] = k.reshape(M, Hkv * D).to(k_out.dtype)
            v_out[idx] = v.reshape(M, Hkv * D).to(v_out.dtype)
        elif k_out is not None:
            k_out.copy_(k.reshape(M, Hkv * D).to(k_out.dtype))
            v_out.copy_(v.reshape(M, Hkv * D).to(v_out.dtype))
        if kv is not None and row_seq is not None:
            kq, ksc = ref.quant_i8_rows(k)
            vq, vsc = ref.quant_i8_rows(v)
            for m in range(M):
                s, p = int(row_seq[m]), int(row_pos[m])
                if s < 0:
                    continue
                page = int(block_table[s, p // PAGE])
                if page < 0:
                    continue
                kv.k[page, :, p % PAGE] = kq[m]
                kv.v[page, :, p % PAGE] = vq[m]
                kv.ks[page, :, p % PAGE] = ksc[m]
                kv.vs[page, :, p % PAGE] = vsc[m]
        return q_out
    lib = _native.cuda()
    code = lib.grm_rope_kvwrite_ex(
        _native.ptr(qkv), _c(qkv.stride(0)), _native.ptr(row_pos), _native.ptr(row_seq), _native.ptr(block_table),
        _c(block_table.stride(0) if block_table is not None else 0), _native.ptr(inv_freq), _native.ptr(q_norm_w),
        _native.ptr(k_norm_w), _f(geom.norm_eps), _f(geom.norm_offset), _native.ptr(q_out), _c(q_out.stride(0)),
        _native.ptr(gate_out), _native.ptr(k_out), _native.ptr(v_out), _c(k_out.stride(0) if k_out is not None else 0),
        _native.ptr(kv.k if kv else None), _native.ptr(kv.v if kv else None), _native.ptr(kv.ks if kv else None),
        _native.ptr(kv.vs if kv else None), _c(M), _c(Hq), _c(Hkv), _c(D), _c(geom.rot), _c(1 if geom.q_gated else 0),
        _c(dense_pos0), _c(q_rows[0] if q_rows else 0), _c(q_rows[1] if q_rows else -1), _native.stream_ptr())
    _native.check(code, "rope_kvwrite")
    return q_out


def gather_kv_dense(kv: KvLayer, pages_of_seq: torch.Tensor, T: int, out_k: torch.Tensor, out_v: torch.Tensor):
    """Dequantize the first T cached tokens of one sequence into dense bf16 [T][Hkv*D] buffers."""
    Hkv, D = kv.k.shape[1], kv.k.shape[3]
    if T <= 0:
        return
    if not kv.k.is_cuda:
        for name, pages, scales, out in (("k", kv.k, kv.ks, out_k), ("v", kv.v, kv.vs, out_v)):
            npg = (T + PAGE - 1) // PAGE
            idx = pages_of_seq[:npg].long()
            d = pages[idx].float() * scales[idx][..., None]           # [npg][Hkv][16][D]
            d = d.permute(0, 2, 1, 3).reshape(npg * PAGE, Hkv * D)[:T]
            out[:T].copy_(d.to(out.dtype))
        return
    lib = _native.cuda()
    for pages, scales, out in ((kv.k, kv.ks, out_k), (kv.v, kv.vs, out_v)):
        code = lib.grm_kv_gather_dequant(_native.ptr(pages), _native.ptr(scales), _native.ptr(pages_of_seq), _native.ptr(out),
                                         _c(T), _c(Hkv), _c(D), _c(out.stride(0)), _native.stream_ptr())
        _native.check(code, "kv_gather_dequant")


def decode_splits(max_len: int, M: int, Hkv: int) -> int:
    """Split-KV factor.  Measured on 148 SMs (one row, 8 kv heads, us per launch at 16 / 32 splits: context 4096 11.6 / 14.2,
    8192 15.3 / 16.9, 16384 21.7 / 20.5, 32768 34.4 / 27.0): up to 16 splits merge through cluster shared memory and
    want at least 8 pages (2 per warp) each; more than 16 fall back to the scratch merge, which only pays from 32 pages
    per split; about 256 CTAs in total at most."""
    pages = max(1, (max_len + PAGE - 1) // PAGE)
    want = max(1, 256 // max(1, M * Hkv))
    cap = int(max(1, min(want, pages // 8 if pages >= 8 else 1, 64)))
    s = 1
    while s * 2 <= cap:     # powers of two only: the decode graphs are keyed by (rows, splits)
        s *= 2
    if s > 16 and pages // s < 32:
        s = 16
    return s


def paged_decode_attn(q: torch.Tensor, row_seq: torch.Tensor, row_pos: torch.Tensor, block_table: torch.Tensor,
                      kv: KvLayer, geom: AttnGeom, out: torch.Tensor, splits: int, ws: Optional[Workspace],
                      gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of M (sequence, position) rows over the paged int8 cache; see attn_decode.cu."""
    M = q.shape[0]
    Hq, Hkv, D = geom.Hq, geom.Hkv, geom.D
    if not q.is_cuda:
        for m in range(M):
            s, p = int(row_seq[m]), int(row_pos[m])
            T = p + 1
            npg = (T + PAGE - 1) // PAGE
            idx = block_table[s, :npg].long()
            kd = (kv.k[idx].float() * kv.ks[idx][..., None]).permute(0, 2, 1, 3).reshape(npg * PAGE, Hkv, D)[:T]
            vd = (kv.v[idx].float() * kv.vs[idx][..., None]).permute(0, 2, 1, 3).reshape(npg * PAGE, Hkv, D)[:T]
            o = ref.attention_rows(q[m: m + 1].float().reshape(1, Hq, D), kd, vd, torch.tensor([p]), geom.scale,
                                   geom.window).reshape(Hq * D)
            if gate is not None:
                o = o * torch.sigmoid(gate[m].float())
            out[m].copy_(o.to(out.dtype))
        return out
    part_o = part_ml = counters = None
    if splits > 1:
        part_o = ws.get("attn_part_o", M * Hq * splits * D, torch.float32)
        part_ml = ws.get("attn_part_ml", M * Hq * splits * 2, torch.float32)
        counters = ws.get("attn_counters", 4096, torch.int32, zero=True)
        if M * Hkv > 4096:
            raise ValueError("too many (row, kv head) pairs for the attention counters")
    code = _native.cuda().grm_paged_decode_attn(
        _native.ptr(q), _c(q.stride(0)), _native.ptr(row_seq), _native.ptr(row_pos), _native.ptr(block_table),
        _c(block_table.stride(0)), _native.ptr(kv.k), _native.ptr(kv.v), _native.ptr(kv.ks), _native.ptr(kv.vs),
        _native.ptr(gate), _native.ptr(out), _c(out.stride(0)), _native.ptr(part_o), _native.ptr(part_ml),
        _native.ptr(counters), _c(M), _c(Hq), _c(Hkv), _c(D), _c(splits), _c(geom.window), _f(geom.scale),
        _native.stream_ptr())
    _native.check(code, "paged_decode_attn")
    return out


FUSED_ROPE_ATTN = os.environ.get("GRIMOIRE_FUSED_ROPE_ATTN", "1") != "0"
# programmatic dependent launch of the decode kernels (a kernel's weight / KV prefetch overlaps its predecessor's tail)
PDL = int(os.environ.get("GRIMOIRE_PDL", "6"))       # mask: 1 GEMV, 2 attention, 4 attention KV prefetch, 8 embed / token pick
_pdl_applied = False


def apply_pdl_switch() -> None:
    """Hand GRIMOIRE_PDL to the kernel library once (the library's default is on)."""
    global _pdl_applied
    if not _pdl_applied and _native.cuda_available():
        _native.cuda().grm_set_pdl(ctypes.c_int(PDL))
        _pdl_applied = True


def paged_decode_attn_fused(qkv: torch.Tensor, inv_freq: torch.Tensor, q_norm_w, k_norm_w, row_seq: torch.Tensor,
                            row_pos: torch.Tensor, block_table: torch.Tensor, kv: KvLayer, geom: AttnGeom, out: torch.Tensor,
                            splits: int, ws: Optional[Workspace], prefetch: bool = False) -> bool:
    """``rope_kvwrite`` + ``paged_decode_attn`` in one launch for rows of different sequences (ungated q): the kernel
    norms / rotates q itself and the CTA that reads a row's last page appends the row's K / V first.  Returns False
    when the case is not served (CPU tensors, gated q, switch off); the caller then runs the two kernels.  ``prefetch``:
    the launch right before this one is the projection that writes ``qkv`` and nothing else this kernel reads, so the
    kernel may fetch the pages of earlier tokens while that launch is still running."""
    if not (qkv.is_cuda and FUSED_ROPE_ATTN) or geom.q_gated or geom.rot < 64:
        return False
    apply_pdl_switch()
    M = qkv.shape[0]
    Hq, Hkv, D = geom.Hq, geom.Hkv, geom.D
    part_o = part_ml = counters = None
    if splits > 1:
        part_o = ws.get("attn_part_o", M * Hq * splits * D, torch.float32)
        part_ml = ws.get("attn_part_ml", M * Hq * splits * 2, torch.float32)
        counters = ws.get("attn_counters", 4096, torch.int32, zero=True)
        if M * Hkv > 4096:
            return False
    code = _native.cuda().grm_paged_decode_attn_fused(
        _native.ptr(qkv), _c(qkv.stride(0)), _native.ptr(inv_freq), _native.ptr(q_norm_w), _native.ptr(k_norm_w), _f(geom.norm_eps),
        _f(geom.norm_offset), _c(geom.rot), _native.ptr(row_seq), _native.ptr(row_pos), _native.ptr(block_table),
        _c(block_table.stride(0)), _native.ptr(kv.k), _native.ptr(kv.v), _native.ptr(kv.ks), _native.ptr(kv.vs), _native.ptr(out),
        _c(out.stride(0)), _native.ptr(part_o), _native.ptr(part_ml), _native.ptr(counters), _c(M), _c(Hq), _c(Hkv), _c(D), _c(splits),
        _c(geom.window), _f(geom.scale), _c(1 if prefetch else 0), _native.stream_ptr())
    if code == -2:
        return False
    _native.check(code, "paged_decode_attn_fused")
    return True


VERIFY_ATTN = os.environ.get("GRIMOIRE_VERIFY_ATTN", "1") != "0"     # verify blocks: (row, head) pairs in the MMA rows
# context length from which verify blocks take the one-pass kernel (measured, 4 rows of the 40 / 8 head split, one pass
# against row by row: 4,096 tokens 23.3 / 17.9 us, 8,192 23.8 / 25.5, 32,768 49.2 / 65.6, 65,536 84.0 / 122.5); below it the
# rows are scored one by one with exactly the arithmetic of single-row steps
VERIFY_ATTN_MIN_CTX = int(os.environ.get("GRIMOIRE_VERIFY_ATTN_MIN_CTX", "8192"))


def verify_rows_per_group(geom: AttnGeom) -> int:
    """Rows of one verify block that share a pass over the cache (floor(16 / G), attn_verify.cu)."""
    G = geom.Hq // geom.Hkv
    return 16 // G if G <= 16 else 0


def verify_groups(slots: Sequence[int], positions: Sequence[int], per: int):
    """Cut the rows of a step into groups for ``paged_verify_attn``: maximal runs of consecutive positions of one
    sequence, at most ``per`` rows each.  Returns lists (slot, first row, rows, first position)."""
    out = []
    i, M = 0, len(slots)
    while i < M:
        n = 1
        while i + n < M and n < per and slots[i + n] == slots[i] and positions[i + n] == positions[i] + n:
            n += 1
        out.append((int(slots[i]), i, n, int(positions[i])))
        i += n
    return out


def paged_verify_attn(q: torch.Tensor, blocks: torch.Tensor, nblocks: int, block_table: torch.Tensor, kv: KvLayer, geom: AttnGeom,
                      out: torch.Tensor, splits: int, ws: Workspace, gate: Optional[torch.Tensor] = None) -> bool:
    """Attention of verify blocks in one pass over the pages per group of rows (attn_verify.cu; launch_verify_attn_dpas,
    src/attn_verify.hpp:48-69).  ``blocks`` is an int32 device tensor [4][>= nblocks]: sequence slot, first row, rows,
    first position of every group (``verify_groups``).  K / V of the rows must already be in the cache.  Returns False
    when the case is not served (CPU tensors, switch off); the caller then runs the per-row kernel."""
    if not (q.is_cuda and VERIFY_ATTN) or verify_rows_per_group(geom) < 1:
        return False
    Hq, Hkv, D = geom.Hq, geom.Hkv, geom.D
    part_o = part_ml = counters = None
    if splits > 1:
        part_o = ws.get("vattn_part_o", nblocks * Hkv * splits * 16 * D, torch.float32)
        part_ml = ws.get("vattn_part_ml", nblocks * Hkv * splits * 16 * 2, torch.float32)
        counters = ws.get("vattn_counters", 4096, torch.int32, zero=True)
        if nblocks * Hkv > 4096:
            return False
    code = _native.cuda().grm_paged_verify_attn(
        _native.ptr(q), _c(q.stride(0)), _native.ptr(blocks[0]), _native.ptr(blocks[1]), _native.ptr(blocks[2]), _native.ptr(blocks[3]),
        _c(nblocks), _native.ptr(block_table), _c(block_table.stride(0)), _native.ptr(kv.k), _native.ptr(kv.v), _native.ptr(kv.ks),
        _native.ptr(kv.vs), _native.ptr(gate), _native.ptr(out), _c(out.stride(0)), _native.ptr(part_o), _native.ptr(part_ml),
        _native.ptr(counters), _c(Hq), _c(Hkv), _c(D), _c(splits), _c(geom.window), _f(geom.scale), _native.stream_ptr())
    if code == -2:
        return False
    _native.check(code, "paged_verify_attn")
    return True


def flash_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, geom: AttnGeom, out: torch.Tensor, q_pos0: int,
                  gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal attention of one sequence's M new rows over its T = q_pos0 + M dense bf16 keys."""
    M = q.shape[0]
    T = q_pos0 + M
    Hq, Hkv, D = geom.Hq, geom.Hkv, geom.D
    if not q.is_cuda:
        o = ref.attention_rows(q.float().reshape(M, Hq, D), k[:T].float().reshape(T, Hkv, D),
                               v[:T].float().reshape(T, Hkv, D), torch.arange(q_pos0, T), geom.scale, geom.window)
        o = o.reshape(M, Hq * D)
        if gate is not None:
            o = o * torch.sigmoid(gate.float())
        out.copy_(o.to(out.dtype))
        return out
    if D in (128, 256) and FLASH_TC and M >= 64 and (gate is None or gate.stride(0) % 8 == 0):
        # tcgen05 / TMEM kernel (head_dim 128, or 256 / gated through its warp-specialised form); it consumes V transposed,
        # built per call in a workspace buffer.  -2: this shape is not served here -> the warp-MMA kernel below
        from .workspace import default_workspace

        ldt = (T + 63) // 64 * 64
        vt = default_workspace(q.device).get("flash_vt", Hkv * D * ldt, torch.bfloat16)
        code = _native.cuda().grm_flash_prefill_tc_gated(_native.ptr(q), _c(q.stride(0)), _native.ptr(k), _native.ptr(v), _c(k.stride(0)),
                                                         _native.ptr(vt), _c(ldt), _native.ptr(gate), _c(gate.stride(0) if gate is not None else 0),
                                                         _native.ptr(out), _c(out.stride(0)), _c(M), _c(T), _c(Hq), _c(Hkv), _c(D),
                                                         _c(q_pos0), _c(geom.window), _f(geom.scale), _native.stream_ptr())
        if code != -2:
            _native.check(code, "flash_prefill_tc")
            return out
    code = _native.cuda().grm_flash_prefill(_native.ptr(q), _c(q.stride(0)), _native.ptr(k), _native.ptr(v), _c(k.stride(0)),
                                            _native.ptr(gate), _native.ptr(out), _c(out.stride(0)), _c(M), _c(T), _c(Hq),
                                            _c(Hkv), _c(D), _c(q_pos0), _c(geom.window), _f(geom.scale),
                                            _native.stream_ptr())
    _native.check(code, "flash_prefill")
    return out


# ---------------------------------------------------------------------------------------------
# embedding / head glue
# ---------------------------------------------------------------------------------------------
def embed(ids: torch.Tensor, table: torch.Tensor, h_out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """bf16 table [V][H] -> fp32 residual rows (reference: launch_embed, src/ops.cpp:684)."""
    if not ids.is_cuda:
        h_out.copy_(table[ids.long()].float() * scale)
        return h_out
    M, H = h_out.shape
    code = _native.cuda().grm_embed(_native.ptr(ids), _native.ptr(table), _native.ptr(h_out), _c(M), _c(H), _c(table.shape[0]),
                                    _c(h_out.stride(0)), _f(scale), _native.stream_ptr())
    _native.check(code, "embed")
    return h_out


def argmax_rows(logits: torch.Tensor, out_ids: torch.Tensor) -> torch.Tensor:
    """Greedy token per row, ties to the lowest index (reference: launch_argmax, src/ops.cpp:611)."""
    if not logits.is_cuda:
        out_ids.copy_(ref.argmax_lowest(logits.float()))
        return out_ids
    M, V = logits.shape
    from .workspace import default_workspace
    ws = default_workspace(logits.device)
    pv = ws.get("argmax_val", max(M, 64) * 64, torch.float32)
    pi = ws.get("argmax_idx", max(M, 64) * 64, torch.int32)
    cnt = ws.get("argmax_counters", 1024, torch.int32, zero=True)
    code = _native.cuda().grm_argmax(_native.ptr(logits), _native.ptr(out_ids), None, _native.ptr(pv), _native.ptr(pi),
                                     _native.ptr(cnt), _c(M), _c(V), _c(logits.stride(0)), _native.stream_ptr())
    _native.check(code, "argmax")
    return out_ids


def status_read(clear: bool = True) -> tuple[int, int, int]:
    """(first error code, detail, count) from the device status block; (0,0,0) when clean."""
    buf = (ctypes.c_uint * 8)()
    code = _native.cuda().grm_status_read(buf, _c(1 if clear else 0), _native.stream_ptr())
    _native.check(code, "status_read")
    return int(buf[0]), int(buf[1]), int(buf[2])
