"""Python wrappers of the Gated DeltaNet and MoE kernels (gdn.cu, moe.cu) with their fp32 oracles as
the CPU path, plus ``FP8BlockLinear`` -- a projection stored as e4m3 with one fp32 scale per 1x128
block along K, executed by the grouped kernel with a single "expert"."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native
from ..formats import codecs as C
from ..formats.codecs import Fmt
from ..formats.quantize import QuantWeight, quantize
from ..ref import gdn_ref, moe_ref


def _c(v):
    return ctypes.c_int(int(v))


# ---------------------------------------------------------------------------------------------
# grouped fp8 GEMM
# ---------------------------------------------------------------------------------------------
MODE = {"swiglu": 0, "f32": 1, "add_f32": 2, "bf16": 3}


def grouped_gemm_fp8(x: torch.Tensor, row_ids: Optional[torch.Tensor], tile_expert: torch.Tensor, tile_row0: torch.Tensor,
                     tile_rows: torch.Tensor, w: torch.Tensor, scale: torch.Tensor, out: torch.Tensor, mode: str,
                     small: bool = False) -> torch.Tensor:
    """out[grouped rows] = x[row_ids] @ W[expert]^T.  w uint8 [E][N][K] (e4m3), scale fp32 [E][N][K/128].
    ``small``: every tile has at most 8 rows (decode) -> the weight-streaming GEMV form of the kernel."""
    E, N, K = w.shape
    nt = tile_expert.shape[0]
    if not x.is_cuda:
        wd = (C.e4m3_to_f32(w).reshape(E, N, K // 128, 128) * scale[..., None]).reshape(E, N, K)
        xs = x.half().float()
        for t in range(nt):
            e, r0, nr = int(tile_expert[t]), int(tile_row0[t]), int(tile_rows[t])
            rows = torch.arange(r0, r0 + nr)
            src = row_ids[rows].long() if row_ids is not None else rows
            y = xs[src] @ wd[e].t()
            if mode == "swiglu":
                out[rows] = (torch.nn.functional.silu(y[:, : N // 2]) * y[:, N // 2:]).to(out.dtype)
            elif mode == "add_f32":
                out[rows] += y
            else:
                out[rows] = y.to(out.dtype)
        return out
    fn = _native.cuda().grm_moe_grouped_gemv if small else _native.cuda().grm_moe_grouped_gemm
    code = fn(_native.ptr(x), _c(x.stride(0)), _native.ptr(row_ids), _native.ptr(tile_expert),
              _native.ptr(tile_row0), _native.ptr(tile_rows), _c(nt), _native.ptr(w), _native.ptr(scale),
              _native.ptr(out), _c(out.stride(0)), _c(N), _c(K), _c(MODE[mode]), _native.stream_ptr())
    _native.check(code, f"moe_grouped_gemm N={N} K={K} tiles={nt} mode={mode}")
    return out


class FP8BlockLinear:
    """Dense projection with block-scaled fp8 weights: one expert, 16-row tiles."""

    def __init__(self, w, device, name: str = ""):
        qw = w if isinstance(w, QuantWeight) else quantize(w, Fmt.FP8_BLOCK)
        if qw.fmt != Fmt.FP8_BLOCK:
            qw = quantize(qw.dequant(), Fmt.FP8_BLOCK)
        self.name, self.N, self.K = name, qw.N, qw.K
        self.device = torch.device(device)
        self.w = qw.payload.reshape(1, qw.N, qw.K).to(self.device).contiguous()
        self.scale = qw.scales.reshape(1, qw.N, qw.K // 128).float().to(self.device).contiguous()
        self._tiles: dict[int, tuple] = {}

    def nbytes(self) -> int:
        return self.w.numel() + self.scale.numel() * 4

    def tiles(self, M: int):
        t = self._tiles.get(M)
        if t is None:
            nt = (M + 15) // 16
            r0 = torch.arange(nt, dtype=torch.int32) * 16
            nr = torch.clamp(M - r0, max=16).to(torch.int32)
            t = (torch.zeros(nt, dtype=torch.int32, device=self.device), r0.to(self.device), nr.to(self.device))
            self._tiles[M] = t
        return t

    def tiles8(self, M: int):
        t = self._tiles.get(-M)
        if t is None:
            t = (torch.zeros(1, dtype=torch.int32, device=self.device), torch.zeros(1, dtype=torch.int32, device=self.device),
                 torch.full((1,), M, dtype=torch.int32, device=self.device))
            self._tiles[-M] = t
        return t

    def forward(self, x: torch.Tensor, out: torch.Tensor, epi: str = "bf16") -> torch.Tensor:
        M = x.shape[0]
        if M <= 8:
            te, r0, nr = self.tiles8(M)
            return grouped_gemm_fp8(x, None, te, r0, nr, self.w, self.scale, out, epi, small=True)
        if M > 64 and x.is_cuda:
            # tall inputs: dequantise once into the shared bf16 scratch and run the tcgen05 GEMM (the policy of the
            # int4 projections as well); SwiGLU weights are [gate | up] here, so the two halves are separate GEMMs
            from .linear import gemm_bf16
            from .workspace import default_workspace

            ws = default_workspace(self.device)
            wb = ws.get("dequant_bf16", self.N * self.K, torch.bfloat16).view(-1)[: self.N * self.K].view(self.N, self.K)
            _native.check(_native.cuda().grm_dequant_fp8_block(_native.ptr(self.w), _native.ptr(self.scale), _native.ptr(wb), _c(self.N),
                                                               _c(self.K), _native.stream_ptr()), f"dequant_fp8_block {self.name}")
            if epi == "swiglu":
                I = self.N // 2
                g = ws.get("fp8_gate_f32", M * I, torch.float32).view(-1)[: M * I].view(M, I)
                u = ws.get("fp8_up_f32", M * I, torch.float32).view(-1)[: M * I].view(M, I)
                gemm_bf16(x, wb[:I], g, "f32")
                gemm_bf16(x, wb[I:], u, "f32")
                torch.mul(torch.nn.functional.silu(g), u, out=g)
                out.copy_(g)
                return out
            return gemm_bf16(x, wb, out, epi)
        te, r0, nr = self.tiles(M)
        return grouped_gemm_fp8(x, None, te, r0, nr, self.w, self.scale, out, epi)

    __call__ = forward


# ---------------------------------------------------------------------------------------------
# routing / combine
# ---------------------------------------------------------------------------------------------
def moe_route(logits: torch.Tensor, E: int, top_k: int, renorm: bool, ids: torch.Tensor, wts: torch.Tensor,
              counts: Optional[torch.Tensor] = None, shared_gate: bool = False):
    """Softmax top-k routing.  ``shared_gate``: wts has top_k + 1 columns and column top_k receives
    sigmoid(logits[:, E]), the shared expert's weight."""
    M = logits.shape[0]
    if not logits.is_cuda:
        i, w = moe_ref.route(logits[:, :E], top_k, renorm)
        ids.copy_(i.to(ids.dtype))
        wts[:, :top_k].copy_(w)
        if shared_gate:
            wts[:, top_k] = torch.sigmoid(logits[:, E].float())
        if counts is not None:
            counts += torch.bincount(i.flatten(), minlength=counts.shape[0]).to(counts.dtype)
        return ids, wts
    code = _native.cuda().grm_moe_route(_native.ptr(logits), _c(logits.stride(0)), _c(M), _c(E), _c(top_k), _c(1 if renorm else 0),
                                        _native.ptr(ids), _c(ids.stride(0)), _native.ptr(wts), _c(wts.stride(0)), _native.ptr(counts),
                                        _c(1 if shared_gate else 0), _native.stream_ptr())
    _native.check(code, "moe_route")
    return ids, wts


def moe_combine(h: torch.Tensor, y: torch.Tensor, pos: torch.Tensor, wts: torch.Tensor) -> torch.Tensor:
    """h[tok] += sum_j wts[tok][j] * y[pos[tok][j]] in slot order (deterministic)."""
    M, slots = pos.shape
    if not h.is_cuda:
        for j in range(slots):
            ok = pos[:, j] >= 0
            h[ok] += wts[ok, j: j + 1] * y[pos[ok, j].long()].float()
        return h
    code = _native.cuda().grm_moe_combine(_native.ptr(h), _c(h.stride(0)), _native.ptr(y), _c(y.stride(0)), _native.ptr(pos),
                                          _native.ptr(wts), _c(M), _c(slots), _c(h.shape[1]), _native.stream_ptr())
    _native.check(code, "moe_combine")
    return h


# ---------------------------------------------------------------------------------------------
# Gated DeltaNet
# ---------------------------------------------------------------------------------------------
def conv4_silu(x: torch.Tensor, w: torch.Tensor, ring: torch.Tensor, ring_tmp: torch.Tensor, row_seq: torch.Tensor,
               row_pos: torch.Tensor, y: torch.Tensor, touched: torch.Tensor) -> torch.Tensor:
    """Depthwise causal conv (k = 4) + SiLU.  ring [slots][C][3] is updated for the slots in ``touched``."""
    M, Cc = x.shape
    if not x.is_cuda:
        rs, rp = row_seq.tolist(), row_pos.tolist()
        m = 0
        while m < M:
            n = 1
            while m + n < M and rs[m + n] == rs[m] and rp[m + n] == rp[m] + n:
                n += 1
            yy, newring = gdn_ref.conv4_silu(x[m: m + n].float(), w, ring[rs[m]])
            y[m: m + n] = yy.to(y.dtype)
            ring[rs[m]] = newring
            m += n
        return y
    code = _native.cuda().grm_conv4_silu(_native.ptr(x), _native.ptr(w), _native.ptr(ring), _native.ptr(ring_tmp), _native.ptr(row_seq),
                                         _native.ptr(row_pos), _native.ptr(y), _c(M), _c(Cc), _c(x.stride(0)), _c(y.stride(0)),
                                         _native.stream_ptr())
    _native.check(code, "conv4_silu")
    ring.index_copy_(0, touched, ring_tmp.index_select(0, touched))
    return y


def gdn_runs(qkv: torch.Tensor, ab: torch.Tensor, z: torch.Tensor, A_log, dt_bias, norm_w, eps: float, state: torch.Tensor,
             run_slot: torch.Tensor, run_start: torch.Tensor, run_len: torch.Tensor, out: torch.Tensor, Hk: int, Hv: int, Dk: int, Dv: int,
             chunked: bool = False):
    """Gated delta rule over runs of rows (see gdn.cu); state [slots][Hv][Dv][Dk] fp32 is updated.
    ``chunked``: the runs are long (prompt chunks) -> the 64-token chunked form instead of the per-token scan."""
    if not qkv.is_cuda:
        for s, r0, n in zip(run_slot.tolist(), run_start.tolist(), run_len.tolist()):
            x = qkv[r0: r0 + n].float()
            q = gdn_ref.l2norm(x[:, : Hk * Dk].reshape(n, Hk, Dk))
            k = gdn_ref.l2norm(x[:, Hk * Dk: 2 * Hk * Dk].reshape(n, Hk, Dk))
            v = x[:, 2 * Hk * Dk:].reshape(n, Hv, Dv)
            a, b = gdn_ref.gates(ab[r0: r0 + n, :Hv], ab[r0: r0 + n, Hv:], A_log, dt_bias)
            o = gdn_ref.gdn_sequence(state[s], q, k, v, a, b)
            out[r0: r0 + n] = gdn_ref.gated_rmsnorm(o, z[r0: r0 + n].float().reshape(n, Hv, Dv), norm_w, eps).reshape(n, Hv * Dv).to(out.dtype)
        return out
    if chunked:
        from .workspace import default_workspace

        M = qkv.shape[0]
        o_raw = default_workspace(qkv.device).get("gdn_o_raw", M * Hv * Dv, torch.float32)
        code = _native.cuda().grm_gdn_chunked(_native.ptr(qkv), _c(qkv.stride(0)), _native.ptr(ab), _c(ab.stride(0)), _native.ptr(z),
                                              _c(z.stride(0)), _native.ptr(A_log), _native.ptr(dt_bias), _native.ptr(norm_w),
                                              ctypes.c_float(eps), _native.ptr(state), _native.ptr(run_slot), _native.ptr(run_start),
                                              _native.ptr(run_len), _c(run_slot.shape[0]), _native.ptr(o_raw), _native.ptr(out),
                                              _c(out.stride(0)), _c(M), _c(Hk), _c(Hv), _c(Dk), _c(Dv), _native.stream_ptr())
        _native.check(code, "gdn_chunked")
        return out
    code = _native.cuda().grm_gdn_runs(_native.ptr(qkv), _c(qkv.stride(0)), _native.ptr(ab), _c(ab.stride(0)), _native.ptr(z), _c(z.stride(0)),
                                       _native.ptr(A_log), _native.ptr(dt_bias), _native.ptr(norm_w), ctypes.c_float(eps), _native.ptr(state),
                                       _native.ptr(run_slot), _native.ptr(run_start), _native.ptr(run_len), _c(run_slot.shape[0]),
                                       _native.ptr(out), _c(out.stride(0)), _c(Hk), _c(Hv), _c(Dk), _c(Dv), _native.stream_ptr())
    _native.check(code, "gdn_runs")
    return out
