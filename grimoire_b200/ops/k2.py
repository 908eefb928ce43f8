"""Operators of the K2-Horizon family (csrc/kernels/k2_ops.cu; CPU path = the host oracles of ref/k2_ref.py) and the MoVA
routed value projection built from them (reference: ``mova_value_m1`` and launch_mova_value_decode,
src/moe_kernels.cpp:465-624: v_proj replaced by a bank of [kv_heads * head_dim, hidden] experts, top-4 by a sigmoid router
with a selection-only bias, each expert output put through SiLU and accumulated with its router weight)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native
from ..formats.codecs import Fmt
from ..formats.quantize import quantize
from ..ref import k2_ref
from . import hybrid as Hb
from .linear import BF16Linear

_c, _f = ctypes.c_int, ctypes.c_float


def rmsnorm_grouped(h: torch.Tensor, w: torch.Tensor, out: torch.Tensor, n_groups: int, eps: float) -> torch.Tensor:
    """out (bf16) = grouped RMSNorm of the fp32 rows ``h``: variance per contiguous group, weight over the whole row."""
    if not h.is_cuda:
        out.copy_(k2_ref.rmsnorm_grouped(h, w, n_groups, eps).to(out.dtype))
        return out
    code = _native.cuda().grm_rmsnorm_grouped(_native.ptr(h), _c(h.stride(0)), _native.ptr(w), _native.ptr(out), _c(out.stride(0)),
                                              _c(h.shape[0]), _c(h.shape[1]), _c(n_groups), _f(eps), _native.stream_ptr())
    _native.check(code, "rmsnorm_grouped")
    return out


def softplus_gate(attn: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, beta: float = k2_ref.K2_GATE_BETA) -> torch.Tensor:
    """out = attn * softplus(gate, beta) (bf16, contiguous, same shape)."""
    if not attn.is_cuda:
        out.copy_(k2_ref.softplus_gate(attn, gate, beta).to(out.dtype))
        return out
    code = _native.cuda().grm_softplus_gate(_native.ptr(attn), _native.ptr(gate), _native.ptr(out), ctypes.c_long(attn.numel()), _f(beta),
                                            _native.stream_ptr())
    _native.check(code, "softplus_gate")
    return out


def router_topk_bias(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, ids: torch.Tensor, wts: torch.Tensor,
                     sigmoid_score: bool = True, normalize: bool = True, scaling: float = 1.0):
    """Top-k on score + bias, weights from the unbiased scores (ties to the lower index)."""
    M, E = logits.shape
    if not logits.is_cuda:
        i, w = k2_ref.router_topk(logits, bias, top_k, sigmoid_score, normalize, scaling)
        ids.copy_(i.to(ids.dtype))
        wts[:, :top_k].copy_(w)
        return ids, wts
    code = _native.cuda().grm_router_topk_bias(_native.ptr(logits), _c(logits.stride(0)), _native.ptr(bias), _c(M), _c(E), _c(top_k),
                                               _c(1 if sigmoid_score else 0), _c(1 if normalize else 0), _f(scaling), _native.ptr(ids),
                                               _c(ids.stride(0)), _native.ptr(wts), _c(wts.stride(0)), _native.stream_ptr())
    _native.check(code, "router_topk_bias")
    return ids, wts


class MovaValue:
    """Routed value projection: ``value = sum_j w_j * silu(expert_j @ x)`` over the top-k of a sigmoid router."""

    def __init__(self, router_w: torch.Tensor, router_bias: Optional[torch.Tensor], experts: torch.Tensor, top_k: int, device,
                 scaling: float = 1.0, max_rows: int = 64):
        self.device = torch.device(device)
        self.E, self.out, self.H = experts.shape
        self.top_k, self.scaling = top_k, scaling
        self.router = BF16Linear(router_w, self.device, "mova.router")
        self.bias = None if router_bias is None else router_bias.to(device=self.device, dtype=torch.float32).contiguous()
        q = quantize(experts.reshape(self.E * self.out, self.H).float(), Fmt.FP8_BLOCK)
        self.w = q.payload.reshape(self.E, self.out, self.H).to(self.device).contiguous()
        self.scale = q.scales.reshape(self.E, self.out, self.H // 128).float().to(self.device).contiguous()
        mk = lambda *s, dt: torch.zeros(*s, dtype=dt, device=self.device)
        self.logits = mk(max_rows, (self.E + 3) // 4 * 4, dt=torch.float32)
        self.ids, self.wts = mk(max_rows, top_k, dt=torch.int32), mk(max_rows, top_k, dt=torch.float32)
        self.y = mk(max_rows * top_k, self.out, dt=torch.float32)
        ar = torch.arange(max_rows * top_k, dtype=torch.int32, device=self.device)
        self.row0, self.rows, self.src = ar, torch.ones_like(ar), (ar // top_k).to(torch.int32)
        self.max_rows = max_rows

    def dequant(self) -> torch.Tensor:
        from ..formats.quantize import QuantWeight

        return QuantWeight(Fmt.FP8_BLOCK, self.E * self.out, self.H, self.w.reshape(-1, self.H).cpu(),
                           scales=self.scale.reshape(-1, self.H // 128).cpu(), group=128).dequant().reshape(self.E, self.out, self.H)

    def forward(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """x bf16 [M][H] -> out bf16 [M][kv_heads * head_dim] (M <= max_rows: decode rows / verify blocks)."""
        M, k = x.shape[0], self.top_k
        if M > self.max_rows:                      # prompt chunks: in pieces of the staging buffers' height
            for m0 in range(0, M, self.max_rows):
                self.forward(x[m0: m0 + self.max_rows], out[m0: m0 + self.max_rows])
            return out
        lg = self.logits[:M, : self.E]
        self.router(x, lg, "f32")
        ids, wts = self.ids[:M], self.wts[:M]
        router_topk_bias(lg, self.bias, k, ids, wts, True, k > 1, self.scaling)
        if not x.is_cuda:
            w = self.dequant()
            xf = x.float()
            y = torch.stack([torch.nn.functional.silu(w[int(ids[m, j])] @ xf[m]) * wts[m, j] for m in range(M) for j in range(k)])
            out.copy_(y.reshape(M, k, self.out).sum(1).to(out.dtype))
            return out
        y = self.y[: M * k]
        Hb.grouped_gemm_fp8(x, self.src[: M * k], ids.reshape(-1), self.row0[: M * k], self.rows[: M * k], self.w, self.scale, y, "f32", small=True)
        code = _native.cuda().grm_mova_combine(_native.ptr(y), _native.ptr(wts), _c(wts.stride(0)), _native.ptr(out), _c(out.stride(0)), _c(M),
                                               _c(k), _c(self.out), _native.stream_ptr())
        _native.check(code, "mova_combine")
        return out

    __call__ = forward
