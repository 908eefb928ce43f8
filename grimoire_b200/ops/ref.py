"""Plain PyTorch fp32 references of every device op.

Two uses: (1) the oracle that the CUDA kernels are compared against in ``tests/ -m gpu`` and
(2) the CPU path of the engine (tiny-model correctness runs, gloo multi-rank tests).  The math here
follows the numerics conventions the reference pins with tests (q/k norm before RoPE, NeoX RoPE
over the first ``rot`` dims, zero-centred norm weights, int8 KV with max|x|/127 scales ...).
"""
from __future__ import annotations

import math
from typing import Optional

import torch

PAGE = 16


def rmsnorm(h: torch.Tensor, w: torch.Tensor, eps: float, offset: float) -> torch.Tensor:
    h = h.float()
    r = torch.rsqrt(h.pow(2).mean(dim=-1, keepdim=True) + eps)
    return h * r * (offset + w.float())


def linear_dequant(x: torch.Tensor, w_deq: torch.Tensor) -> torch.Tensor:
    """x [M][K] (any float dtype, rounded to bf16 like the kernel input) @ dequantized W[N][K]^T in fp32."""
    return x.bfloat16().float() @ w_deq.float().t()


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.silu(gate.float()) * up.float()


def rope_inv_freq(rot: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))


def apply_rope(x: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, rot: int) -> torch.Tensor:
    """x [M][H][D] fp32, NeoX half-split over the first ``rot`` dims (src/ops.cpp:870-912)."""
    ang = pos.float()[:, None] * inv_freq[None, :]          # [M][rot/2]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., : rot // 2], x[..., rot // 2: rot]
    out = x.clone()
    out[..., : rot // 2] = a * cos - b * sin
    out[..., rot // 2: rot] = b * cos + a * sin
    return out


def head_rmsnorm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float, offset: float) -> torch.Tensor:
    if w is None:
        return x
    r = torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
    return x * r * (offset + w.float())


def quant_i8_rows(x: torch.Tensor):
    """Per-(token, head) int8 quantisation: scale = max|x|/127 (src/kv_k8.hpp:19-59)."""
    amax = x.abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.round(x / scale[..., None]).clamp(-127, 127).to(torch.int8)
    return q, scale


def attention_rows(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor, scale: float,
                   window: int = 0) -> torch.Tensor:
    """q [M][Hq][D]; k,v [T][Hkv][D] (dequantized); row m sees keys 0..q_pos[m] (within window)."""
    M, Hq, D = q.shape
    T, Hkv, _ = k.shape
    G = Hq // Hkv
    kk = k.float().repeat_interleave(G, dim=1)               # [T][Hq][D]
    vv = v.float().repeat_interleave(G, dim=1)
    s = torch.einsum("mhd,thd->mht", q.float(), kk) * scale
    keys = torch.arange(T)[None, None, :]
    qp = q_pos.long()[:, None, None]
    ok = keys <= qp
    if window > 0:
        ok = ok & (keys > qp - window)
    s = s.masked_fill(~ok, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("mht,thd->mhd", p, vv)


def argmax_lowest(logits: torch.Tensor) -> torch.Tensor:
    """arg-max with ties resolved to the lowest index."""
    mx = logits.max(dim=-1, keepdim=True).values
    idx = torch.arange(logits.shape[-1], device=logits.device).expand_as(logits)
    big = torch.full_like(idx, logits.shape[-1])
    return torch.where(logits == mx, idx, big).min(dim=-1).values.to(torch.int32)


def softmax_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
