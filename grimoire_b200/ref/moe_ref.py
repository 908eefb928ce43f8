"""fp32 oracle of the MoE block (route_ref / moe_forward_ref, src/moe_ref.cpp:30-107,
include/b70/moe.hpp:182-185): softmax over ALL experts, top-k (ties to the lowest index),
renormalise over the k, SwiGLU experts, plus the shared expert scaled by sigmoid(x . w_gate)."""
from __future__ import annotations

import torch
import torch.nn.functional as F


def route(logits: torch.Tensor, top_k: int, renorm: bool = True):
    """logits [M][E] -> (ids int64 [M][k] sorted by descending probability, weights fp32 [M][k])."""
    p = torch.softmax(logits.float(), dim=-1)
    E = p.shape[-1]
    # descending probability, ties to the lowest index: sort by (-p, index)
    order = torch.sort(torch.stack([(-p).double(), torch.arange(E, dtype=torch.float64).expand_as(p)], -1)[..., 0], dim=-1, stable=True).indices
    ids = order[:, :top_k]
    w = p.gather(1, ids)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return ids, w


def expert_ffn(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    return (F.silu(x @ wg.float().t()) * (x @ wu.float().t())) @ wd.float().t()


def moe_forward(x: torch.Tensor, router_w: torch.Tensor, experts, top_k: int, shared=None, shared_gate_w=None, renorm=True):
    """x [M][H] fp32; experts = list of (gate [I][H], up [I][H], down [H][I]) fp32; shared likewise."""
    x = x.float()
    ids, w = route(x.bfloat16().float() @ router_w.float().t(), top_k, renorm)
    y = torch.zeros_like(x)
    for m in range(x.shape[0]):
        for j in range(top_k):
            g, u, d = experts[int(ids[m, j])]
            y[m] += w[m, j] * expert_ffn(x[m: m + 1], g, u, d)[0]
    if shared is not None:
        s = expert_ffn(x, *shared)
        if shared_gate_w is not None:
            s = s * torch.sigmoid(x @ shared_gate_w.float().t())
        y += s
    return y, ids, w
