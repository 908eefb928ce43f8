"""Host oracles of the operators only the K2-Horizon family needs (include/b70/k2_horizon.hpp; the architecture is a
Qwen3-MoE with three substitutions and a routed value projection):

* grouped RMSNorm: the variance is taken per contiguous group of the row, the weight still spans the whole row;
* softplus attention gate: ``attn * softplus(gate, beta)`` with torch's softplus (identity once beta * x > 20), beta = ln 2;
* sigmoid router whose bias steers the SELECTION only: top-k ranks on score + bias, the returned weights are the unbiased
  scores (normalised over the k when asked, then scaled); ties go to the lower expert index;
* MoVA value mixture: ``sum_j w_j * silu(expert_j @ x)`` -- SiLU on the expert OUTPUT, before the router weight;
* layer classification: a layer is sparse when it is not in ``mlp_only_layers``, experts exist and (idx + 1) is a multiple of
  the sparse step.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

K2_GATE_BETA = math.log(2.0)


def rmsnorm_grouped(x: torch.Tensor, w: torch.Tensor, n_groups: int, eps: float) -> torch.Tensor:
    rows, n = x.shape
    xg = x.float().reshape(rows, n_groups, n // n_groups)
    y = xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + eps)
    return y.reshape(rows, n) * w.float()


def softplus(x: torch.Tensor, beta: float) -> torch.Tensor:
    bx = beta * x.float()
    return torch.where(bx > 20.0, x.float(), torch.log1p(torch.exp(torch.clamp(bx, max=20.0))) / beta)


def softplus_gate(attn: torch.Tensor, gate: torch.Tensor, beta: float = K2_GATE_BETA) -> torch.Tensor:
    return attn.float() * softplus(gate, beta)


def router_topk(logits: torch.Tensor, bias, top_k: int, sigmoid_score: bool = True, normalize: bool = True, scaling: float = 1.0):
    """logits [M][E] -> (ids int64 [M][k] in rank order, weights fp32 [M][k])."""
    lg = logits.float()
    score = torch.sigmoid(lg) if sigmoid_score else torch.softmax(lg, dim=-1)
    sel = score + (bias.float()[None, :] if bias is not None else 0.0)
    E = lg.shape[-1]
    # descending on the biased value, ties to the lower index
    order = torch.sort(-sel.double(), dim=-1, stable=True).indices[:, :top_k]
    w = score.gather(1, order)
    if normalize:
        tot = w.sum(-1, keepdim=True)
        w = torch.where(tot > 0, w / tot, w)
    return order, w * scaling


def mova_value(x: torch.Tensor, router_w: torch.Tensor, router_bias, experts: torch.Tensor, top_k: int, scaling: float = 1.0) -> torch.Tensor:
    """x [M][H]; router_w [E][H]; experts [E][out][H] -> routed value projection [M][out]."""
    xf = x.float()
    ids, w = router_topk(xf @ router_w.float().t(), router_bias, top_k, True, top_k > 1, scaling)
    out = torch.zeros(x.shape[0], experts.shape[1])
    for m in range(x.shape[0]):
        for j in range(top_k):
            out[m] += w[m, j] * F.silu(experts[int(ids[m, j])].float() @ xf[m])
    return out


def is_sparse_layer(idx: int, mlp_only_layers, n_experts: int, sparse_step: int) -> bool:
    if idx in set(mlp_only_layers or ()) or n_experts <= 0 or sparse_step <= 0:
        return False
    return (idx + 1) % sparse_step == 0
