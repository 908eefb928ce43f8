"""fp32 oracles of the Gated DeltaNet operators (host), the role of the CPU emulations in the
reference's tests/test_deltanet.cpp and the recurrence stated in src/deltanet.cpp:28-43,122-127,217:

    w = S k ;  S = a*S + beta * (v - a*w) k^T ;  o = (S q) / sqrt(Dk)

with q/k head = v head // (Hv/Hk), a = exp(-exp(A_log) * softplus(a_raw + dt_bias)), beta =
sigmoid(b_raw), q and k L2-normalised per head (x * rsqrt(sum x^2 + 1e-6)), and a depthwise causal
conv (kernel 4, no bias, w[K-1] multiplies the current token) + SiLU over the packed [q|k|v]
channels in front.  The gated output norm is rms_norm(o) * w * silu(z) -- not rms_norm(o * silu(z)).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def l2norm(x: torch.Tensor) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).sum(dim=-1, keepdim=True) + 1e-6)


def gates(a_raw: torch.Tensor, b_raw: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor):
    a = torch.exp(-torch.exp(A_log.float()) * F.softplus(a_raw.float() + dt_bias.float()))
    return a, torch.sigmoid(b_raw.float())


def conv4_silu(x: torch.Tensor, w: torch.Tensor, ring: torch.Tensor):
    """x [T][C] new tokens, w [C][4], ring [C][3] (older tokens, oldest first).  Returns (y [T][C], new ring)."""
    T, C = x.shape
    hist = torch.cat([ring.float().t(), x.float()], dim=0)            # [3+T][C]
    y = torch.zeros(T, C)
    for j in range(4):
        y += hist[j: j + T] * w.float()[:, j]
    return F.silu(y), hist[-3:].t().contiguous()


def gdn_step(S: torch.Tensor, q, k, v, a, beta):
    """One token, all heads.  S [Hv][Dv][Dk]; q,k [Hk][Dk]; v [Hv][Dv]; a,beta [Hv].  Returns o [Hv][Dv]; S is updated in place."""
    Hv, Dv, Dk = S.shape
    rep = Hv // q.shape[0]
    qh, kh = q.float().repeat_interleave(rep, dim=0), k.float().repeat_interleave(rep, dim=0)     # [Hv][Dk]
    w = torch.einsum("hvk,hk->hv", S, kh)
    a3, b3 = a.float()[:, None, None], beta.float()[:, None, None]
    S.mul_(a3).add_(b3 * (v.float() - a.float()[:, None] * w)[:, :, None] * kh[:, None, :])
    return torch.einsum("hvk,hk->hv", S, qh) / math.sqrt(Dk)


def gdn_sequence(S, q, k, v, a, beta):
    """T tokens through gdn_step (the oracle the chunked / fused kernels are compared with)."""
    return torch.stack([gdn_step(S, q[t], k[t], v[t], a[t], beta[t]) for t in range(q.shape[0])])


def gated_rmsnorm(o: torch.Tensor, z: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """o,z [..., Dv]: rms_norm(o) * w * silu(z) (plain weight convention)."""
    r = torch.rsqrt(o.float().pow(2).mean(dim=-1, keepdim=True) + eps)
    return o.float() * r * w.float() * F.silu(z.float())
