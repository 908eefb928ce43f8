"""Sampling options, the counter-based generator and the host reference of the device sampler.

``SamplingOptions`` and the generator follow include/b70/sampling.hpp:10-35 (temperature, top-k
<= 64 with default 20, top-p, seed; uniform = splitmix64(seed, position) so a captured decode graph
holds no generator state).  ``coupled_sample`` is speculative sampling with a shared uniform
(Leviathan et al., algorithm 1; include/b70/speculative_sampling.hpp:39-61): a draft token is kept
with probability min(1, p_target/p_draft), otherwise a token is drawn from the normalised residual
max(0, p_target - p_draft), so the output distribution equals the target's.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import _native

MASK64 = (1 << 64) - 1
TOP_K_MAX = 64


@dataclass
class SamplingOptions:
    temperature: float = 0.0        # 0 = greedy
    top_k: int = 20
    top_p: float = 1.0
    seed: int = 0

    def validate(self) -> "SamplingOptions":
        if self.temperature < 0 or not math.isfinite(self.temperature):
            raise ValueError("temperature must be a finite number >= 0")
        if not (1 <= self.top_k <= TOP_K_MAX):
            raise ValueError(f"top_k must be in 1..{TOP_K_MAX}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError("top_p must be in (0, 1]")
        return self

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0 or self.top_k == 1


def splitmix64(seed: int, position: int) -> int:
    x = (seed ^ ((position * 0x9E3779B97F4A7C15) & MASK64)) & MASK64
    x = (x + 0x9E3779B97F4A7C15) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    return x ^ (x >> 31)


def uniform(seed: int, position: int) -> float:
    return (splitmix64(seed, position) >> 11) * (1.0 / 9007199254740992.0)


def sample_ref(logits: torch.Tensor, opt: SamplingOptions, position: int) -> int:
    """Host reference of sample.cu for one row of fp32 logits."""
    lg = logits.float().cpu()
    k = max(1, min(TOP_K_MAX, opt.top_k))
    # descending by value, ties to the lowest index
    order = sorted(range(lg.numel()), key=lambda i: (-float(lg[i]), i))[:k] if lg.numel() <= 4096 else None
    if order is None:
        vals, idx = torch.topk(lg, k)
        pairs = sorted(zip((-vals).tolist(), idx.tolist()))
        order = [i for _, i in pairs]
    if opt.temperature <= 0 or k == 1:
        return order[0]
    tv = torch.tensor([float(lg[i]) for i in order], dtype=torch.float32)
    pr = torch.exp((tv - tv[0]) / opt.temperature)
    s = float(pr.sum())
    keep = k
    if 0.0 < opt.top_p < 1.0:
        acc = 0.0
        for r in range(k):
            acc += float(pr[r]) / s
            if acc >= opt.top_p:
                keep = r + 1
                break
    ksum = float(pr[:keep].sum())
    u = float(torch.tensor(uniform(opt.seed, position), dtype=torch.float64).float()) * ksum
    acc = 0.0
    for r in range(keep):
        acc += float(pr[r])
        if u < acc:
            return order[r]
    return order[keep - 1]


class DeviceSampler:
    """Per-row sampling parameters resident on the device + the kernel call (graph friendly)."""

    def __init__(self, max_rows: int, device):
        self.device = torch.device(device)
        z = lambda dt: torch.zeros(max_rows, dtype=dt, device=self.device)
        self.temperature, self.top_p = z(torch.float32), torch.ones(max_rows, dtype=torch.float32, device=self.device)
        self.top_k = torch.ones(max_rows, dtype=torch.int32, device=self.device)
        self.seeds = z(torch.int64)
        self.cand_val = torch.empty(max_rows * 64 * 64, dtype=torch.float32, device=self.device)
        self.cand_idx = torch.empty(max_rows * 64 * 64, dtype=torch.int32, device=self.device)
        self.counters = z(torch.int32)

    def set_rows(self, opts: Sequence[SamplingOptions]) -> None:
        n = len(opts)
        self.temperature[:n] = torch.tensor([o.temperature for o in opts], dtype=torch.float32)
        self.top_p[:n] = torch.tensor([o.top_p for o in opts], dtype=torch.float32)
        self.top_k[:n] = torch.tensor([o.top_k for o in opts], dtype=torch.int32)
        self.seeds[:n] = torch.tensor([o.seed - (1 << 64) if o.seed >= (1 << 63) else o.seed for o in opts], dtype=torch.int64)

    def sample(self, logits: torch.Tensor, positions: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        M, V = logits.shape
        c = ctypes.c_int
        code = _native.cuda().grm_sample_logits(_native.ptr(logits), c(logits.stride(0)), c(V), _native.ptr(positions),
                                                _native.ptr(self.temperature), _native.ptr(self.top_p), _native.ptr(self.top_k),
                                                _native.ptr(self.seeds), _native.ptr(self.cand_val), _native.ptr(self.cand_idx),
                                                _native.ptr(self.counters), _native.ptr(out), c(M), _native.stream_ptr())
        _native.check(code, "sample_logits")
        return out


def coupled_sample(p_target: torch.Tensor, p_draft: torch.Tensor, draft_token: int, u_accept: float, u_resample: float):
    """Speculative sampling step for one position.  Returns (token, accepted)."""
    pt, pd = float(p_target[draft_token]), float(p_draft[draft_token])
    if pd <= 0.0 or u_accept < min(1.0, pt / pd):
        if pd > 0.0:
            return draft_token, True
    resid = (p_target.double() - p_draft.double()).clamp_min(0.0)
    z = float(resid.sum())
    if z <= 0.0:
        resid, z = p_target.double(), float(p_target.double().sum())
    cdf = torch.cumsum(resid / z, dim=0)
    tok = int(torch.searchsorted(cdf, torch.tensor(u_resample, dtype=torch.float64)).clamp_max(p_target.numel() - 1))
    return tok, False
