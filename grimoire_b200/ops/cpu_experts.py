"""Host expert pool: the experts of an MoE layer that are kept in (pinned) host memory instead of on the device, computed
on CPU threads for the routes that name them (csrc/host/cpu_experts.cpp).  They hold the same block-scaled e4m3 bytes the
device kernels read, so a host expert and a device expert give the same product up to summation order.

Reference: the RAM tier of the tiered-MoE manager -- experts placed in VRAM or pinned RAM by routing hits
(upload_tiered_experts, src/grimoire.cpp:18373), host rows computed by an AVX2 pool and folded into the MoE sum
(src/cpu_experts.cpp; tiered_moe_cpu_rows, src/grimoire.cpp:18784)."""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _native

_c, _f = ctypes.c_int, ctypes.c_float


class CpuExperts:
    def __init__(self, first: int, gate_up: torch.Tensor, gate_up_scale: torch.Tensor, down: torch.Tensor, down_scale: torch.Tensor,
                 pin: bool = False, threads: int = 0):
        """Experts ``first``, ``first + 1``, ... of a layer: gate_up uint8 [n][2I][H] + fp32 scales [n][2I][H/128], down uint8
        [n][H][I] + scales [n][H][I/128]."""
        self.first, self.n = first, gate_up.shape[0]
        self.I, self.H = down.shape[2], down.shape[1]
        keep = lambda t, dt: (t.to(dtype=dt, device="cpu").contiguous().pin_memory() if pin else t.to(dtype=dt, device="cpu").contiguous())
        self.gu, self.gus = keep(gate_up, torch.uint8), keep(gate_up_scale, torch.float32)
        self.dn, self.dns = keep(down, torch.uint8), keep(down_scale, torch.float32)
        self.threads = threads or int(os.environ.get("GRIMOIRE_CPU_EXPERT_THREADS", "0") or 0) or min(32, os.cpu_count() or 1)
        self.rows_served = 0

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.gu, self.gus, self.dn, self.dns))

    def run(self, x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor) -> torch.Tensor | None:
        """x bf16 [M][H] (host), ids int32 [M][k] (host; experts >= ``first`` are this pool's), wts fp32 [M][k] -> the
        pool's share of the layer output, fp32 [M][H] on the host (None when no route names a host expert)."""
        M, k = ids.shape
        mine = ids >= self.first
        if not bool(mine.any()):
            return None
        rows = torch.arange(M, dtype=torch.int32)[:, None].expand(M, k)[mine].contiguous()        # row-major mask: rows ascend
        exp = (ids[mine] - self.first).to(torch.int32).contiguous()
        w = wts[:, :k][mine].to(torch.float32).contiguous()
        out = torch.zeros(M, self.H, dtype=torch.float32)
        x = x.contiguous()
        lib = _native.host()
        rc = lib.grm_cx_moe_rows(_native.ptr(self.gu), _native.ptr(self.gus), _native.ptr(self.dn), _native.ptr(self.dns), _native.ptr(x),
                                 _c(x.stride(0)), _native.ptr(rows), _native.ptr(exp), _native.ptr(w), _c(rows.numel()), _native.ptr(out),
                                 _c(out.stride(0)), _c(self.H), _c(self.I), _c(self.threads))
        if rc != 0:
            raise RuntimeError(f"cpu expert rows: code {rc}")
        self.rows_served += int(rows.numel())
        return out
