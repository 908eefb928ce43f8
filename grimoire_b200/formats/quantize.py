"""Weight descriptor and host quantizers for every runtime format.

``QuantWeight`` mirrors the reference's descriptor (include/b70/weights.hpp:264-404: fmt, N, K,
payload K-major ``[N][bytes_per_row]``, per-row or per-group scales, int4 zeros) and ``quantize``
its host quantizers (src/quantize.cpp:81-320): per-row absmax for INT8 / FP8, asymmetric
round-to-nearest INT4 with an optional clipping-range search and importance weighting, OCP MX
shared exponents for MXFP4 / MXFP8.  Added here: symmetric int4 (GPTQ ``sym=True`` checkpoints),
block-scaled fp8 (e4m3 with one fp32 scale per 1x128 block) and NVFP4.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import codecs as C
from .codecs import Fmt


@dataclass
class QuantWeight:
    """One quantized ``[N][K]`` matrix in the *logical* (row-major, K-major) layout.

    payload : uint8 ``[N][row_bytes]``   (int4/fp4: two codes per byte, even k in the low nibble;
              bf16: 2 bytes per element little-endian)
    scales  : INT8/FP8 per row fp32 ``[N]``; INT4 fp16 ``[N][K/group]``; MX uint8 E8M0
              ``[N][K/32]``; FP8_BLOCK fp32 ``[N][K/128]``; NVFP4 uint8 E4M3 ``[N][K/16]``
    zeros   : INT4 only, uint8 ``[N][K/group]`` (real zero point 0..15; 8 when symmetric)
    """

    fmt: Fmt
    N: int
    K: int
    payload: torch.Tensor
    scales: Optional[torch.Tensor] = None
    zeros: Optional[torch.Tensor] = None
    group: int = 0
    global_scale: float = 1.0
    meta: dict = field(default_factory=dict)

    def dequant(self) -> torch.Tensor:
        """fp32 ``[N][K]`` reference dequantisation (the ``at(n,k)`` oracle, weights.hpp:346-365)."""
        N, K = self.N, self.K
        f = self.fmt
        if f == Fmt.BF16:
            return self.payload.view(torch.bfloat16).reshape(N, K).float()
        if f == Fmt.INT8:
            return self.payload.view(torch.int8).float() * self.scales.float()[:, None]
        if f == Fmt.FP8_E4M3:
            return C.e4m3_to_f32(self.payload) * self.scales.float()[:, None]
        if f == Fmt.FP8_E5M2:
            return C.e5m2_to_f32(self.payload) * self.scales.float()[:, None]
        if f == Fmt.INT4:
            q = C.unpack_nibbles(self.payload).float().reshape(N, K // self.group, self.group)
            z = self.zeros.float()[:, :, None]
            s = self.scales.float()[:, :, None]
            return ((q - z) * s).reshape(N, K)
        if f == Fmt.MXFP4:
            v = C.e2m1_to_f32(C.unpack_nibbles(self.payload)).reshape(N, K // C.MX_BLOCK, C.MX_BLOCK)
            return (v * C.e8m0_to_f32(self.scales)[:, :, None]).reshape(N, K)
        if f == Fmt.MXFP8:
            v = C.e4m3_to_f32(self.payload).reshape(N, K // C.MX_BLOCK, C.MX_BLOCK)
            return (v * C.e8m0_to_f32(self.scales)[:, :, None]).reshape(N, K)
        if f == Fmt.FP8_BLOCK:
            v = C.e4m3_to_f32(self.payload).reshape(N, K // C.FP8_BLOCK_K, C.FP8_BLOCK_K)
            return (v * self.scales.float()[:, :, None]).reshape(N, K)
        if f == Fmt.NVFP4:
            v = C.e2m1_to_f32(C.unpack_nibbles(self.payload)).reshape(N, K // C.NVFP4_BLOCK, C.NVFP4_BLOCK)
            s = C.e4m3_to_f32(self.scales)[:, :, None] * self.global_scale
            return (v * s).reshape(N, K)
        raise ValueError(f"dequant: unsupported format {f!r}")

    def nbytes(self) -> int:
        n = self.payload.numel() * self.payload.element_size()
        for t in (self.scales, self.zeros):
            if t is not None:
                n += t.numel() * t.element_size()
        return n


def _int4_group_quant(w: torch.Tensor, group: int, symmetric: bool, search: bool,
                      importance: Optional[torch.Tensor]):
    N, K = w.shape
    wg = w.reshape(N, K // group, group)
    if symmetric:
        amax = wg.abs().amax(dim=-1, keepdim=True)
        scale = (amax / 7.0).clamp_min(1e-10)
        scale = scale.half().float()
        q = torch.round(wg / scale).clamp(-8, 7) + 8
        zero = torch.full_like(scale, 8.0)
        return q, scale.squeeze(-1), zero.squeeze(-1)
    imp = None if importance is None else importance.float().reshape(1, K // group, group)
    lo0 = wg.amin(dim=-1, keepdim=True).clamp_max(0.0)
    hi0 = wg.amax(dim=-1, keepdim=True).clamp_min(0.0)
    best = None
    shrinks = [1.0] if not search else [1.0, 0.95, 0.9, 0.85, 0.8, 0.75, 0.7]
    for sh in shrinks:
        lo, hi = lo0 * sh, hi0 * sh
        scale = ((hi - lo) / 15.0).clamp_min(1e-10).half().float()
        zero = torch.round(-lo / scale).clamp(0, 15)
        q = (torch.round(wg / scale) + zero).clamp(0, 15)
        err = ((q - zero) * scale - wg) ** 2
        if imp is not None:
            err = err * imp
        err = err.sum(dim=-1, keepdim=True)
        if best is None:
            best = (err, q, scale, zero)
        else:
            take = err < best[0]
            best = (torch.where(take, err, best[0]), torch.where(take, q, best[1]),
                    torch.where(take, scale, best[2]), torch.where(take, zero, best[3]))
    _, q, scale, zero = best
    return q, scale.squeeze(-1), zero.squeeze(-1)


def quantize(w: torch.Tensor, fmt: Fmt, *, group: int = C.INT4_GROUP, symmetric: bool = False,
             search: bool = False, importance: Optional[torch.Tensor] = None) -> QuantWeight:
    """Quantize an fp32/bf16 ``[N][K]`` matrix to ``fmt`` (round to nearest).

    ``importance`` is an optional ``[K]`` activation-importance vector that weights the int4
    rounding error when ``search`` picks a clipping range (imatrix steering,
    src/quantize.cpp:170-250)."""
    w = w.detach().float()
    N, K = w.shape
    if fmt == Fmt.BF16:
        return QuantWeight(fmt, N, K, w.bfloat16().contiguous().view(torch.uint8).reshape(N, K * 2))
    if fmt in (Fmt.INT8, Fmt.FP8_E4M3, Fmt.FP8_E5M2):
        amax = w.abs().amax(dim=1).clamp_min(1e-30)
        if fmt == Fmt.INT8:
            scale = amax / 127.0
            q = torch.round(w / scale[:, None]).clamp(-127, 127).to(torch.int8).view(torch.uint8)
        elif fmt == Fmt.FP8_E4M3:
            scale = amax / C.E4M3_MAX
            q = C.f32_to_e4m3(w / scale[:, None])
        else:
            scale = amax / C.E5M2_MAX
            q = C.f32_to_e5m2(w / scale[:, None])
        return QuantWeight(fmt, N, K, q.contiguous(), scales=scale.float())
    if fmt == Fmt.INT4:
        if K % group:
            raise ValueError(f"K={K} not a multiple of the int4 group {group}")
        q, scale, zero = _int4_group_quant(w, group, symmetric, search, importance)
        payload = C.pack_nibbles(q.reshape(N, K).to(torch.uint8))
        return QuantWeight(fmt, N, K, payload, scales=scale.half(), zeros=zero.to(torch.uint8), group=group)
    if fmt in (Fmt.MXFP4, Fmt.MXFP8):
        if K % C.MX_BLOCK:
            raise ValueError("K must be a multiple of 32 for MX formats")
        wb = w.reshape(N, K // C.MX_BLOCK, C.MX_BLOCK)
        amax = wb.abs().amax(dim=-1)
        e = C.pick_e8m0(amax, 2 if fmt == Fmt.MXFP4 else 8)
        inv = 1.0 / C.e8m0_to_f32(e)[:, :, None]
        if fmt == Fmt.MXFP4:
            payload = C.pack_nibbles(C.f32_to_e2m1(wb * inv).reshape(N, K))
        else:
            payload = C.f32_to_e4m3(wb * inv).reshape(N, K)
        return QuantWeight(fmt, N, K, payload.contiguous(), scales=e.contiguous(), group=C.MX_BLOCK)
    if fmt == Fmt.FP8_BLOCK:
        if K % C.FP8_BLOCK_K:
            raise ValueError("K must be a multiple of 128 for block-scaled fp8")
        wb = w.reshape(N, K // C.FP8_BLOCK_K, C.FP8_BLOCK_K)
        scale = (wb.abs().amax(dim=-1) / C.E4M3_MAX).clamp_min(1e-30)
        payload = C.f32_to_e4m3(wb / scale[:, :, None]).reshape(N, K)
        return QuantWeight(fmt, N, K, payload.contiguous(), scales=scale.float().contiguous(), group=C.FP8_BLOCK_K)
    if fmt == Fmt.NVFP4:
        if K % C.NVFP4_BLOCK:
            raise ValueError("K must be a multiple of 16 for NVFP4")
        wb = w.reshape(N, K // C.NVFP4_BLOCK, C.NVFP4_BLOCK)
        gmax = float(w.abs().max().clamp_min(1e-30))
        gscale = gmax / (C.E4M3_MAX * 6.0)
        bs = C.f32_to_e4m3(wb.abs().amax(dim=-1) / 6.0 / gscale)
        dec = (C.e4m3_to_f32(bs) * gscale).clamp_min(1e-30)
        payload = C.pack_nibbles(C.f32_to_e2m1(wb / dec[:, :, None]).reshape(N, K))
        return QuantWeight(fmt, N, K, payload, scales=bs.contiguous(), group=C.NVFP4_BLOCK, global_scale=gscale)
    raise ValueError(f"quantize: unsupported target format {fmt!r}")


def slice_rows(qw: QuantWeight, a: int, b: int) -> QuantWeight:
    """Rows [a, b) of a quantized matrix (column-parallel TP shard: tp_take_rows, grimoire.cpp:5256)."""
    sc = qw.scales[a:b] if qw.scales is not None else None
    zr = qw.zeros[a:b] if qw.zeros is not None else None
    return QuantWeight(qw.fmt, b - a, qw.K, qw.payload[a:b].contiguous(), scales=None if sc is None else sc.contiguous(),
                       zeros=None if zr is None else zr.contiguous(), group=qw.group, global_scale=qw.global_scale)


def slice_cols(qw: QuantWeight, a: int, b: int) -> QuantWeight:
    """K columns [a, b) of a quantized matrix (row-parallel TP shard: tp_take_cols,
    grimoire.cpp:5300-5346).  The cut must fall on scale-group boundaries."""
    f = qw.fmt
    if f == Fmt.BF16:
        return QuantWeight(f, qw.N, b - a, qw.payload.reshape(qw.N, qw.K, 2)[:, a:b].reshape(qw.N, -1).contiguous())
    per_row_scale = f in (Fmt.INT8, Fmt.FP8_E4M3, Fmt.FP8_E5M2)
    bits4 = f in (Fmt.INT4, Fmt.MXFP4, Fmt.NVFP4)
    g = 1 if per_row_scale else qw.group
    if a % g or b % g or (bits4 and (a % 2 or b % 2)):
        raise ValueError(f"column slice [{a},{b}) does not fall on group boundaries of {g}")
    pay = qw.payload[:, a // 2: b // 2] if bits4 else qw.payload[:, a:b]
    sc = qw.scales if per_row_scale else qw.scales[:, a // g: b // g]
    zr = None if qw.zeros is None else qw.zeros[:, a // g: b // g].contiguous()
    return QuantWeight(f, qw.N, b - a, pay.contiguous(), scales=sc.contiguous(), zeros=zr, group=qw.group,
                       global_scale=qw.global_scale)
