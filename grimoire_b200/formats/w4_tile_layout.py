"""Execution layout of int4 weights for the sm_100a small-M kernel (``smallm_w4.cu``).

The reference has an analogous load-time re-tiling for its int8 DPAS path (B70Q4, 64x128 tiles,
include/b70/b70q4.hpp, src/b70q4.cpp).  This layout is built for the m16n8k16 bf16 MMA A fragment:

  w  : int32 ``[N/32][K/64][2][32][4]``  -- row tile ``nt = 2*ns + half`` (16 rows), k tile of 64,
       lane ``L`` (g = L//4, t = L%4) owns 4 words; word ``j`` is k16 step ``j``; nibble ``i`` of a
       word is W[16*nt + g + 8*(i&1)][64*kt + 16*t + 4*j + 2*((i>>1)&1) + (i>>2)]: the 16 columns a
       lane needs from a k tile are contiguous, so its activation fragment is two 16-byte reads.
  sz : int32 ``[N/16][K/group][16]``     -- low 16 bits fp16 scale bits, high 16 bits bf16(128+zero).

``interleave_gate_up`` orders a fused gate|up matrix so that row tile 2s holds gate rows
16s..16s+15 and row tile 2s+1 the matching up rows: one warp then owns both halves of 16 SwiGLU
outputs and the activation is applied in registers.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import codecs as C
from .codecs import Fmt
from .quantize import QuantWeight


@dataclass
class W4Tiled:
    """Device-ready int4 weight: tiles + packed scale/zero words."""

    w: torch.Tensor        # int32 [N/32][K/64][2][32][4]
    sz: torch.Tensor       # int32 [N/16][K/group][16]
    N: int
    K: int
    group: int

    def to(self, device) -> "W4Tiled":
        return W4Tiled(self.w.to(device), self.sz.to(device), self.N, self.K, self.group)

    def nbytes(self) -> int:
        return self.w.numel() * 4 + self.sz.numel() * 4


def _nibble_weights(device=None) -> torch.Tensor:
    # nibble index i = r8 + 2*k8 + 4*h ; combined below in (h, k8, r8) order
    i = torch.arange(8, dtype=torch.int64, device=device)
    return (1 << (4 * i)).reshape(2, 2, 2)   # [h][k8][r8]


def tile_w4(qw: QuantWeight) -> W4Tiled:
    """Logical INT4 QuantWeight -> tiled execution layout (pads N up to a multiple of 32)."""
    if qw.fmt != Fmt.INT4:
        raise ValueError("tile_w4 needs an INT4 weight")
    N, K, group = qw.N, qw.K, qw.group
    if K % 64 or group not in (64, 128, 256) or K % group:
        raise ValueError(f"tile_w4: unsupported K={K} group={group}")
    q = C.unpack_nibbles(qw.payload).to(torch.int64)                    # [N][K]
    scales, zeros = qw.scales.half(), qw.zeros.to(torch.int64)
    Np = (N + 31) // 32 * 32
    if Np != N:
        dev = q.device
        q = torch.cat([q, torch.full((Np - N, K), 8, dtype=torch.int64, device=dev)])
        scales = torch.cat([scales, torch.zeros(Np - N, scales.shape[1], dtype=torch.half, device=dev)])
        zeros = torch.cat([zeros, torch.full((Np - N, zeros.shape[1]), 8, dtype=torch.int64, device=dev)])
    NS, KT = Np // 32, K // 64
    # rows: 32*ns + 16*half + 8*r8 + g ; k: 64*kt + 16*t + 4*j + 2*k8 + h
    q9 = q.reshape(NS, 2, 2, 8, KT, 4, 4, 2, 2)         # ns half r8 g kt t j k8 h
    q9 = q9.permute(0, 4, 1, 3, 5, 6, 8, 7, 2)          # ns kt half g t j h k8 r8
    words = (q9 * _nibble_weights(q.device)).sum(dim=(-1, -2, -3))
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    w = words.reshape(NS, KT, 2, 32, 4).contiguous()
    s_bits = scales.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF        # [Np][G]
    z_bits = C.f32_to_bf16_bits((zeros + 128).float()).to(torch.int64) & 0xFFFF   # exact in bf16
    szw = s_bits | (z_bits << 16)
    szw = torch.where(szw >= 2 ** 31, szw - 2 ** 32, szw).to(torch.int32)
    G = K // group
    sz = szw.reshape(Np // 16, 16, G).permute(0, 2, 1).contiguous()      # [N/16][G][16]
    return W4Tiled(w, sz, Np, K, group)


def untile_w4(t: W4Tiled) -> QuantWeight:
    """Inverse of ``tile_w4`` (used by the layout round-trip test and by the CPU oracle)."""
    NS, KT = t.N // 32, t.K // 64
    words = t.w.to(torch.int64) & 0xFFFFFFFF
    shifts = (4 * torch.arange(8, dtype=torch.int64, device=t.w.device)).reshape(2, 2, 2)   # [h][k8][r8]
    q9 = (words.reshape(NS, KT, 2, 8, 4, 4, 1, 1, 1) >> shifts) & 0xF     # ns kt half g t j h k8 r8
    q = q9.permute(0, 2, 8, 3, 1, 4, 5, 7, 6).reshape(t.N, t.K)          # ns half r8 g kt t j k8 h
    szw = t.sz.to(torch.int64) & 0xFFFFFFFF
    G = t.K // t.group
    szr = szw.permute(0, 2, 1).reshape(t.N, G)
    scales = (szr & 0xFFFF).to(torch.int16).view(torch.half)
    zeros = (C.bf16_bits_to_f32(((szr >> 16) & 0xFFFF).to(torch.int32)) - 128).to(torch.uint8)
    return QuantWeight(Fmt.INT4, t.N, t.K, C.pack_nibbles(q.to(torch.uint8)), scales=scales, zeros=zeros,
                       group=t.group)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stack gate ``[I][...]`` and up ``[I][...]`` as [16 gate rows, 16 up rows, 16 gate rows, ...]."""
    I = gate.shape[0]
    if I % 16 or up.shape != gate.shape:
        raise ValueError("gate/up must have equal shapes with rows a multiple of 16")
    g = gate.reshape(I // 16, 1, 16, *gate.shape[1:])
    u = up.reshape(I // 16, 1, 16, *up.shape[1:])
    return torch.cat([g, u], dim=1).reshape(2 * I, *gate.shape[1:])


def concat_rows(parts: list[QuantWeight]) -> QuantWeight:
    """Row-wise concatenation of INT4 weights with equal K and group (fused q|k|v, gate|up), the
    counterpart of concat_rows_quantized_t (grimoire.cpp:1960)."""
    f = parts[0]
    for p in parts:
        if p.fmt != f.fmt or p.K != f.K or p.group != f.group:
            raise ValueError("concat_rows: mismatched weights")
    return QuantWeight(f.fmt, sum(p.N for p in parts), f.K, torch.cat([p.payload for p in parts]),
                       scales=None if f.scales is None else torch.cat([p.scales for p in parts]),
                       zeros=None if f.zeros is None else torch.cat([p.zeros for p in parts]), group=f.group)


def interleave_gate_up_q(gate: QuantWeight, up: QuantWeight) -> QuantWeight:
    """Quantized version of ``interleave_gate_up`` (rows permuted, codes untouched)."""
    return QuantWeight(gate.fmt, gate.N * 2, gate.K, interleave_gate_up(gate.payload, up.payload),
                       scales=None if gate.scales is None else interleave_gate_up(gate.scales, up.scales),
                       zeros=None if gate.zeros is None else interleave_gate_up(gate.zeros, up.zeros), group=gate.group)


def tile_mx(qw: QuantWeight):
    """MXFP4 ``[N][K]`` (payload [N][K/2] bytes, even k in the low nibble; e8m0 scales [N][K/32]) -> the execution
    layout of the tiled small-M kernel.  Returns (w int32 [N/32][K/64][2][32][4], sz uint8 [N/16][K/32][16]).

    A lane's 32-bit word j of a k tile holds the four A-fragment bytes of k16 step j: byte b = 2*hi + r8 is row
    ``16*half + g + 8*r8`` and the column pair ``16 j + 2 t + 8 hi`` (+1) of the tile, so one hardware e2m1x2 -> f16x2
    conversion per byte yields the fragment registers (a0, a1, a2, a3) in order."""
    if qw.fmt != Fmt.MXFP4 or qw.N % 32 or qw.K % 64:
        raise ValueError("tile_mx needs an MXFP4 weight with N % 32 == 0 and K % 64 == 0")
    N, K = qw.N, qw.K
    P = qw.payload.reshape(N // 32, 2, 2, 8, K // 64, 4, 2, 4)          # (rt, half, r8, g, kt, j, hi, t)
    w = P.permute(0, 4, 1, 3, 7, 5, 6, 2).contiguous()                  # (rt, kt, half, g, t, j, hi, r8)
    w = w.reshape(N // 32, K // 64, 2, 32, 16).view(torch.int32).reshape(N // 32, K // 64, 2, 32, 4)
    sz = qw.scales.reshape(N // 16, 16, K // 32).permute(0, 2, 1).contiguous()
    return w, sz
