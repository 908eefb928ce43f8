"""Row-block int4 layout for the tensor-core decode stream (csrc/kernels/gemv_w4_tc.cu).

The weight ``[N][K]`` (group 128) is cut into stages of 128 rows x 128 k.  One stage is one contiguous 8704-byte record
-- one bulk copy into shared memory -- laid out for a thread that owns ONE row:

* bytes [0, 8192): row r (0..127) owns 64 bytes = four 16-byte chunks; chunk i covers k in [32 i, 32 i + 32) and sits at
  position ``i ^ ((r >> 1) & 3)`` of the row's 64 bytes, so that the 16-byte reads of eight neighbouring rows fall into
  eight different bank groups.  Inside a chunk, 32-bit word j holds k0 = 32 i + 8 j .. k0 + 7: byte b carries k0 + b in
  its low nibble and k0 + 4 + b in its high nibble, so ``w & 0x0f0f0f0f`` and ``(w >> 4) & 0x0f0f0f0f`` are the two
  32-bit columns (four consecutive k each, in order) of the tensor-memory A operand -- three logic operations for
  eight weights;
* bytes [8192, 8704): one word per row, fp16 scale | bf16(128 + zero) << 16 (the encoding of w4_tile_layout).

Records are ordered ``[N / 128][K / 128]``: the stages of one row block are consecutive, which is the order the
persistent kernel walks them in.  The reference has no counterpart (its int4 GEMV reads the checkpoint layout,
src/gemv_decode.cpp:77-347); this layout exists because the unpack cost per weight decides whether one row of
activations can be fed to the tensor cores at the memory rate.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import codecs as C
from .codecs import Fmt
from .quantize import QuantWeight

ROWS = 128
KSTEP = 128
STAGE_BYTES = ROWS * KSTEP // 2 + ROWS * 4


@dataclass
class W4RowBlock:
    data: torch.Tensor      # uint8 [N/128][K/128][8704]
    N: int                  # padded to a multiple of 128
    K: int
    rows: int               # logical rows

    def to(self, device) -> "W4RowBlock":
        return W4RowBlock(self.data.to(device), self.N, self.K, self.rows)

    def nbytes(self) -> int:
        return self.data.numel()


def supported(qw: QuantWeight) -> bool:
    return qw.fmt == Fmt.INT4 and qw.group == 128 and qw.K % 128 == 0 and qw.K <= 20480


def pack_rowblock(qw: QuantWeight) -> W4RowBlock:
    """Logical INT4 QuantWeight (group 128) -> row-block records (N padded to 128 with zero-scale rows)."""
    if not supported(qw):
        raise ValueError("pack_rowblock needs an INT4 weight with group 128 and K a multiple of 128 (<= 20480)")
    N, K = qw.N, qw.K
    q = C.unpack_nibbles(qw.payload).to(torch.int64)                    # [N][K]
    scales, zeros = qw.scales.half(), qw.zeros.to(torch.int64)
    Np = (N + ROWS - 1) // ROWS * ROWS
    if Np != N:
        dev = q.device
        q = torch.cat([q, torch.full((Np - N, K), 8, dtype=torch.int64, device=dev)])
        scales = torch.cat([scales, torch.zeros(Np - N, scales.shape[1], dtype=torch.half, device=dev)])
        zeros = torch.cat([zeros, torch.full((Np - N, zeros.shape[1]), 8, dtype=torch.int64, device=dev)])
    NB, KG = Np // ROWS, K // KSTEP
    # k = 128 kg + 32 i + 8 j + 4 h + b   ->   [nb][r][kg][i][j][h][b]
    q7 = q.reshape(NB, ROWS, KG, 4, 4, 2, 4)
    byte = (q7[..., 0, :] | (q7[..., 1, :] << 4)).to(torch.uint8)      # [nb][r][kg][i][j][b]
    byte = byte.permute(0, 2, 1, 3, 4, 5).reshape(NB, KG, ROWS, 4, 16)  # [nb][kg][r][chunk i][16 bytes]
    r = torch.arange(ROWS, device=q.device)
    pos = torch.arange(4, device=q.device)[None, :] ^ ((r[:, None] >> 1) & 3)      # [r][i] -> physical position
    phys = torch.empty_like(byte)
    phys.scatter_(3, pos[None, None, :, :, None].expand(NB, KG, ROWS, 4, 16), byte)
    s_bits = scales.contiguous().view(torch.int16).to(torch.int64) & 0xFFFF        # [Np][KG]
    z_bits = C.f32_to_bf16_bits((zeros + 128).float()).to(torch.int64) & 0xFFFF
    szw = (s_bits | (z_bits << 16)).reshape(NB, ROWS, KG).permute(0, 2, 1)         # [nb][kg][r]
    szb = torch.stack([(szw >> (8 * i)) & 0xFF for i in range(4)], dim=-1).to(torch.uint8).reshape(NB, KG, ROWS * 4)
    data = torch.cat([phys.reshape(NB, KG, ROWS * 64), szb], dim=2).contiguous()
    assert data.shape[2] == STAGE_BYTES
    return W4RowBlock(data, Np, K, N)


def unpack_rowblock(t: W4RowBlock) -> QuantWeight:
    """Inverse of ``pack_rowblock`` (layout round-trip test, CPU oracle)."""
    NB, KG = t.N // ROWS, t.K // KSTEP
    d = t.data.cpu()
    phys = d[:, :, : ROWS * 64].reshape(NB, KG, ROWS, 4, 16)
    r = torch.arange(ROWS)
    pos = torch.arange(4)[None, :] ^ ((r[:, None] >> 1) & 3)
    byte = torch.gather(phys, 3, pos[None, None, :, :, None].expand(NB, KG, ROWS, 4, 16)).to(torch.int64)
    b6 = byte.reshape(NB, KG, ROWS, 4, 4, 4)                            # [nb][kg][r][i][j][b]
    q7 = torch.stack([b6 & 0xF, b6 >> 4], dim=-2)                       # [nb][kg][r][i][j][h][b]
    q = q7.permute(0, 2, 1, 3, 4, 5, 6).reshape(t.N, t.K)
    szb = d[:, :, ROWS * 64:].reshape(NB, KG, ROWS, 4).to(torch.int64)
    szw = szb[..., 0] | (szb[..., 1] << 8) | (szb[..., 2] << 16) | (szb[..., 3] << 24)
    szr = szw.permute(0, 2, 1).reshape(t.N, KG)
    scales = (szr & 0xFFFF).to(torch.int16).view(torch.half)
    zeros = (C.bf16_bits_to_f32(((szr >> 16) & 0xFFFF).to(torch.int32)) - 128).to(torch.uint8)
    return QuantWeight(Fmt.INT4, t.N, t.K, C.pack_nibbles(q.to(torch.uint8)), scales=scales, zeros=zeros, group=128)
