"""GPTQ / AutoGPTQ / AutoRound 4-bit checkpoint triples.

Checkpoint layout (include/b70/gptq.hpp:22-52,80-93 documents the same convention):
  qweight I32 ``[in/8][out]``   eight 4-bit codes per word packed along IN (code i in bits 4i..4i+3)
  qzeros  I32 ``[in/g][out/8]`` eight 4-bit zero codes per word packed along OUT, stored as zero-1
  scales  F16 ``[in/g][out]``
  w[out][in] = (code - (zcode + 1)) * scale            (the "+1" is the silent-when-wrong part)
The group size is derived from the scales shape, not from the config
(src/qwen35_loader.cpp:1584-1607).  ``g_idx`` (act-order) is accepted only when it is the trivial
``k // g`` map.

Unlike the reference's repack (src/gptq.cpp:26-84), the fp16 scales are kept as fp16 all the way
to the kernel, which converts them to fp32 exactly.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import codecs as C
from .codecs import Fmt
from .quantize import QuantWeight


def gptq_group_size(qweight: torch.Tensor, scales: torch.Tensor) -> int:
    in_features = qweight.shape[0] * 8
    groups = scales.shape[0]
    if groups <= 0 or in_features % groups:
        raise ValueError(f"GPTQ: {in_features} input features not divisible into {groups} groups")
    return in_features // groups


def _unpack_i32_nibbles(words: torch.Tensor, dim: int) -> torch.Tensor:
    """Expand int32 words into 8 nibbles along ``dim`` (nibble i = bits 4i..4i+3)."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, dtype=torch.int64) * 4
    if dim == 0:       # [R][C] -> [R*8][C]
        out = (w[:, None, :] >> shifts[None, :, None]) & 0xF
        return out.reshape(w.shape[0] * 8, w.shape[1])
    out = (w[:, :, None] >> shifts[None, None, :]) & 0xF     # [R][C] -> [R][C*8]
    return out.reshape(w.shape[0], w.shape[1] * 8)


def _pack_i32_nibbles(codes: torch.Tensor, dim: int) -> torch.Tensor:
    c = codes.to(torch.int64) & 0xF
    shifts = torch.arange(8, dtype=torch.int64) * 4
    if dim == 0:
        c = c.reshape(c.shape[0] // 8, 8, c.shape[1])
        w = (c << shifts[None, :, None]).sum(dim=1)
    else:
        c = c.reshape(c.shape[0], c.shape[1] // 8, 8)
        w = (c << shifts[None, None, :]).sum(dim=2)
    w = torch.where(w >= 2 ** 31, w - 2 ** 32, w)
    return w.to(torch.int32)


def gptq_unpack(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                g_idx: Optional[torch.Tensor] = None) -> QuantWeight:
    """GPTQ triple -> logical INT4 QuantWeight ``[out][in]`` (zero = stored code + 1)."""
    group = gptq_group_size(qweight, scales)
    K = qweight.shape[0] * 8
    N = qweight.shape[1]
    if g_idx is not None:
        trivial = torch.arange(K, dtype=g_idx.dtype) // group
        if not torch.equal(g_idx.cpu(), trivial):
            raise ValueError("GPTQ act-order (non-trivial g_idx) checkpoints are not supported")
    q = _unpack_i32_nibbles(qweight.cpu(), 0).t().contiguous()          # [N][K]
    # zero = stored code + 1 in 1..16 with no wrap: a stored 15 means 16 (src/gptq.cpp:44 dequantises with
    # znib + 1, :73 repacks uint8(z + 1)); zeros travel as bytes, so 16 needs no special case downstream
    z = _unpack_i32_nibbles(qzeros.cpu(), 1) + 1                        # [K/g][N]
    zeros = z[:, :N].t().contiguous().to(torch.uint8)                   # [N][K/g]
    sc = scales.cpu().t().contiguous().half()                           # [N][K/g]
    return QuantWeight(Fmt.INT4, N, K, C.pack_nibbles(q.to(torch.uint8)), scales=sc, zeros=zeros, group=group)


def gptq_pack(qw: QuantWeight):
    """Logical INT4 QuantWeight -> (qweight, qzeros, scales) GPTQ triple (for synthetic checkpoints)."""
    if qw.fmt != Fmt.INT4:
        raise ValueError("gptq_pack needs an INT4 weight")
    q = C.unpack_nibbles(qw.payload)                                    # [N][K]
    qweight = _pack_i32_nibbles(q.t().contiguous(), 0)                  # [K/8][N]
    if int(qw.zeros.min()) < 1 or int(qw.zeros.max()) > 16:
        raise ValueError("GPTQ stores zero - 1 in 4 bits: only zero points 1..16 can be written")
    zc = (qw.zeros.to(torch.int64) - 1).t().contiguous()                # [K/g][N]
    if zc.shape[1] % 8:
        raise ValueError("out features must be a multiple of 8 for GPTQ qzeros packing")
    qzeros = _pack_i32_nibbles(zc, 1)                                   # [K/g][N/8]
    scales = qw.scales.t().contiguous().half()                          # [K/g][N]
    return qweight, qzeros, scales


def gptq_dequant_4bit(qweight, qzeros, scales, g_idx=None) -> torch.Tensor:
    """fp32 ``[out][in]`` dequantisation of a GPTQ triple (oracle; cf. src/gptq.cpp:26)."""
    return gptq_unpack(qweight, qzeros, scales, g_idx).dequant()
