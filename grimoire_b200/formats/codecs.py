"""Bit-exact element codecs (torch, vectorised): bf16, E8M0, E2M1, E4M3, E5M2 and the format table.

Same role as the reference's SYCL-free codec header (include/b70/formats.hpp:65-246), which both its
host tests and its device code compile; here the torch versions are the oracle for the CUDA
kernels' in-register decoders and for the C++ codecs in csrc/host/codecs.hpp.
"""
from __future__ import annotations

import enum

import torch


class Fmt(enum.IntEnum):
    """Weight formats.  Numbering follows include/b70/formats.hpp:237-239 and is extended with
    the block-scaled fp8 (e4m3, 1x128 scales) and NVFP4 formats this engine adds."""

    BF16 = 0
    FP8_E4M3 = 1
    FP8_E5M2 = 2
    INT8 = 3
    INT4 = 4
    MXFP8 = 5
    MXFP4 = 6
    Q4_K = 7
    Q6_K = 8
    Q5_K = 9
    Q8_0 = 10
    IQ4_XS = 11
    IQ4_NL = 12
    FP8_BLOCK = 13   # e4m3 payload, fp32 scale per 1x128 block along K
    NVFP4 = 14       # e2m1 payload, e4m3 scale per 16, fp32 global scale


MX_BLOCK = 32        # elements per E8M0 scale (formats.hpp:245)
INT4_GROUP = 128     # default int4 group (formats.hpp:246)
NVFP4_BLOCK = 16
FP8_BLOCK_K = 128

PROJ_NAMES = {
    "int4": Fmt.INT4, "int8": Fmt.INT8, "mxfp4": Fmt.MXFP4, "mxfp8": Fmt.MXFP8,
    "fp8": Fmt.FP8_E4M3, "fp8_e4m3": Fmt.FP8_E4M3, "fp8-e4m3": Fmt.FP8_E4M3,
    "fp8_e5m2": Fmt.FP8_E5M2, "fp8-e5m2": Fmt.FP8_E5M2, "bf16": Fmt.BF16,
    "fp8_block": Fmt.FP8_BLOCK, "nvfp4": Fmt.NVFP4,
}

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def bits_per_elem(fmt: Fmt, group: int = INT4_GROUP) -> float:
    """Storage cost including scales (cf. formats.hpp:503-558)."""
    return {
        Fmt.BF16: 16.0, Fmt.FP8_E4M3: 8.0, Fmt.FP8_E5M2: 8.0, Fmt.INT8: 8.0,
        Fmt.INT4: 4.0 + 24.0 / group, Fmt.MXFP8: 8.0 + 8.0 / MX_BLOCK, Fmt.MXFP4: 4.0 + 8.0 / MX_BLOCK,
        Fmt.FP8_BLOCK: 8.0 + 32.0 / FP8_BLOCK_K, Fmt.NVFP4: 4.0 + 8.0 / NVFP4_BLOCK,
        Fmt.Q4_K: 4.5, Fmt.Q5_K: 5.5, Fmt.Q6_K: 6.5625, Fmt.Q8_0: 8.5, Fmt.IQ4_XS: 4.25, Fmt.IQ4_NL: 4.5,
    }[fmt]


# ---- bf16 ------------------------------------------------------------------------------------
def f32_to_bf16_bits(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (int32 holding 16 bits); NaN stays NaN."""
    u = x.float().contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    lsb = (u >> 16) & 1
    r = (u + 0x7FFF + lsb) >> 16
    nan = torch.isnan(x.float())
    r = torch.where(nan, torch.full_like(r, 0x7FC0), r)
    return (r & 0xFFFF).to(torch.int32)


def bf16_bits_to_f32(b: torch.Tensor) -> torch.Tensor:
    return ((b.to(torch.int64) & 0xFFFF) << 16).to(torch.int32).view(torch.float32)


# ---- E8M0 (power-of-two block scale) ------------------------------------------------------------
def e8m0_to_f32(e: torch.Tensor) -> torch.Tensor:
    """2^(e-127); 255 decodes to NaN (formats.hpp:105-109)."""
    e = e.to(torch.int32)
    out = torch.pow(torch.tensor(2.0, dtype=torch.float64, device=e.device), (e - 127).double()).float()
    return torch.where(e == 255, torch.full_like(out, float("nan")), out)


def pick_e8m0(amax: torch.Tensor, emax_elem: int) -> torch.Tensor:
    """OCP MX shared exponent: clamp(floor(log2 amax) - emax_elem + 127, 0, 254)
    (src/quantize.cpp:45-56).  amax == 0 maps to exponent 0... kept at 127 (scale 1) instead so an
    all-zero block decodes to zeros with a finite scale."""
    amax = amax.float()
    safe = torch.where(amax > 0, amax, torch.ones_like(amax))
    e = torch.floor(torch.log2(safe.double())).to(torch.int32) - emax_elem + 127
    # guard log2 rounding at exact powers of two
    two = torch.tensor(2.0, dtype=torch.float64, device=amax.device)
    up = torch.pow(two, (e + 1 - 127 + emax_elem).double())
    e = torch.where(safe.double() >= up, e + 1, e)
    lo = torch.pow(two, (e - 127 + emax_elem).double())
    e = torch.where(safe.double() < lo, e - 1, e)
    e = e.clamp(0, 254)
    return torch.where(amax > 0, e, torch.full_like(e, 127)).to(torch.uint8)


# ---- E2M1 (fp4) --------------------------------------------------------------------------------
def e2m1_to_f32(code: torch.Tensor) -> torch.Tensor:
    code = code.to(torch.int64)
    tbl = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=code.device)
    mag = tbl[code & 7]
    return torch.where((code & 8) != 0, -mag, mag)


def f32_to_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto {0,.5,1,1.5,2,3,4,6} with saturation (formats.hpp:129-151)."""
    x = x.float()
    a = x.abs()
    # decision thresholds are the midpoints; ties go to the even code (mantissa bit 0)
    code = torch.zeros_like(a, dtype=torch.int64)
    mids = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)
    for i, m in enumerate(mids):
        nxt = i + 1
        if nxt % 2 == 0:   # next code is even: a tie rounds up to it
            code = torch.where(a >= m, torch.full_like(code, nxt), code)
        else:              # next code is odd: a tie stays on the even code below
            code = torch.where(a > m, torch.full_like(code, nxt), code)
    code = torch.where(torch.isnan(a), torch.full_like(code, 7), code)
    sign = (torch.signbit(x)).to(torch.int64) << 3
    return (code | sign).to(torch.uint8)


# ---- fp8 -----------------------------------------------------------------------------------------
E4M3_MAX = 448.0
E5M2_MAX = 57344.0


def f32_to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """RNE with saturation to +-448 (formats.hpp:171-195); returns uint8 codes."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).view(torch.uint8)


def e4m3_to_f32(code: torch.Tensor) -> torch.Tensor:
    return code.to(torch.uint8).view(torch.float8_e4m3fn).float()


def f32_to_e5m2(x: torch.Tensor) -> torch.Tensor:
    return x.float().clamp(-E5M2_MAX, E5M2_MAX).to(torch.float8_e5m2).view(torch.uint8)


def e5m2_to_f32(code: torch.Tensor) -> torch.Tensor:
    return code.to(torch.uint8).view(torch.float8_e5m2).float()


# ---- nibble packing ------------------------------------------------------------------------------
def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] 4-bit codes -> [..., K/2] bytes, even element in the low nibble."""
    c = codes.to(torch.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).contiguous()


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    p = packed.to(torch.uint8)
    out = torch.stack((p & 0xF, p >> 4), dim=-1)
    return out.reshape(*p.shape[:-1], p.shape[-1] * 2)
