"""Quantized linear layers: the python face of smallm_w4.cu, dequant.cu and gemm_tcgen05.cu.

``W4Linear`` is the int4-g128 projection.  ``forward`` picks the kernel by row count, the way the
reference's ``mm()`` dispatcher does (grimoire.cpp:21042-21370: GEMV / small-M DPAS / large-M
GEMM): M <= 64 rows run the weight-streaming small-M kernel, larger M dequantizes the weight once
into the shared bf16 scratch and runs the tcgen05 GEMM.  Epilogues are part of the kernels:
``bf16`` store, ``f32`` store, ``add_f32`` (residual stream ``h += y``) and ``swiglu`` (fused
gate|up weight, rows interleaved per 16).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import _native
from ..formats.codecs import Fmt
from ..formats.quantize import QuantWeight
from ..formats.w4_tile_layout import W4Tiled, tile_w4
from ..formats import w4_rowblock
from .workspace import Workspace, default_workspace

EPI = {"bf16": 0, "f32": 1, "add_f32": 2, "swiglu": 3, "rs_push": 4}
SMALLM_MAX = 64
_SMS = 148


def _c(v):
    return ctypes.c_int(int(v))


# GRIMOIRE_W4_I8=1 runs the small-M int4 product on the int8 tensor-core path: activations are carried as
# two int8 levels per weight group (15 bits, a smaller rounding error than bf16 inputs), products are
# exact integers.  Measured on B200 it executes 38 % fewer instructions but is not faster end to end (the
# activation quantisation pass costs what the leaner loop saves), so the bf16 MMA path is the default.
W4_I8 = os.environ.get("GRIMOIRE_W4_I8", "0") != "0"
# MXFP4 small-M products through the tiled kernel (GRIMOIRE_MX_TILED=0: the natural-layout kernel of smallm_mx.cu)
MX_TILED = os.environ.get("GRIMOIRE_MX_TILED", "1") != "0"


GEMV_W4 = os.environ.get("GRIMOIRE_GEMV_W4", "1") != "0"   # single-row int4 projections on the CUDA-core GEMV


FUSED_NORM = os.environ.get("GRIMOIRE_FUSED_NORM", "1") != "0"   # RMSNorm inside the single-row GEMV prologue
# Batch-invariant mode: every batch height (1 row as well as verify blocks and user batches) runs the tensor-core small-M
# kernels, whose per-row arithmetic does not depend on the height, so a row scored alone and the same row scored inside a
# verify block give the same bits -- the contract speculative decoding needs to reproduce plain greedy decoding exactly
# (tools/test_spec_e2e.cpp in the reference).  Switched on by whatever enables speculation (a draft head, copy drafts in
# the scheduler); costs ~20 us of projections per layer on single-row steps, which are rare once drafts are accepted.
BATCH_INVARIANT = False
_GEMV_W4_DEFAULT = GEMV_W4


def set_batch_invariant(on: bool) -> bool:
    """Returns the previous state.  Decode graphs captured in the other mode must be dropped by the caller."""
    global BATCH_INVARIANT, GEMV_W4
    prev = BATCH_INVARIANT
    BATCH_INVARIANT = bool(on)
    GEMV_W4 = False if on else _GEMV_W4_DEFAULT
    return prev


# single-row int4 g128 projections as a tensor-core weight stream (gemv_w4_tc.cu; needs a second copy of the weight in the
# row-block layout): 0 off, 1 on
W4_TC = os.environ.get("GRIMOIRE_W4_TC", "0") != "0"
# every CTA of the fused form re-reads the residual row and the norm weights (60 KB at H = 5120): worth it for a layer's
# projections (a few hundred CTAs), not for a vocabulary-sized head (~9,500 CTAs)
FUSED_NORM_MAX_N = int(os.environ.get("GRIMOIRE_FUSED_NORM_MAX_N", "40960"))


def quant_x_i8(x: torch.Tensor, K: int, group: int, ws: Workspace):
    """bf16 rows -> (hi int8 [M][ldq], lo int8 [M][ldq], table float2 [M][K/group]) in workspace buffers."""
    M = x.shape[0]
    ldq = (K + 15) // 16 * 16
    G = K // group
    hi = ws.get("xq_hi", SMALLM_MAX * ldq, torch.int8).view(-1)[: M * ldq].view(M, ldq)
    lo = ws.get("xq_lo", SMALLM_MAX * ldq, torch.int8).view(-1)[: M * ldq].view(M, ldq)
    tab = ws.get("xq_tab", SMALLM_MAX * G * 2, torch.float32).view(-1)[: M * G * 2].view(M, G * 2)
    code = _native.cuda().grm_quant_x_i8(_native.ptr(x), _c(x.stride(0)), _c(M), _c(K), _c(group), _native.ptr(hi), _native.ptr(lo),
                                         _c(ldq), _native.ptr(tab), _c(G), _native.stream_ptr())
    _native.check(code, f"quant_x_i8 M={M} K={K}")
    return hi, lo, tab


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, epi: str = "bf16", bn: int = 0,
              max_ctas: int = 0, peer_out: Optional[list[int]] = None, my_rank: int = 0) -> torch.Tensor:
    """out = a[M][K] @ b[N][K]^T on the tcgen05 kernel (bf16 in, fp32 accumulate in TMEM)."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    M, K = a.shape
    N = b.shape[0]
    lib = _native.cuda()
    world = 0
    parr = None
    if peer_out is not None:
        world = len(peer_out)
        parr = (ctypes.c_void_p * world)(*peer_out)
    code = lib.grm_gemm_bf16(_native.ptr(a), _c(a.stride(0)), _native.ptr(b), _c(b.stride(0)), _native.ptr(out),
                             _c(out.stride(0)), _c(M), _c(N), _c(K), _c(EPI[epi]), _c(bn), _c(max_ctas), parr,
                             _c(world), _c(my_rank), _native.stream_ptr())
    _native.check(code, f"gemm_bf16 M={M} N={N} K={K} epi={epi}")
    return out


class W4Linear:
    """int4 group-quantized ``[N][K]`` projection resident on one device."""

    def __init__(self, qw: QuantWeight, device, name: str = "", swiglu: bool = False,
                 workspace: Optional[Workspace] = None):
        self.name = name
        self.N, self.K, self.group = qw.N, qw.K, qw.group
        self.rb = None                             # row-block copy for the tensor-core single-row stream (W4_TC)
        self.swiglu = swiglu                       # rows are gate/up interleaved per 16
        self.device = torch.device(device)
        self.ws = workspace or default_workspace(device)
        if self.device.type == "cuda":
            t = tile_w4(qw).to(self.device)
            self.tiled: Optional[W4Tiled] = t
            self.Np = t.N
            self.w_ref = None
            if W4_TC and w4_rowblock.supported(qw) and (not swiglu or qw.N % 32 == 0):
                self.rb = w4_rowblock.pack_rowblock(qw).to(self.device)
        else:
            self.tiled = None
            self.Np = qw.N
            self.w_ref = qw.dequant()              # fp32 oracle weights for the CPU path
        self.out_features = self.N // 2 if swiglu else self.N

    def nbytes(self) -> int:
        return self.tiled.nbytes() if self.tiled is not None else self.w_ref.numel() * 4

    def slice_rows(self, r0: int, n: int) -> "W4Linear":
        """Rows [r0, r0 + n) as a projection of their own (r0 a multiple of 32: whole 32-row tiles are contiguous in the
        tiled layout, so the slice is a copy of a byte range).  Used for the vocabulary-split lm_head."""
        if self.swiglu or r0 % 32 or r0 < 0 or n <= 0 or r0 + n > self.N:
            raise ValueError("slice_rows needs a 32-row aligned start inside a plain projection")
        o = object.__new__(W4Linear)
        o.name, o.K, o.group, o.swiglu, o.device, o.ws = f"{self.name}[{r0}:{r0 + n}]", self.K, self.group, False, self.device, self.ws
        o.N = o.out_features = n
        if self.tiled is not None:
            t = self.tiled
            npad = (n + 31) // 32 * 32
            o.tiled = W4Tiled(t.w[r0 // 32:(r0 + npad) // 32].clone(), t.sz[r0 // 16:(r0 + npad) // 16].clone(), npad, t.K, t.group)
            o.Np, o.w_ref = npad, None
        else:
            o.tiled, o.Np, o.w_ref = None, n, self.w_ref[r0:r0 + n].clone()
        return o

    # -- kernel selection ---------------------------------------------------------------------
    def _plan_smallm(self, M: int):
        tiles32 = self.Np // 32
        rows = 32 if (self.swiglu or tiles32 >= 2 * _SMS) and M <= 16 else 16
        if self.swiglu:
            rows = 32
        tiles = self.Np // rows
        G = self.K // self.group
        ksplit = 1
        if tiles < _SMS and G >= 16:
            want = min(G // 8, max(1, (2 * _SMS) // tiles))
            while want > 1 and G % want:
                want -= 1
            ksplit = max(1, want)
        force = int(os.environ.get("GRIMOIRE_SMALLM_KSPLIT", "0"))      # tuning override
        if force > 0 and G % force == 0 and not self.swiglu:
            ksplit = force
        return rows, ksplit, tiles

    def forward(self, x: torch.Tensor, out: torch.Tensor, epi: str = "bf16") -> torch.Tensor:
        """x bf16 [M][K] -> out (dtype/shape by ``epi``); returns ``out``."""
        M = x.shape[0]
        if self.swiglu and epi != "swiglu":
            raise ValueError("a gate|up interleaved weight must run with the swiglu epilogue")
        if self.device.type != "cuda":
            return self._forward_ref(x, out, epi)
        t = self.tiled
        lib = _native.cuda()
        if M == 1 and not BATCH_INVARIANT and getattr(self, "rb", None) is not None and self._tc_row(x, None, None, out, epi, 0.0, 0.0):
            return out
        if M == 1 and GEMV_W4 and t.K <= 20480:
            # one row: CUDA-core weight stream (gemv_w4.cu); the tensor-core kernel below serves 2..64 rows
            code = lib.grm_gemv_w4(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(out), _c(t.N), _c(t.K), _c(t.group),
                                   _c(EPI[epi]), _native.stream_ptr())
            _native.check(code, f"gemv_w4 {self.name} N={t.N} K={t.K}")
            return out
        if M <= SMALLM_MAX:
            rows, ksplit, tiles = self._plan_smallm(M)
            scratch = counters = None
            if ksplit > 1:
                mt = 1
                while mt * 8 < M:          # the kernel is instantiated for 1, 2, 4 or 8 row tiles
                    mt *= 2
                scratch = self.ws.get("smallm_scratch", ksplit * tiles * (rows // 16) * mt * 128, torch.float32)
                counters = self.ws.get("smallm_counters", 8192, torch.int32, zero=True)
            if W4_I8 and M <= 32:       # wider batches keep the bf16 path (the int8 accumulators would spill)
                xq = quant_x_i8(x, t.K, t.group, self.ws)
                code = lib.grm_smallm_w4_i8(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(xq[0]), _native.ptr(xq[1]), _c(xq[0].stride(0)),
                                            _native.ptr(xq[2]), _c(xq[2].stride(0) // 2), _native.ptr(out), _native.ptr(scratch),
                                            _native.ptr(counters), _c(M), _c(t.N), _c(t.K), _c(out.stride(0)), _c(t.group),
                                            _c(EPI[epi]), _c(rows), _c(ksplit), _native.stream_ptr())
                _native.check(code, f"smallm_w4_i8 {self.name} M={M} N={t.N} K={t.K}")
                return out
            code = lib.grm_smallm_w4(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(out),
                                     _native.ptr(scratch), _native.ptr(counters), _c(M), _c(t.N), _c(t.K),
                                     _c(x.stride(0)), _c(out.stride(0)), _c(t.group), _c(EPI[epi]), _c(rows),
                                     _c(ksplit), _native.stream_ptr())
            _native.check(code, f"smallm_w4 {self.name} M={M} N={t.N} K={t.K}")
            return out
        return gemm_bf16(x, w4_dequant_into(self), out, epi)

    __call__ = forward

    def _tc_row(self, x, h, norm_w, out, epi: str, eps: float, offset: float) -> bool:
        """One row through the tensor-core weight stream (gemv_w4_tc.cu); False when the launcher refuses the shape."""
        rb = self.rb
        lib = _native.cuda()
        lib.grm_gemv_w4_tc_scratch_floats.restype = ctypes.c_long
        lib.grm_gemv_w4_tc_scratch_flags.restype = ctypes.c_long
        partial = self.ws.get("w4tc_partial", int(lib.grm_gemv_w4_tc_scratch_floats(_c(rb.N))), torch.float32)
        flags = self.ws.get("w4tc_flags", max(4096, int(lib.grm_gemv_w4_tc_scratch_flags(_c(rb.N)))), torch.int32, zero=True)
        code = lib.grm_gemv_w4_tc(_native.ptr(rb.data), _native.ptr(x), _native.ptr(h), _native.ptr(norm_w), ctypes.c_float(eps),
                                  ctypes.c_float(offset), _native.ptr(out), _c(self.N), _c(self.K), _c(EPI[epi]), _native.ptr(partial),
                                  _native.ptr(flags), ctypes.c_uint(0), _native.stream_ptr())
        if code == -2:
            return False
        _native.check(code, f"gemv_w4_tc {self.name} N={self.N} K={self.K}")
        return True

    def fused_norm(self, h: torch.Tensor, norm_w: torch.Tensor, out: torch.Tensor, epi: str, eps: float, offset: float) -> bool:
        """``out = epi(RMSNorm(h) @ W^T)`` for one fp32 residual row with the norm inside the GEMV prologue (one launch
        instead of two).  Returns False when the shape or device is not served; the caller then runs norm + forward."""
        t = self.tiled
        if (not BATCH_INVARIANT and getattr(self, "rb", None) is not None and FUSED_NORM and h.shape[0] == 1 and h.dtype == torch.float32 and h.shape[1] == self.K
                and self._tc_row(None, h, norm_w, out, epi, eps, offset)):
            return True
        if (not GEMV_W4 or not FUSED_NORM or self.device.type != "cuda" or t is None or h.shape[0] != 1 or t.K > 20480
                or h.dtype != torch.float32 or h.shape[1] != t.K or t.N > FUSED_NORM_MAX_N):
            return False
        code = _native.cuda().grm_gemv_w4_norm(_native.ptr(t.w), _native.ptr(t.sz), None, _native.ptr(h), _native.ptr(norm_w),
                                               ctypes.c_float(eps), ctypes.c_float(offset), _native.ptr(out), _c(t.N), _c(t.K),
                                               _c(t.group), _c(EPI[epi]), _native.stream_ptr())
        _native.check(code, f"gemv_w4_norm {self.name} N={t.N} K={t.K}")
        return True

    def _forward_ref(self, x, out, epi):
        y = x.bfloat16().float() @ self.w_ref.t()
        if epi == "swiglu":
            I = self.N // 2
            y3 = y.reshape(x.shape[0], I // 16, 2, 16)
            y = (torch.nn.functional.silu(y3[:, :, 0]) * y3[:, :, 1]).reshape(x.shape[0], I)
            out.copy_(y.to(out.dtype))
        elif epi == "add_f32":
            out.add_(y)
        else:
            out.copy_(y.to(out.dtype))
        return out


class BF16Linear:
    """Unquantized bf16 ``[N][K]`` projection (tied lm_head, router, small gate projections).

    M <= 8 rows stream the weight through gemv_bf16.cu; more rows run the tcgen05 GEMM."""

    def __init__(self, w: torch.Tensor, device, name: str = ""):
        self.name = name
        self.w = w.to(device=device, dtype=torch.bfloat16).contiguous()
        self.N, self.K = self.w.shape
        self.device = torch.device(device)
        self.swiglu = False
        self.out_features = self.N

    def nbytes(self) -> int:
        return self.w.numel() * 2

    def slice_rows(self, r0: int, n: int) -> "BF16Linear":
        """Rows [r0, r0 + n) as a projection of their own (a view: a tied lm_head keeps sharing the embedding table)."""
        o = object.__new__(BF16Linear)
        o.name, o.w, o.device, o.swiglu = f"{self.name}[{r0}:{r0 + n}]", self.w[r0:r0 + n], self.device, False
        o.N, o.K = o.w.shape
        o.out_features = o.N
        return o

    def forward(self, x: torch.Tensor, out: torch.Tensor, epi: str = "bf16") -> torch.Tensor:
        M = x.shape[0]
        if self.device.type != "cuda":
            y = x.bfloat16().float() @ self.w.float().t()
            if epi == "add_f32":
                out.add_(y)
            else:
                out.copy_(y.to(out.dtype))
            return out
        if M <= 8 and epi in ("bf16", "f32", "add_f32"):
            code = _native.cuda().grm_gemv_bf16(_native.ptr(self.w), _native.ptr(x), _native.ptr(out), _c(M), _c(self.N),
                                                _c(self.K), _c(self.w.stride(0)), _c(x.stride(0)), _c(out.stride(0)),
                                                _c(0 if epi == "bf16" else 1), _c(1 if epi == "add_f32" else 0),
                                                _native.stream_ptr())
            _native.check(code, f"gemv_bf16 {self.name}")
            return out
        return gemm_bf16(x, self.w, out, epi)

    __call__ = forward


ROWQ_KIND = {Fmt.BF16: 0, Fmt.INT8: 1, Fmt.FP8_E4M3: 2, Fmt.FP8_E5M2: 3, Fmt.MXFP8: 4}


class RowQLinear:
    """Projection in one of the byte-per-weight formats of ``--proj`` (bf16, int8, fp8 e4m3 / e5m2 with a scale per
    output row, MXFP8 with an e8m0 scale per 32 weights): the reference's int8 / fp8 / mxfp8 / bf16 GEMV and small-M
    rows (src/gemv_decode.cpp:77-347, src/gemm_fast.cpp).  Up to 8 rows stream the weight through smallm_rowq.cu (wider
    small batches in chunks of 8); tall inputs dequantise into the shared bf16 scratch and run the tcgen05 GEMM.
    ``swiglu`` weights are gate/up interleaved per 16 rows, as for the int4 path."""

    def __init__(self, qw: QuantWeight, device, name: str = "", swiglu: bool = False, workspace: Optional[Workspace] = None):
        if qw.fmt not in ROWQ_KIND or qw.K % 32:
            raise ValueError(f"RowQLinear: unsupported weight {qw.fmt!r} K={qw.K}")
        self.name, self.N, self.K, self.swiglu, self.fmt = name, qw.N, qw.K, swiglu, qw.fmt
        self.kind = ROWQ_KIND[qw.fmt]
        self.device = torch.device(device)
        self.ws = workspace or default_workspace(self.device)
        self.out_features = self.N // 2 if swiglu else self.N
        self.w = qw.payload.to(self.device).contiguous()
        self.scale = self.e8 = None
        if qw.fmt == Fmt.MXFP8:
            self.e8 = qw.scales.to(self.device).contiguous()
        elif qw.scales is not None:
            self.scale = qw.scales.float().to(self.device).contiguous()
        self.w_ref = qw.dequant() if self.device.type != "cuda" else None

    def nbytes(self) -> int:
        return self.w.numel() + (0 if self.scale is None else self.scale.numel() * 4) + (0 if self.e8 is None else self.e8.numel())

    def dequant_into_scratch(self) -> torch.Tensor:
        wb = self.ws.get("dequant_bf16", self.N * self.K, torch.bfloat16).view(-1)[: self.N * self.K].view(self.N, self.K)
        code = _native.cuda().grm_dequant_rowq(_native.ptr(self.w), _native.ptr(self.scale), _native.ptr(self.e8), _native.ptr(wb),
                                               _c(self.kind), _c(self.N), _c(self.K), ctypes.c_long(self.w.stride(0)), _c(self.K),
                                               _native.stream_ptr())
        _native.check(code, f"dequant_rowq {self.name}")
        return wb

    def bf16_weights(self, resident_only: bool = False):
        """The bf16 [N][K] form for the tcgen05 GEMM: the resident copy (made on first use while device memory allows, see
        ``_bf16_cache_admit``), else an expansion into the shared scratch (None with ``resident_only``)."""
        cached = getattr(self, "_bf16", None)
        if cached is not None:
            return cached
        if self.kind == 0:
            return None if resident_only else self.dequant_into_scratch()
        if not getattr(self, "_bf16_refused", False) and _bf16_cache_admit(self.N * self.K * 2, self.device):
            self._bf16 = self.dequant_into_scratch().clone()
            return self._bf16
        if not torch.cuda.is_current_stream_capturing():
            self._bf16_refused = True            # (a refusal during graph capture is only "not now")
        return None if resident_only else self.dequant_into_scratch()

    def forward(self, x: torch.Tensor, out: torch.Tensor, epi: str = "bf16") -> torch.Tensor:
        M = x.shape[0]
        if self.swiglu and epi != "swiglu":
            raise ValueError("a gate|up interleaved weight must run with the swiglu epilogue")
        if self.device.type != "cuda":
            return W4Linear._forward_ref(self, x, out, epi)
        if M > SMALLM_MAX:
            return gemm_bf16(x, self.bf16_weights(), out, epi)
        if M >= 4 and self.kind != 0 and not BATCH_INVARIANT and self.bf16_weights(resident_only=True) is not None:
            # 4..64 rows: the row kernel's cost grows with the rows (int8, 27B gate|up: 28-41 us at one row, 184-193 us at
            # eight) and it makes one weight pass per 8 rows; with a resident bf16 copy one pass of the tcgen05 GEMM over 2
            # bytes per weight is cheaper
            return gemm_bf16(x, self.bf16_weights(resident_only=True), out, epi)
        lib = _native.cuda()
        for m0 in range(0, M, 8):
            m = min(8, M - m0)
            code = lib.grm_smallm_rowq(_native.ptr(self.w), _native.ptr(self.scale), _native.ptr(self.e8), _native.ptr(x[m0: m0 + m]),
                                       _native.ptr(out[m0: m0 + m]), _c(self.kind), _c(m), _c(self.N), _c(self.K),
                                       ctypes.c_long(self.w.stride(0)), _c(x.stride(0)), _c(out.stride(0)), _c(EPI[epi]),
                                       _native.stream_ptr())
            _native.check(code, f"smallm_rowq {self.name} M={m} N={self.N} K={self.K}")
        return out

    __call__ = forward


def gemm_bf16_tp(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor], epi: str, *, peer_out=None, peer_cnt=None,
                 world: int = 1, my_rank: int = 0, ag_cnt: Optional[torch.Tensor] = None, ag_expect: int = 0, ldo: int = 0) -> int:
    """Tensor-parallel variants of the tcgen05 GEMM (see grm_gemm_bf16_tp): ``epi='rs_push'`` pushes
    bf16 partial tiles to the owner ranks and counts arrivals; ``ag_cnt`` makes the producer warp
    wait per m tile for rows pushed by their owners.  Returns the number of block columns used."""
    M, K = a.shape
    N = b.shape[0]
    nt = ctypes.c_int(0)
    code = _native.cuda().grm_gemm_bf16_tp(
        _native.ptr(a), _c(a.stride(0)), _native.ptr(b), _c(b.stride(0)), _native.ptr(out), _c(ldo or (out.stride(0) if out is not None else N)),
        _c(M), _c(N), _c(K), _c(EPI[epi]), _c(0), peer_out, peer_cnt, _c(world), _c(my_rank), _native.ptr(ag_cnt),
        ctypes.c_uint(ag_expect & 0xFFFFFFFF), ctypes.byref(nt), _native.stream_ptr())
    _native.check(code, f"gemm_bf16_tp M={M} N={N} K={K} epi={epi}")
    return nt.value


# Resident bf16 copies of int4 projections for the prompt path.  Expanding a weight on every prefill call costs its bf16
# size in writes and again in reads (0.3 ms per 27B layer, a tenth of a 4,096-row chunk on one GPU and a third of it when
# the rows are split over 8 context-parallel replicas); 180 GB holds the 27B model twice over in bf16, so the expansion
# is kept after the first use while free device memory stays above a reserve.  GRIMOIRE_W4_BF16_CACHE_GB: 0 = never,
# N = at most N GB, unset = whatever leaves 24 GB free.
_BF16_CACHE_ENV = os.environ.get("GRIMOIRE_W4_BF16_CACHE_GB", "")
_bf16_cached_bytes = 0


def _bf16_cache_admit(nbytes: int, device) -> bool:
    global _bf16_cached_bytes
    if _BF16_CACHE_ENV == "0":
        return False
    if torch.cuda.is_current_stream_capturing():
        return False
    if _BF16_CACHE_ENV:
        if _bf16_cached_bytes + nbytes > float(_BF16_CACHE_ENV) * 1e9:
            return False
    free, _ = torch.cuda.mem_get_info(device)
    if free - nbytes < 24e9:
        return False
    _bf16_cached_bytes += nbytes
    return True


def w4_dequant_into(lin: "W4Linear") -> torch.Tensor:
    """The bf16 [N][K] form of an int4 (or byte-per-weight) projection for the tcgen05 GEMM: the resident copy when there
    is (room for) one, else an expansion into the shared scratch."""
    if isinstance(lin, RowQLinear):
        return lin.dequant_into_scratch()
    t = lin.tiled
    cached = getattr(lin, "_bf16", None)
    if cached is not None:
        return cached[: lin.N]
    keep = not getattr(lin, "_bf16_refused", False) and _bf16_cache_admit(t.N * t.K * 2, lin.device)
    if keep:
        wbuf = torch.empty(t.N, t.K, dtype=torch.bfloat16, device=lin.device)
    else:
        if not torch.cuda.is_current_stream_capturing():
            lin._bf16_refused = True             # (a refusal during graph capture is only "not now")
        wbuf = lin.ws.get("dequant_bf16", t.N * t.K, torch.bfloat16).view(-1)[: t.N * t.K].view(t.N, t.K)
    code = _native.cuda().grm_dequant_w4(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(wbuf), _c(t.N), _c(t.K), _c(t.group),
                                         _c(t.K), _native.stream_ptr())
    _native.check(code, f"dequant_w4 {lin.name}")
    if keep:
        lin._bf16 = wbuf
    return wbuf[: lin.N]


class MXLinear:
    """MXFP4 ``[N][K]`` projection (e2m1 in blocks of 32 with an e8m0 scale), weights in the
    checkpoint's natural layout.  1..64 rows run the hand-written small-M kernel in passes of 8 rows
    (smallm_mx.cu); taller inputs dequantise once into a bf16 scratch and use the tcgen05 GEMM --
    the reference's policy for its MXFP4 path as well (gemv_mxfp4 for decode, dequant + oneDNN for
    prefill, src/kernels.hpp:163-169, src/gemm_fast.cpp:26-31).  ``swiglu`` weights are gate/up
    interleaved per 16 rows like the int4 ones."""

    def __init__(self, qw: QuantWeight, device, name: str = "", swiglu: bool = False, workspace: Optional[Workspace] = None):
        if qw.fmt != Fmt.MXFP4:
            raise ValueError("MXLinear needs an MXFP4 weight")
        self.name, self.N, self.K, self.swiglu = name, qw.N, qw.K, swiglu
        self.device = torch.device(device)
        self.ws = workspace or default_workspace(device)
        self.tiled = None
        self.out_features = self.N // 2 if swiglu else self.N
        self.tw = self.tsz = None
        if self.device.type == "cuda":
            self.w = qw.payload.to(self.device).contiguous()
            self.s = qw.scales.to(self.device).contiguous()
            self.w_ref = None
            if qw.N % 32 == 0 and qw.K % 64 == 0 and MX_TILED:
                from ..formats.w4_tile_layout import tile_mx

                tw, tsz = tile_mx(qw)
                self.tw, self.tsz = tw.to(self.device), tsz.to(self.device)
        else:
            self.w = self.s = None
            self.w_ref = qw.dequant()

    def nbytes(self) -> int:
        return (self.w.numel() + self.s.numel()) if self.w is not None else self.w_ref.numel() * 4

    def forward(self, x: torch.Tensor, out: torch.Tensor, epi: str = "bf16") -> torch.Tensor:
        M = x.shape[0]
        if self.swiglu and epi != "swiglu":
            raise ValueError("a gate|up interleaved weight must run with the swiglu epilogue")
        if self.device.type != "cuda":
            return W4Linear._forward_ref(self, x, out, epi)
        lib = _native.cuda()
        if M == 1 and GEMV_W4 and self.tw is not None and self.K <= 20480:
            # one row: CUDA-core weight stream over the same tiles (gemv_w4.cu), bf16 activations read directly
            code = lib.grm_gemv_mx(_native.ptr(self.tw), _native.ptr(self.tsz), _native.ptr(x), None, None, ctypes.c_float(0.0),
                                   ctypes.c_float(0.0), _native.ptr(out), _c(self.N), _c(self.K), _c(EPI[epi]), _native.stream_ptr())
            _native.check(code, f"gemv_mx {self.name} N={self.N} K={self.K}")
            return out
        if M <= SMALLM_MAX and self.tw is not None:
            # tiled path: the int4 kernel's ring / warp layout / epilogues with the MXFP4 math
            ld16 = self.K
            x16 = self.ws.get("mx_x16p", SMALLM_MAX * ld16, torch.float16).view(-1)[: M * ld16].view(M, ld16)
            _native.check(lib.grm_x16_lane_order(_native.ptr(x), _c(x.stride(0)), _native.ptr(x16), _c(ld16), _c(M), _c(self.K),
                                                 _native.stream_ptr()), "x16_lane_order")
            rows = 32 if (self.swiglu or self.N // 32 >= 2 * _SMS) and M <= 16 else 16
            code = lib.grm_smallm_mx_tiled(_native.ptr(self.tw), _native.ptr(self.tsz), _native.ptr(x16), _native.ptr(out), None, None,
                                           _c(M), _c(self.N), _c(self.K), _c(ld16), _c(out.stride(0)), _c(EPI[epi]), _c(rows), _c(1),
                                           _native.stream_ptr())
            _native.check(code, f"smallm_mx_tiled {self.name} M={M} N={self.N} K={self.K}")
            return out
        if M <= SMALLM_MAX:
            ld16 = (self.K + 7) // 8 * 8
            x16 = self.ws.get("mx_x16", 8 * ld16, torch.float16)
            code_epi = {"bf16": 0, "f32": 1, "add_f32": 2, "swiglu": 3}[epi]
            for m0 in range(0, M, 8):
                m = min(8, M - m0)
                code = lib.grm_smallm_mx(_native.ptr(self.w), _native.ptr(self.s), _native.ptr(x[m0: m0 + m]), _c(x.stride(0)),
                                         _native.ptr(x16), _c(ld16), _native.ptr(out[m0: m0 + m]), _c(out.stride(0)), _c(m), _c(self.N),
                                         _c(self.K), _c(code_epi), _native.stream_ptr())
                _native.check(code, f"smallm_mx {self.name} M={m} N={self.N} K={self.K}")
            return out
        wbuf = self.ws.get("dequant_bf16", self.N * self.K, torch.bfloat16).view(-1)[: self.N * self.K].view(self.N, self.K)
        _native.check(lib.grm_dequant_mxfp4(_native.ptr(self.w), _native.ptr(self.s), _native.ptr(wbuf), _c(self.N), _c(self.K),
                                            _native.stream_ptr()), f"dequant_mxfp4 {self.name}")
        return gemm_bf16(x, wbuf, out, epi)

    def fused_norm(self, h: torch.Tensor, norm_w: torch.Tensor, out: torch.Tensor, epi: str, eps: float, offset: float) -> bool:
        """RMSNorm of one fp32 residual row inside the single-row GEMV prologue (see W4Linear.fused_norm)."""
        if (not GEMV_W4 or not FUSED_NORM or self.device.type != "cuda" or self.tw is None or h.shape[0] != 1 or self.K > 20480
                or h.dtype != torch.float32 or h.shape[1] != self.K):
            return False
        code = _native.cuda().grm_gemv_mx(_native.ptr(self.tw), _native.ptr(self.tsz), None, _native.ptr(h), _native.ptr(norm_w),
                                          ctypes.c_float(eps), ctypes.c_float(offset), _native.ptr(out), _c(self.N), _c(self.K),
                                          _c(EPI[epi]), _native.stream_ptr())
        _native.check(code, f"gemv_mx_norm {self.name} N={self.N} K={self.K}")
        return True

    __call__ = forward


class GgufLinear:
    """A projection kept as the raw ggml blocks of its GGUF checkpoint (``--proj native`` on a .gguf file): decode steps
    (<= 8 rows) read the stored bytes directly (gemv_gguf.cu; gemv_native_qk, src/gemv_decode.cpp:1216-1274 in the
    reference), taller inputs expand the rows to bf16 for the tcgen05 GEMM.  ``parts`` are (raw uint8 [n][row_bytes], ggml
    type id) in output-row order: fused q|k|v (and gate, up) keep their own block types, each part is one launch writing
    its slice of the output columns.  ``swiglu``: parts are (gate, up) of equal height and the output is silu(gate) * up."""

    def __init__(self, parts, K: int, device, name: str = "", swiglu: bool = False, workspace: Optional[Workspace] = None):
        self.name, self.K, self.swiglu = name, K, swiglu
        self.device = torch.device(device)
        self.ws = workspace or default_workspace(device)
        self.parts = [(raw.to(self.device).contiguous(), int(t)) for raw, t in parts]
        self.N = sum(raw.shape[0] for raw, _ in self.parts)
        if swiglu and (len(self.parts) != 2 or self.parts[0][0].shape[0] != self.parts[1][0].shape[0]):
            raise ValueError("a SwiGLU GgufLinear takes exactly (gate, up) of equal height")
        self.out_features = self.N // 2 if swiglu else self.N

    def nbytes(self) -> int:
        return sum(raw.numel() for raw, _ in self.parts)

    def dequant(self) -> torch.Tensor:
        """fp32 [N][K] through the host decoder (oracle, CPU path)."""
        from ..formats.gguf import dequantize

        return torch.cat([dequantize(t, raw.cpu(), raw.shape[0] * self.K).reshape(raw.shape[0], self.K) for raw, t in self.parts])

    def _rows(self, x, out, epi_code: int, ldo: int, col0: int, part) -> None:
        raw, t = part
        lib = _native.cuda()
        M = x.shape[0]
        esz = out.element_size()
        step = max(1, min(8, (200 * 1024) // (2 * self.K)))       # the kernel stages the rows' activations in shared memory
        for m0 in range(0, M, step):
            m = min(step, M - m0)
            optr = ctypes.c_void_p(out.data_ptr() + (m0 * ldo + col0) * esz)
            code = lib.grm_gemv_gguf(_c(t), _native.ptr(raw), ctypes.c_long(raw.stride(0)), _native.ptr(x[m0: m0 + m]), _c(x.stride(0)), optr,
                                     _c(ldo), _c(m), _c(raw.shape[0]), _c(self.K), _c(epi_code), _native.stream_ptr())
            _native.check(code, f"gemv_gguf {self.name} type={t} M={m} N={raw.shape[0]} K={self.K}")

    def forward(self, x: torch.Tensor, out: torch.Tensor, epi: str = "bf16") -> torch.Tensor:
        M = x.shape[0]
        if self.swiglu != (epi == "swiglu"):
            raise ValueError("the swiglu epilogue goes with a (gate, up) weight and nothing else does")
        if self.device.type != "cuda":
            w = self.dequant()
            y = x.bfloat16().float() @ w.t()
            if self.swiglu:
                I = self.N // 2
                out.copy_((torch.nn.functional.silu(y[:, :I]) * y[:, I:]).to(out.dtype))
            elif epi == "add_f32":
                out.add_(y)
            else:
                out.copy_(y.to(out.dtype))
            return out
        lib = _native.cuda()
        if M > SMALLM_MAX:
            # taller inputs: expand to bf16 once per call and run the tcgen05 GEMM (gate | up as two GEMMs + the product)
            wb = self.ws.get("dequant_bf16", self.N * self.K, torch.bfloat16).view(-1)[: self.N * self.K].view(self.N, self.K)
            r0 = 0
            for raw, t in self.parts:
                code = lib.grm_dequant_gguf(_c(t), _native.ptr(raw), ctypes.c_long(raw.stride(0)), _native.ptr(wb[r0:]), ctypes.c_long(self.K),
                                            _c(raw.shape[0]), _c(self.K), _native.stream_ptr())
                _native.check(code, f"dequant_gguf {self.name}")
                r0 += raw.shape[0]
            if not self.swiglu:
                return gemm_bf16(x, wb, out, epi)
            tmp = self.ws.get("gguf_gu", M * self.N, torch.float32).view(-1)[: M * self.N].view(M, self.N)
            gemm_bf16(x, wb, tmp, "f32")
            I = self.N // 2
            _native.check(lib.grm_swiglu_mul(_native.ptr(tmp), ctypes.c_void_p(tmp.data_ptr() + 4 * I), _native.ptr(out), _c(M), _c(I), _c(self.N),
                                             _c(out.stride(0)), _native.stream_ptr()), "swiglu_mul")
            return out
        if self.swiglu:
            I = self.N // 2
            tmp = self.ws.get("gguf_gu", M * self.N, torch.float32).view(-1)[: M * self.N].view(M, self.N)
            self._rows(x, tmp, 1, self.N, 0, self.parts[0])
            self._rows(x, tmp, 1, self.N, I, self.parts[1])
            _native.check(lib.grm_swiglu_mul(_native.ptr(tmp), ctypes.c_void_p(tmp.data_ptr() + 4 * I), _native.ptr(out), _c(M), _c(I), _c(self.N),
                                             _c(out.stride(0)), _native.stream_ptr()), "swiglu_mul")
            return out
        col = 0
        for part in self.parts:
            self._rows(x, out, EPI[epi], out.stride(0), col, part)
            col += part[0].shape[0]
        return out

    __call__ = forward
