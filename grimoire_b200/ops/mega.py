"""Single-row decode of a dense int4 model through the persistent phase kernel (``decode_mega.cu``).

The projections of one decode token are described once, at model load, as a device-resident table of phases
(weight, prologue, epilogue); a launch then runs a run of consecutive phases with grid barriers in between while
the producer warps keep streaming weights across the boundaries.  Launch plan for L layers (attention stays its own
kernel between the launches)::

    [qkv_0]  attn_0  [o_0 | gate_up_0 | down_0 | qkv_1]  attn_1  ...  [o_L-1 | gate_up_L-1 | down_L-1 | head]

which is 2 launches per layer instead of 5 (the reference records ~29 per layer into its command graph,
src/grimoire.cpp:23640-23712).  Under tensor parallelism the o / down phases all-reduce in their epilogue.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .. import _native
from .linear import W4Linear

MEGA = os.environ.get("GRIMOIRE_MEGA", "0") != "0"     # opt-in until it beats the per-projection kernels
COOP = 1 if os.environ.get("GRIMOIRE_MEGA_COOP", "1") != "0" else 0    # cooperative launch (co-residency guaranteed)
PRO_X, PRO_NORM = 0, 1
EPI_BF16, EPI_F32, EPI_ADD, EPI_SWIGLU = 0, 1, 2, 3
MAX_K = 20480


class MegaPhase(ctypes.Structure):
    _fields_ = [("w", ctypes.c_void_p), ("sz", ctypes.c_void_p), ("x", ctypes.c_void_p), ("nw", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("N", ctypes.c_int), ("rp", ctypes.c_int), ("K", ctypes.c_int), ("g64", ctypes.c_int),
                ("pro", ctypes.c_int), ("epi", ctypes.c_int), ("eps", ctypes.c_float), ("offset", ctypes.c_float),
                ("ar_region", ctypes.c_int), ("pad", ctypes.c_int)]


def _phase(lin: W4Linear, pro: int, epi: int, x, nw, out, eps: float, offset: float, ar_region: int = -1) -> MegaPhase:
    t = lin.tiled
    ph = MegaPhase()
    ph.w, ph.sz = t.w.data_ptr(), t.sz.data_ptr()
    ph.x = 0 if x is None else x.data_ptr()
    ph.nw = 0 if nw is None else nw.data_ptr()
    ph.out = out.data_ptr()
    ph.N, ph.rp, ph.K, ph.g64 = lin.N, t.N // 32, t.K, t.group // 64
    ph.pro, ph.epi, ph.eps, ph.offset, ph.ar_region, ph.pad = pro, epi, eps, offset, ar_region, 0
    return ph


def linear_ok(lin) -> bool:
    return (isinstance(lin, W4Linear) and lin.tiled is not None and lin.tiled.K <= MAX_K and lin.tiled.K % 64 == 0
            and lin.tiled.group in (64, 128, 256))


class MegaTable:
    """Phase table + scratch of one (model, activation buffers) pair."""

    def __init__(self, phases: list[MegaPhase], device, h: torch.Tensor, tp=None):
        lib = _native.cuda()
        assert lib.grm_mega_phase_bytes() == ctypes.sizeof(MegaPhase)
        self.device = torch.device(device)
        self.n = len(phases)
        raw = b"".join(bytes(p) for p in phases)
        self.table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(self.device)
        self.h = h
        self.sync = torch.zeros(4, dtype=torch.int32, device=self.device)
        if os.environ.get("GRIMOIRE_MEGA_BPS"):
            lib.grm_mega_set_ctas_per_sm(int(os.environ["GRIMOIRE_MEGA_BPS"]))
        grid = lib.grm_mega_grid()
        self.max_k = max(p.K for p in phases)
        self.pstride = max(1, max(lib.grm_mega_max_parts(p.rp, p.K, grid) for p in phases) - 1)
        max_rp = max(p.rp for p in phases)
        self.parts = torch.zeros(max_rp * self.pstride * 32 * 2, dtype=torch.float32, device=self.device)    # {value, epoch} pairs
        self.tp = tp
        self.spin = int(os.environ.get("GRIMOIRE_MEGA_SPIN", "0"))
        if os.environ.get("GRIMOIRE_MEGA_SLOTS"):
            lib.grm_mega_set_slot_cap(int(os.environ["GRIMOIRE_MEGA_SLOTS"]))
        self.grid = grid

    def run(self, first: int, count: int, timeline: Optional[torch.Tensor] = None) -> None:
        """Launch phases [first, first + count).  ``timeline``: int64 [count][grid][5] device tensor that receives the SM
        clock of every CTA's thread 0 at: phase entered, grid barrier passed, activations staged, last ring stage
        consumed, row pairs finalised (diagnostics; None in normal operation)."""
        tp = self.tp
        recv, world, rank, rows = None, 1, 0, 0
        if tp is not None:
            recv, world, rank, rows = tp.mega_recv.ptr_array(), tp.world, tp.rank, tp.mega_rows
        code = _native.cuda().grm_decode_mega(
            _native.ptr(self.table), ctypes.c_int(first), ctypes.c_int(count), _native.ptr(self.h), _native.ptr(self.sync),
            _native.ptr(self.parts), ctypes.c_int(self.pstride), ctypes.c_int(self.max_k), recv,
            ctypes.c_int(world), ctypes.c_int(rank), ctypes.c_int(rows), ctypes.c_uint(self.spin), ctypes.c_int(COOP), _native.ptr(timeline), _native.stream_ptr())
        _native.check(code, f"decode_mega phases {first}..{first + count - 1}")

    def reset(self) -> None:
        """Clear the barrier words after a reported timeout (the arrival count may be left mid-way)."""
        self.sync.zero_()
        self.parts.zero_()


def dense_supported(model) -> bool:
    """Every projection is a tiled int4 weight, plain (ungated) attention, no pipeline stages, and under tensor
    parallelism the fused exchange buffers exist."""
    if not MEGA or model.device.type != "cuda" or model.pp_world != 1 or model.geom.q_gated or not model.layers:
        return False
    for L in model.layers:
        if not (linear_ok(L.qkv) and linear_ok(L.o) and linear_ok(L.gate_up) and linear_ok(L.down) and L.gate_up.swiglu):
            return False
    if model.tp is not None and (not model.tp.fused or getattr(model.tp, "mega_recv", None) is None):
        return False
    return True


def build_dense_table(model, buf) -> MegaTable:
    """Phases of one decode token of ``model`` over the activation buffers ``buf`` (row 0)."""
    cfg = model.cfg
    eps, off = cfg.rms_norm_eps, cfg.norm_offset
    h, qkv, attn, act = buf.h[0], buf.qkv[0], buf.attn[0], buf.act[0]
    tp = model.tp
    ar = (0, 1) if tp is not None else (-1, -1)
    phases: list[MegaPhase] = []
    layers = model.layers
    phases.append(_phase(layers[0].qkv, PRO_NORM, EPI_BF16, None, layers[0].in_norm, qkv, eps, off))
    for i, L in enumerate(layers):
        phases.append(_phase(L.o, PRO_X, EPI_ADD, attn, None, h, eps, off, ar[0]))
        phases.append(_phase(L.gate_up, PRO_NORM, EPI_SWIGLU, None, L.post_norm, act, eps, off))
        phases.append(_phase(L.down, PRO_X, EPI_ADD, act, None, h, eps, off, ar[1]))
        if i + 1 < len(layers):
            phases.append(_phase(layers[i + 1].qkv, PRO_NORM, EPI_BF16, None, layers[i + 1].in_norm, qkv, eps, off))
    head_in_table = linear_ok(model.lm_head) and not model.lm_head.swiglu
    if head_in_table:
        v0 = model.head_split[0] if getattr(model, "head_split", None) else 0      # a vocabulary shard writes its columns
        phases.append(_phase(model.lm_head, PRO_NORM, EPI_F32, None, model.final_norm, buf.logits[0, v0:], eps, off))
    t = MegaTable(phases, model.device, h, tp)
    t.head_in_table = head_in_table
    t.n_layers = len(layers)
    return t


def table_for(model, buf) -> Optional[MegaTable]:
    t = getattr(buf, "_mega_table", None)
    if t is None:
        t = build_dense_table(model, buf)
        buf._mega_table = t
    return t
