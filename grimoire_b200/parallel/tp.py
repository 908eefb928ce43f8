"""Tensor parallelism ("Megatron" split, one all-reduce per block = two per layer).

Same partitioning as the reference's tp_mega mode (grimoire.cpp:2500-2534, slicing :5256-5368):
each rank *is* the model with 1/W of the q / kv heads and of the FFN width; q|k|v and gate|up keep
row blocks, o_proj and down_proj keep K columns, embeddings / norms / lm_head are replicated and
every rank therefore picks the same token.  What differs is the exchange.  The reference stages
partial sums through host memory (tp_small_allreduce, ~33 us per [1][H] exchange,
grimoire.cpp:6499-6679); here the row-parallel projection and the all-reduce are ONE kernel
(smallm_w4.cu, EPI_AR_ADD): each CTA pushes its partial tile into every peer's receive region over
NVLink, raises a per-(tile, source) flag, waits (bounded) for the peers' flags and sums the W
partials in rank order, so all ranks hold bit-identical results.

Peer memory comes from ``torch.distributed._symmetric_memory`` (allocation + handle exchange only;
all traffic is issued by our kernels).  Rows beyond the small-M kernel's range (prefill chunks) use
the fused GEMM reduce-scatter / all-gather path when available and an NCCL all-reduce otherwise;
the NCCL composition is also the measured baseline (``fused=False``).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from ..ops import linear as L
from ..ops.linear import SMALLM_MAX, W4Linear


class CommTimeout(RuntimeError):
    """A bounded device-side wait on a peer ran out (the kernel returned; the context is usable)."""


class SymmetricBuffer:
    """A tensor allocated at the same offset on every rank, with the peers' mappings."""

    def __init__(self, numel: int, dtype: torch.dtype, group, device):
        import torch.distributed._symmetric_memory as symm_mem

        self.local = symm_mem.empty(numel, dtype=dtype, device=device)
        self.local.zero_()
        self.handle = symm_mem.rendezvous(self.local, group=group.group_name)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.world = len(self.ptrs)

    def ptr_array(self):
        return (ctypes.c_void_p * self.world)(*self.ptrs)


def pick_candidates(vals: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """The split head's decision per row over the ranks' candidates ``vals`` / ``idx`` [M][W]: the highest value, on a
    tie the lowest vocabulary index; an index of INT_MAX (a rank without a finite logit) only wins when every rank has
    none (tp_head_pick_at, src/grimoire.cpp:5421-5449)."""
    bv, bi = vals[:, 0], idx[:, 0]
    for r in range(1, vals.shape[1]):
        cv, ci = vals[:, r], idx[:, r]
        better = (cv > bv) | ((cv == bv) & (ci < bi))
        bv = torch.where(better, cv, bv)
        bi = torch.where(better, ci, bi)
    return bi


class TensorParallel:
    def __init__(self, group, device, fused: Optional[bool] = None):
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if fused is None:
            fused = os.environ.get("GRIMOIRE_TP_FUSED", "1") != "0"
        self.fused = fused and self.device.type == "cuda"
        self.recv: Optional[SymmetricBuffer] = None
        self.flags: Optional[SymmetricBuffer] = None
        self.epochs: Optional[torch.Tensor] = None
        self.partial: Optional[torch.Tensor] = None
        self.spin = int(os.environ.get("GRIMOIRE_TP_SPIN", "0"))
        self.sp_enabled = os.environ.get("GRIMOIRE_TP_SP", "1") != "0"     # fused sequence-parallel prefill
        self.stats = {"fused_allreduce": 0, "nccl_allreduce": 0}

    def attach(self, model, max_rows: int = 64) -> None:
        """Size the exchange buffers for ``model`` (hidden width) and hook the model's row-parallel ops."""
        H = model.cfg.hidden_size
        model.tp = self
        self.partial = torch.zeros(max_rows, H, dtype=torch.float32, device=self.device)
        if not self.fused:
            return
        tiles = (H + 31) // 32 * 32 // 16
        nv_max = 8 * 128 * 2                               # MT = 8, R = 1, {value, epoch} pairs
        try:
            # + a separate range for the single-row GEMV's partials (16 {value, epoch} pairs per tile), see grm_gemv_w4_allreduce
            self.gemv_off = 2 * self.world * tiles * nv_max
            self.recv = SymmetricBuffer(self.gemv_off + 2 * self.world * tiles * 32, torch.float32, self.group, self.device)
            self.flags = SymmetricBuffer(tiles * self.world, torch.int32, self.group, self.device)
            # exchange regions of the persistent decode kernel (ops/mega.py): [2][world][rows] {value, epoch} pairs
            self.mega_rows = (H + 31) // 32 * 32
            self.mega_recv = SymmetricBuffer(2 * self.world * self.mega_rows * 2, torch.float32, self.group, self.device)
        except Exception as e:  # pragma: no cover - depends on the driver / fabric
            raise RuntimeError(f"symmetric peer memory is unavailable ({e}); set GRIMOIRE_TP_FUSED=0 to run the "
                               f"NCCL-only baseline") from e
        self.epochs = torch.zeros(tiles, dtype=torch.int32, device=self.device)
        dist.barrier(self.group)
        torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------------------------------
    # vocabulary-split lm_head (tp_head_split / tp_head_pick, src/grimoire.cpp:5381-5449)
    # ------------------------------------------------------------------------------------------
    def split_head(self, model, max_rows: int = 64) -> bool:
        """Keep only this rank's block of lm_head rows (blocks of ceil(V / W) rounded up to 32 rows, the last one shorter).
        A decode step then streams 1/W of the head and picks the token with ``head_pick``; whole logits rows are
        gathered on demand.  Returns False (head stays replicated) when the projection type cannot be sliced, the
        model shares its head with a draft head, or GRIMOIRE_TP_HEAD_SPLIT=0."""
        head = getattr(model, "lm_head", None)
        if (self.world < 2 or os.environ.get("GRIMOIRE_TP_HEAD_SPLIT", "1") == "0" or head is None or not hasattr(head, "slice_rows")
                or getattr(head, "swiglu", False) or getattr(model, "pp_world", 1) != 1 or getattr(model, "head_split", None) is not None):
            return False
        V = model.cfg.vocab_size
        vs = (V + self.world - 1) // self.world
        vs = (vs + 31) // 32 * 32
        if vs * (self.world - 1) >= V:
            return False                      # a rank would be left without rows
        v0 = self.rank * vs
        vn = min(V, v0 + vs) - v0
        model.lm_head = head.slice_rows(v0, vn)
        model.head_split = (v0, vn)
        self.head_vs, self.head_rows = vs, max_rows
        if self.fused:
            self.head_recv = SymmetricBuffer(2 * self.world * max_rows * 2 * 2, torch.int32, self.group, self.device)
            self.head_epochs = torch.zeros(max_rows, dtype=torch.int32, device=self.device)
            dist.barrier(self.group)
            torch.cuda.synchronize(self.device)
        self.stats["head_pick"] = 0
        return True

    def head_pick(self, logits: torch.Tensor, v0: int, vn: int, out_ids: torch.Tensor) -> torch.Tensor:
        """Greedy token per row from the ranks' logits slices: every rank offers its best (value, index), the highest
        value wins and ties go to the lowest index.  ``logits`` is the full-width [M][V] buffer whose columns
        [v0, v0 + vn) this rank has filled."""
        M = logits.shape[0]
        local = logits[:, v0:v0 + vn]
        self.stats["head_pick"] += 1
        if self.fused and M <= self.head_rows:
            code = _native.cuda().grm_tp_head_pick(
                _native.ptr(local), ctypes.c_int(logits.stride(0)), ctypes.c_int(M), ctypes.c_int(vn), ctypes.c_int(v0),
                self.head_recv.ptr_array(), _native.ptr(self.head_epochs), _native.ptr(out_ids), None, ctypes.c_int(self.world),
                ctypes.c_int(self.rank), ctypes.c_int(self.head_rows), ctypes.c_uint(self.spin), _native.stream_ptr())
            _native.check(code, "tp_head_pick")
            return out_ids
        # composition of library calls (CPU ranks, NCCL baseline): same rule
        lf = local.float()
        lf = torch.where(torch.isnan(lf), torch.full_like(lf, float("-inf")), lf)
        val, idx = lf.max(dim=1)
        first = (lf == val[:, None]).int().argmax(dim=1)              # lowest index among equal values
        cand = torch.stack([val.double(), torch.where(torch.isinf(val) & (val < 0), torch.full_like(first, 0x7fffffff), first + v0).double()], dim=1)
        allc = [torch.empty_like(cand) for _ in range(self.world)]
        dist.all_gather(allc, cand.contiguous(), group=self.group)
        allc = torch.stack(allc, dim=1)                               # [M][W][2]
        out_ids.copy_(pick_candidates(allc[..., 0], allc[..., 1].long()).to(out_ids.dtype))
        return out_ids

    def gather_head(self, logits: torch.Tensor) -> torch.Tensor:
        """Fill the other ranks' column blocks of the [n][V] logits rows (all-gather of the slices)."""
        n, V = logits.shape
        vs, W = self.head_vs, self.world
        v0 = self.rank * vs
        mine = torch.zeros(n, vs, dtype=logits.dtype, device=logits.device)
        mine[:, : min(V, v0 + vs) - v0] = logits[:, v0:v0 + vs]
        parts = torch.empty(W, n, vs, dtype=logits.dtype, device=logits.device)
        dist.all_gather(list(parts.unbind(0)), mine, group=self.group)
        for r in range(W):
            if r != self.rank:
                a = r * vs
                b = min(V, a + vs)
                logits[:, a:b] = parts[r][:, : b - a]
        return logits

    # ------------------------------------------------------------------------------------------
    def row_parallel_add(self, lin, x: torch.Tensor, h: torch.Tensor) -> None:
        """h (fp32 [M][H], replicated) += all-reduce over ranks of ``x @ W_rank^T``."""
        M = x.shape[0]
        if self.fused and M == 1 and L.GEMV_W4 and isinstance(lin, W4Linear) and lin.tiled is not None and lin.tiled.K <= 20480:
            # one row: the CUDA-core GEMV with the same one-shot all-reduce in its epilogue
            t = lin.tiled
            code = _native.cuda().grm_gemv_w4_allreduce(
                _native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(h), ctypes.c_int(t.N), ctypes.c_int(t.K),
                ctypes.c_int(t.group), self.recv.ptr_array(), ctypes.c_long(self.gemv_off), self.flags.ptr_array(),
                _native.ptr(self.epochs), ctypes.c_int(self.world), ctypes.c_int(self.rank), ctypes.c_uint(self.spin),
                _native.stream_ptr())
            if code != -2:
                _native.check(code, f"gemv_w4_allreduce {lin.name}")
                self.stats["fused_allreduce"] += 1
                return
        if (self.fused and M == 1 and L.GEMV_W4 and isinstance(lin, L.MXLinear) and getattr(lin, "tw", None) is not None and lin.K <= 20480
                and not lin.swiglu):
            # MXFP4, one row: the same one-shot all-reduce in the MXFP4 GEMV's epilogue (region and epochs shared with int4)
            code = _native.cuda().grm_gemv_mx_allreduce(
                _native.ptr(lin.tw), _native.ptr(lin.tsz), _native.ptr(x), _native.ptr(h), ctypes.c_int(lin.N), ctypes.c_int(lin.K),
                self.recv.ptr_array(), ctypes.c_long(self.gemv_off), _native.ptr(self.epochs), ctypes.c_int(self.world),
                ctypes.c_int(self.rank), ctypes.c_uint(self.spin), _native.stream_ptr())
            if code != -2:
                _native.check(code, f"gemv_mx_allreduce {lin.name}")
                self.stats["fused_allreduce"] += 1
                return
        if self.fused and M <= SMALLM_MAX and isinstance(lin, W4Linear) and lin.tiled is not None:
            t = lin.tiled
            code = _native.cuda().grm_smallm_w4_allreduce(
                _native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(h), ctypes.c_int(M), ctypes.c_int(t.N),
                ctypes.c_int(t.K), ctypes.c_int(x.stride(0)), ctypes.c_int(h.stride(0)), ctypes.c_int(t.group),
                self.recv.ptr_array(), self.flags.ptr_array(), _native.ptr(self.epochs), ctypes.c_int(self.world),
                ctypes.c_int(self.rank), ctypes.c_uint(self.spin), _native.stream_ptr())
            _native.check(code, f"smallm_w4_allreduce {lin.name}")
            self.stats["fused_allreduce"] += 1
            return
        part = self.partial[:M] if self.partial is not None and M <= self.partial.shape[0] else torch.empty(
            M, h.shape[1], dtype=torch.float32, device=h.device)
        lin(x, part, "f32")
        dist.all_reduce(part, group=self.group)
        h.add_(part)
        self.stats["nccl_allreduce"] += 1

    # ------------------------------------------------------------------------------------------
    # fused prefill: GEMM -> reduce-scatter, all-gather -> GEMM, norms on the token shard
    # ------------------------------------------------------------------------------------------
    def sp_ready(self, M: int) -> bool:
        """The fused sequence-parallel prefill needs whole 128-row tiles per rank."""
        return self.fused and self.device.type == "cuda" and M % (self.world * 128) == 0 and M > 0

    def sp_setup(self, M: int, H: int) -> None:
        if getattr(self, "_sp_M", 0) >= M and getattr(self, "_sp_H", 0) == H:
            if getattr(self, "_sp_cur_M", M) != M:
                # a different chunk height touches a different set of tiles: restart the arrival
                # counters (all ranks, between launches) so the monotonic expectations stay aligned
                torch.cuda.synchronize(self.device)
                dist.barrier(self.group)
                self.sp_rs_cnt.local.zero_()
                for c in self.sp_ag_cnt:
                    c.local.zero_()
                self._rs_expect, self._ag_expect = 0, [0, 0]
                torch.cuda.synchronize(self.device)
                dist.barrier(self.group)
                self._sp_cur_M = M
            return
        self._sp_cur_M = M
        W = self.world
        R = M // W
        self.sp_x = [SymmetricBuffer(M * H, torch.bfloat16, self.group, self.device) for _ in range(2)]          # gathered activations
        self.sp_recv = [SymmetricBuffer(W * R * H, torch.bfloat16, self.group, self.device) for _ in range(2)]    # partial slots
        self.sp_rs_cnt = SymmetricBuffer((R // 128) * W + 8, torch.int32, self.group, self.device)
        self.sp_ag_cnt = [SymmetricBuffer(M // 128 + 8, torch.int32, self.group, self.device) for _ in range(2)]
        self.sp_hs = torch.zeros(R, H, dtype=torch.float32, device=self.device)
        self._sp_M, self._sp_H = M, H
        self._rs_expect = 0
        self._ag_expect = [0, 0]
        self._sp_flip = 0
        self._rs_flip = 0
        dist.barrier(self.group)
        torch.cuda.synchronize(self.device)

    def sp_reduce_norm_allgather(self, hs: torch.Tensor, norm_w, eps: float, offset: float, reduce: bool, M: int):
        """Owner side: hs (+= sum of the W partials of the last row-parallel GEMM); when ``norm_w``
        is given, push rms(hs)*w into every rank's activation copy.  Returns (x_full view, ag counter
        tensor, expected count) for the consuming GEMM."""
        W, R, H = self.world, hs.shape[0], hs.shape[1]
        recv = cnt = None
        if reduce:
            recv = self.sp_recv[self._rs_flip ^ 1].local       # the buffer the last rs_push wrote
            cnt = self.sp_rs_cnt.local
        xi = self._sp_flip
        x_ptrs = ag_ptrs = None
        if norm_w is not None:
            x_ptrs, ag_ptrs = self.sp_x[xi].ptr_array(), self.sp_ag_cnt[xi].ptr_array()
            self._ag_expect[xi] += 128
        code = _native.cuda().grm_rs_reduce_norm_ag(
            _native.ptr(hs), ctypes.c_int(hs.stride(0)), _native.ptr(recv), _native.ptr(cnt), ctypes.c_uint(self._rs_expect & 0xFFFFFFFF),
            _native.ptr(norm_w), ctypes.c_float(eps), ctypes.c_float(offset), x_ptrs, ag_ptrs, ctypes.c_int(R), ctypes.c_int(H),
            ctypes.c_int(W), ctypes.c_int(self.rank), ctypes.c_uint(self.spin), _native.stream_ptr())
        _native.check(code, "rs_reduce_norm_ag")
        if norm_w is None:
            return None, None, 0
        self._sp_flip ^= 1
        return self.sp_x[xi].local[: M * H].view(M, H), self.sp_ag_cnt[xi].local, self._ag_expect[xi]

    def sp_gemm_allgathered(self, lin, x_full, ag_cnt, ag_expect, out, epi: str):
        """Column-parallel projection whose A rows arrive by all-gather pushes (waits per m tile)."""
        from ..ops.linear import gemm_bf16_tp, w4_dequant_into

        w = w4_dequant_into(lin)
        gemm_bf16_tp(x_full, w, out, epi, ag_cnt=ag_cnt, ag_expect=ag_expect)

    def sp_gemm_reduce_scatter(self, lin, x, M: int, H: int):
        """Row-parallel projection whose epilogue pushes partial tiles to the row owners."""
        from ..ops.linear import gemm_bf16_tp, w4_dequant_into

        w = w4_dequant_into(lin)
        buf = self.sp_recv[self._rs_flip]
        nt = gemm_bf16_tp(x, w, None, "rs_push", peer_out=buf.ptr_array(), peer_cnt=self.sp_rs_cnt.ptr_array(), world=self.world,
                          my_rank=self.rank, ldo=H)
        self._rs_expect += 4 * nt
        self._rs_flip ^= 1

    def check(self) -> None:
        """Raise CommTimeout if a fused kernel recorded a peer-wait timeout."""
        if self.device.type != "cuda":
            return
        from ..ops.core import status_read

        code, detail, n = status_read()
        if code:
            raise CommTimeout(f"device status code {code} detail {detail:#x} ({n} events) on rank {self.rank}")
