"""Expert parallelism for the MoE layers: each rank owns E/W experts and a contiguous shard of the
step's rows; tokens travel to the owners of their chosen experts and back.

Two implementations of the same contract ``moe(layer, x, h, wts, ids, M)`` (``h += MoE(x)`` for all
rows, identical on every rank afterwards):

* **fused** (GPU, default): the dispatch / plan / grouped-GEMM-with-push / combine / apply chain of
  ``ep_fused.cu`` + ``moe.cu`` over symmetric peer memory -- no NCCL call, no host round trip,
  replayable from a CUDA graph.  Row shards: rank s owns rows [s*Mq, (s+1)*Mq), Mq = ceil(M/W).
* **allreduce** (CPU ranks under gloo, and the measured NCCL baseline on GPUs): every rank evaluates
  its local experts for all rows and the partial sums are all-reduced.  This is the composition the
  reference uses between its two cards (expert partials exchanged with the tensor-parallel
  all-reduce, grimoire.cpp:15364-15453 with tp_small_allreduce :6499).

Expert e lives on rank e // (E/W) (``models/expert_placement.py`` can permute experts before the
split so hot experts spread evenly).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native
from ..ops import hybrid as Hb
from .tp import CommTimeout, SymmetricBuffer


def _c(v):
    return ctypes.c_int(int(v))


class _LocalBuffer:
    """Stand-in for ``SymmetricBuffer`` when the "group" is this GPU alone."""

    def __init__(self, numel: int, dtype: torch.dtype, device):
        self.local = torch.zeros(numel, dtype=dtype, device=device)
        self.ptrs, self.world = [self.local.data_ptr()], 1

    def ptr_array(self):
        return (ctypes.c_void_p * 1)(*self.ptrs)


class ExpertParallel:
    def __init__(self, group, device, num_experts: int, top_k: int, hidden: int, inter: int, max_rows: int,
                 fused: Optional[bool] = None):
        """``group`` None: a single-GPU instance -- the same device-side dispatch / plan / grouped GEMM /
        combine chain with local buffers, used for prompt chunks so that grouping tokens by expert needs no
        host round trip."""
        self.group, self.device = group, torch.device(device)
        self.rank, self.world = (dist.get_rank(group), dist.get_world_size(group)) if group is not None else (0, 1)
        if num_experts % self.world:
            raise ValueError(f"{num_experts} experts do not split over {self.world} ranks")
        self.E, self.E_loc, self.k, self.H, self.I = num_experts, num_experts // self.world, top_k, hidden, inter
        if fused is None:
            fused = os.environ.get("GRIMOIRE_EP_FUSED", "1") != "0"
        self.fused = fused and self.device.type == "cuda"
        self.max_rows = max_rows
        self.spin = int(os.environ.get("GRIMOIRE_EP_SPIN", "0"))
        self.stats = {"fused_layers": 0, "allreduce_layers": 0}
        if self.fused:
            self._setup_fused()

    # ------------------------------------------------------------------------------------------
    def expert_range(self) -> tuple[int, int]:
        return self.rank * self.E_loc, (self.rank + 1) * self.E_loc

    def shard(self, M: int) -> tuple[int, int, int]:
        """(Mq, first row, rows) of this rank's shard of an M-row step."""
        Mq = (M + self.world - 1) // self.world
        lo = min(M, self.rank * Mq)
        return Mq, lo, min(M, lo + Mq) - lo

    def _setup_fused(self) -> None:
        W, k, H, dev, g = self.world, self.k, self.H, self.device, self.group
        Mq_max = (self.max_rows + W - 1) // W
        self.cap = Mq_max * k                              # rows one source can send to one owner
        i32, f32, bf = torch.int32, torch.float32, torch.bfloat16
        mkbuf = (lambda n, dt: SymmetricBuffer(n, dt, g, dev)) if g is not None else (lambda n, dt: _LocalBuffer(n, dt, dev))
        self.xrecv = mkbuf(W * self.cap * H, bf)
        self.rowdst = mkbuf(W * self.cap, i32)
        self.groups = mkbuf(W * self.E_loc * 2, i32)
        self.flags = mkbuf(8, i32)
        self.y = mkbuf(Mq_max * (k + 1) * H, f32)
        self.done = mkbuf(8, i32)
        self.gather = mkbuf(2 * self.max_rows * H if W > 1 else 8, f32)
        self.hflags = mkbuf(8, i32)
        z = lambda *s, dt=i32: torch.zeros(*s, dtype=dt, device=dev)
        self.state = z(16)
        self.counts, self.ebase, self.cursors = z(self.E), z(self.E), z(self.E)
        self.max_tiles = (W * self.cap + 31) // 32 + W * self.E_loc
        self.tile_expert, self.tile_row0, self.tile_rows, self.tile_src = (z(self.max_tiles) for _ in range(4))
        self.n_tiles = z(1)
        self.act = z(W * self.cap, self.I, dt=bf)
        # decode (<= ll_rows rows): replicated routing, local experts only, all-reduce inside the combine kernel
        self.ll_rows = 8
        self.ll_cap = self.ll_rows * H
        self.ll_recv = mkbuf(2 * W * self.ll_cap * 2, f32)                 # {value, epoch} pairs [2 parity][W][cap]
        self.ll_epochs = z((self.ll_cap + 255) // 256)
        self.ll_te, self.ll_nr = z(self.ll_rows * k), z(self.ll_rows * k)
        self.ll_pos = z(self.ll_rows * (k + 1))
        if g is not None:
            dist.barrier(g)
        torch.cuda.synchronize(dev)

    # ------------------------------------------------------------------------------------------
    def moe_fused(self, moe, x: torch.Tensor, h: torch.Tensor, lg: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor,
                  act_s: torch.Tensor, M: int, renorm: bool) -> None:
        """x bf16 [M][H] and h fp32 [M][H] are replicated; lg fp32 [M][E+1] router logits (last column the
        shared-expert gate).  ``moe`` holds this rank's expert slice."""
        lib, st = _native.cuda(), _native.stream_ptr()
        W, k, H, E = self.world, self.k, self.H, self.E
        Mq, lo, n = self.shard(M)
        xs, hs, lgs, idl, wl = x[lo: lo + n], h[lo: lo + n], lg[lo: lo + n], ids[:n], wts[:n]
        self.counts.zero_()
        if n:
            Hb.moe_route(lgs, E, k, renorm, idl, wl, self.counts, shared_gate=True)
        _native.check(lib.grm_ep_prefix(_native.ptr(self.counts), _native.ptr(self.ebase), _native.ptr(self.cursors),
                                        self.groups.ptr_array(), _c(E), _c(self.E_loc), _c(W), _c(self.rank), _c(self.cap), st), "ep_prefix")
        _native.check(lib.grm_ep_dispatch(_native.ptr(xs) if n else None, _c(x.stride(0)), _native.ptr(idl), _c(ids.stride(0)),
                                          _native.ptr(self.ebase), _native.ptr(self.cursors), self.xrecv.ptr_array(),
                                          self.rowdst.ptr_array(), self.flags.ptr_array(), _native.ptr(self.state), _c(n), _c(k), _c(H),
                                          _c(self.E_loc), _c(W), _c(self.rank), _c(self.cap), st), "ep_dispatch")
        _native.check(lib.grm_ep_plan(_native.ptr(self.flags.local), _native.ptr(self.groups.local), _native.ptr(self.tile_expert),
                                      _native.ptr(self.tile_row0), _native.ptr(self.tile_rows), _native.ptr(self.tile_src),
                                      _native.ptr(self.n_tiles), _native.ptr(self.state), _c(self.E_loc), _c(W), _c(self.max_tiles),
                                      ctypes.c_uint(self.spin), st), "ep_plan")
        bound = min(self.max_tiles, (W * Mq * k + 31) // 32 + min(W * self.E_loc, W * Mq * k))
        N1, I = moe.gate_up.shape[1], self.I
        _native.check(lib.grm_moe_grouped_gemm_ep(
            _native.ptr(self.xrecv.local), _c(H), _native.ptr(self.tile_expert), _native.ptr(self.tile_row0), _native.ptr(self.tile_rows),
            _native.ptr(self.tile_src), _native.ptr(self.n_tiles), _c(bound), _native.ptr(moe.gate_up), _native.ptr(moe.gate_up_scale),
            _native.ptr(self.act), _c(I), _c(N1), _c(H), _c(0), None, None, None, _c(W), _c(1 if M <= 8 else 0), st), "ep gate_up")
        _native.check(lib.grm_moe_grouped_gemm_ep(
            _native.ptr(self.act), _c(I), _native.ptr(self.tile_expert), _native.ptr(self.tile_row0), _native.ptr(self.tile_rows),
            _native.ptr(self.tile_src), _native.ptr(self.n_tiles), _c(bound), _native.ptr(moe.down), _native.ptr(moe.down_scale),
            None, _c(H), _c(H), _c(I), _c(4), _native.ptr(self.rowdst.local), self.y.ptr_array(), self.done.ptr_array(), _c(W),
            _c(1 if M <= 8 else 0), st),
            "ep down+combine push")
        yl = self.y.local.view(-1, H)
        has_shared = 0
        if moe.shared_gu is not None:
            has_shared = 1
            if n:
                moe.shared_gu(xs, act_s[:n], "swiglu")
                moe.shared_down(act_s[:n], yl[n * k: n * (k + 1)], "f32")
        nblk = (H + 127) // 128
        _native.check(lib.grm_ep_combine(_native.ptr(hs) if n else None, _c(h.stride(0)), _native.ptr(yl), _c(H), _native.ptr(wl),
                                         _c(wts.stride(0)), _native.ptr(self.done.local), self.gather.ptr_array(), self.hflags.ptr_array(),
                                         _native.ptr(self.state), _c(n), _c(k), _c(H), _c(has_shared), _c(nblk), _c(W), _c(self.rank),
                                         _c(lo), _c(M), ctypes.c_uint(self.spin), st), "ep_combine")
        if W > 1:
            _native.check(lib.grm_ep_apply(_native.ptr(h), _c(h.stride(0)), _native.ptr(self.gather.local), _native.ptr(self.hflags.local),
                                           _native.ptr(self.state), _c(M), _c(H), _c(Mq), _c(self.rank), ctypes.c_uint(self.spin), st),
                          "ep_apply")
        self.stats["fused_layers"] += 1

    # ------------------------------------------------------------------------------------------
    def decode_tiles(self, ids: torch.Tensor, M: int):
        """Replicated choices ``ids`` [M][k] -> (tile_expert, tile_rows, pos [M][k+1]) over this rank's experts: a choice
        owned elsewhere becomes an empty tile and a skipped combine slot; rank 0 owns the (replicated) shared expert."""
        e0, e1 = self.expert_range()
        te, nr, pos = self.ll_te[: M * self.k], self.ll_nr[: M * self.k], self.ll_pos[: M * (self.k + 1)].view(M, self.k + 1)
        code = _native.cuda().grm_ep_decode_prep(_native.ptr(ids), _c(ids.stride(0)), _c(M), _c(self.k), _c(e0), _c(e1),
                                                 _c(1 if self.rank == 0 else 0), _native.ptr(te), _native.ptr(nr), _native.ptr(pos),
                                                 _native.stream_ptr())
        _native.check(code, "ep_decode_prep")
        return te, nr, pos

    def combine_allreduce(self, h: torch.Tensor, y: torch.Tensor, pos: torch.Tensor, wts: torch.Tensor, M: int) -> None:
        """h += sum over ranks of the weighted sum of this rank's expert outputs (one kernel, see ep_fused.cu)."""
        code = _native.cuda().grm_ep_combine_allreduce(
            _native.ptr(h), _c(h.stride(0)), _native.ptr(y), _c(y.stride(0)), _native.ptr(pos), _native.ptr(wts), _c(M), _c(self.k + 1),
            _c(self.H), self.ll_recv.ptr_array(), ctypes.c_long(self.ll_cap), _native.ptr(self.ll_epochs), _c(self.world), _c(self.rank),
            ctypes.c_uint(self.spin), _native.stream_ptr())
        _native.check(code, "ep_combine_allreduce")
        self.stats["fused_layers"] += 1

    def moe_allreduce(self, moe, x: torch.Tensor, h: torch.Tensor, lg: torch.Tensor, M: int, renorm: bool, ids_out=None) -> None:
        """Local experts for all rows, partial sums all-reduced (CPU ranks, and the NCCL baseline).  ``ids_out`` int32 [M][k]
        receives the routing decision (every rank makes the same one)."""
        E, k, H = self.E, self.k, self.H
        dev = x.device
        ids = ids_out if ids_out is not None else torch.empty(M, k, dtype=torch.int32, device=dev)
        wts = torch.empty(M, k, dtype=torch.float32, device=dev)
        Hb.moe_route(lg, E, k, renorm, ids, wts)
        e0, e1 = self.expert_range()
        flat = ids.reshape(-1).long()
        mine = ((flat >= e0) & (flat < e1)).nonzero().reshape(-1)
        part = torch.zeros(M, H, dtype=torch.float32, device=dev)
        if mine.numel():
            loc = flat[mine] - e0
            order = torch.sort(loc, stable=True).indices
            pairs = mine[order]                                   # pair index = row * k + choice, grouped by local expert
            le = loc[order]
            counts = torch.bincount(le, minlength=self.E_loc).cpu()
            tiles_per = (counts + 15) // 16
            starts = torch.cumsum(counts, 0) - counts
            te = torch.repeat_interleave(torch.arange(self.E_loc), tiles_per)
            within = torch.arange(int(tiles_per.sum())) - torch.repeat_interleave(torch.cumsum(tiles_per, 0) - tiles_per, tiles_per)
            r0 = starts[te] + within * 16
            nr = torch.minimum(torch.full_like(r0, 16), counts[te] - within * 16)
            te, r0, nr = (t.to(torch.int32).to(dev) for t in (te, r0, nr))
            src = (pairs // k).to(torch.int32)
            act = torch.empty(pairs.numel(), self.I, dtype=torch.bfloat16, device=dev)
            y = torch.empty(pairs.numel(), H, dtype=torch.float32, device=dev)
            Hb.grouped_gemm_fp8(x, src, te, r0, nr, moe.gate_up, moe.gate_up_scale, act, "swiglu")
            Hb.grouped_gemm_fp8(act, None, te, r0, nr, moe.down, moe.down_scale, y, "f32")
            w = wts.reshape(-1)[pairs]
            # per-row sums in (row, choice) order so the local partial is reproducible
            back = torch.argsort(pairs)
            part.index_add_(0, (pairs[back] // k), y[back] * w[back, None])
        if moe.shared_gu is not None:
            # the shared expert is replicated: the owner of a row's shard adds it once
            Mq, lo, n = self.shard(M)
            if n:
                a = torch.empty(n, moe.shared_gu.N // 2, dtype=torch.bfloat16, device=dev)
                ys = torch.empty(n, H, dtype=torch.float32, device=dev)
                moe.shared_gu(x[lo: lo + n], a, "swiglu")
                moe.shared_down(a, ys, "f32")
                part[lo: lo + n] += torch.sigmoid(lg[lo: lo + n, E])[:, None] * ys
        if self.world > 1:
            dist.all_reduce(part, group=self.group)
        h.add_(part)
        self.stats["allreduce_layers"] += 1

    def check(self) -> None:
        if self.device.type != "cuda":
            return
        from ..ops.core import status_read

        code, detail, n = status_read()
        if code:
            raise CommTimeout(f"device status code {code} detail {detail:#x} ({n} events) on rank {self.rank}")
