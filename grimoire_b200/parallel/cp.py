"""Context parallelism for prompt reading: the rows of a prefill chunk are split over the ranks.

Every rank holds the whole model (27B int4 is 14 GB of 180) and the whole KV cache.  For a chunk of M rows rank r runs the
projections, the MLP and the attention of rows [r M/R, (r + 1) M/R) only -- 1/R of the FLOPs -- and the one thing the
ranks exchange per layer is the chunk's fresh k | v rows (raw, before the head norm and RoPE): each rank pushes the rows it
just projected into every peer's copy of the chunk's q|k|v matrix, then all ranks apply norm + RoPE and append the WHOLE
chunk's K / V to their own cache, so the cache stays replicated and the attention of the local query rows reads past and
present keys from local memory.  That is 2 x kv_width x M bf16 per layer (16 MB for a 4096-row chunk of the 27B model)
against ~1 ms of per-rank compute: on NVLink the exchange is noise, which is why this scheme rather than a ring of K/V
blocks (ring attention trades bandwidth for memory; a 131,072-token int8 cache is 17 GB here and fits every rank).
Decode after such a prefill runs replicated (every rank steps the same token), or the cache can be handed to a
tensor-parallel engine.

The reference is single-rank for long prompts (include/b70/generation.hpp:202-213) and has no counterpart.

Exchange.  On CUDA ranks the rows travel by peer stores from a small copy kernel of ours into symmetric memory
(``SymmetricBuffer``), with one arrival counter per rank and layer parity; waits are bounded and report through the status
block.  The composition of library calls (``fused=False``, and CPU ranks) is an all-gather.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native


class ContextParallel:
    def __init__(self, group, device, fused: Optional[bool] = None):
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if fused is None:
            fused = os.environ.get("GRIMOIRE_CP_FUSED", "1") != "0"
        self.fused = fused and self.device.type == "cuda"
        self.kvbuf = None
        self.cnt = None
        self.rows = 0
        self.width = 0
        self.expect = 0
        self.spin = int(os.environ.get("GRIMOIRE_TP_SPIN", "0"))
        self.stats = {"chunks": 0, "exchanges": 0}
        self.balanced = os.environ.get("GRIMOIRE_CP_BALANCED", "0") not in ("", "0")
        self._layouts: dict = {}

    def attach(self, model, max_rows: int) -> None:
        """Hook ``model`` (a whole, unsharded DenseModel) so that prefill chunks whose rows divide over the ranks take the
        context-parallel path."""
        if getattr(model, "tp_world", 1) != 1 or getattr(model, "pp_world", 1) != 1:
            raise ValueError("context parallelism runs over whole model replicas (no tensor / pipeline shards)")
        model.cp = self
        geom = model.geom
        self.width = 2 * geom.Hkv * geom.D
        self.rows = max_rows
        if self.fused:
            from .tp import SymmetricBuffer

            # two parities of the chunk's k|v rows, so that a rank one layer ahead never overwrites rows a peer still reads
            self.kvbuf = SymmetricBuffer(2 * max_rows * self.width, torch.bfloat16, self.group, self.device)
            self.cnt = SymmetricBuffer(2 * 8, torch.int32, self.group, self.device)
            dist.barrier(self.group)
            torch.cuda.synchronize(self.device)

    def ready(self, M: int) -> bool:
        return M % self.world == 0 and M // self.world >= 1 and M <= self.rows

    def local_rows(self, M: int) -> tuple[int, int]:
        """This rank's rows of the chunk in EXCHANGE order (see ``layout``): always one contiguous range."""
        per = M // self.world
        return self.rank * per, (self.rank + 1) * per

    def layout(self, M: int):
        """How the chunk's rows map onto the ranks: contiguous shares by default; with GRIMOIRE_CP_BALANCED=1 the balanced
        split below.  (Measured on 2 GPUs the two come out even, 28.4 against 28.8 ms for a 16-layer 4,096-row chunk: a
        rank's attention time is set by its longest query block's walk over the keys, not by its total work, and the late
        piece of the balanced split walks as many keys as the last contiguous share does.)
        Causal attention makes late rows dearer than early ones, so with
        2 R pieces of M / (2 R) rows rank r takes piece r and piece 2 R - 1 - r: every rank then sees the same number of
        (query, key) pairs.  The ranks work on the chunk in exchange order -- rank 0's two pieces, rank 1's two pieces, ...
        -- in which each rank's rows are contiguous; ``perm[j]`` is the chunk row that sits at exchange index j.
        Returns (segments of this rank as (first chunk row, rows) in local order, perm or None for the identity)."""
        hit = self._layouts.get(M)
        if hit is not None:
            return hit
        W, r = self.world, self.rank
        if not self.balanced or M % (2 * W) or M // (2 * W) < 8:
            per = M // W
            out = ([(r * per, per)], None)
        else:
            p = M // (2 * W)
            pieces = []
            for q in range(W):
                pieces += [q, 2 * W - 1 - q]
            perm = torch.cat([torch.arange(x * p, (x + 1) * p) for x in pieces]).to(self.device)
            out = ([(r * p, p), ((2 * W - 1 - r) * p, p)], perm)
        self._layouts[M] = out
        return out

    def owner_index(self, rows: torch.Tensor, M: int):
        """For chunk rows ``rows`` (long tensor): (owner rank, index within the owner's local rows)."""
        segs, perm = self.layout(M)
        if perm is None:
            per = M // self.world
            return rows // per, rows % per
        p = M // (2 * self.world)
        piece = rows // p
        late = piece >= self.world
        owner = torch.where(late, 2 * self.world - 1 - piece, piece)
        return owner, rows % p + late.long() * p

    def exchange_kv(self, qkv: torch.Tensor, M: int, qsz: int, parity: int) -> None:
        """``qkv`` [M][qsz + width], rows in exchange order: the local rows' k | v columns are valid; on return every row's
        are."""
        a, b = self.local_rows(M)
        self.stats["exchanges"] += 1
        if self.fused:
            self.expect += int(_native.cuda().grm_cp_push_grid(ctypes.c_int(b - a)))     # arrivals per source so far
            code = _native.cuda().grm_cp_push_rows(
                _native.ptr(qkv), ctypes.c_int(qkv.stride(0)), ctypes.c_int(qsz), ctypes.c_int(self.width), ctypes.c_int(a), ctypes.c_int(b),
                ctypes.c_int(M), self.kvbuf.ptr_array(), self.cnt.ptr_array(), ctypes.c_int(parity), ctypes.c_uint(self.expect & 0xFFFFFFFF),
                ctypes.c_int(self.rows), ctypes.c_int(self.world), ctypes.c_int(self.rank), ctypes.c_uint(self.spin), _native.stream_ptr())
            _native.check(code, "cp_push_rows")
            return
        mine = qkv[a:b, qsz:].contiguous()
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine, group=self.group)
        per = b - a
        for r, t in enumerate(parts):
            if r != self.rank:
                qkv[r * per:(r + 1) * per, qsz:] = t

    def broadcast_rows(self, t: torch.Tensor, owner: int) -> torch.Tensor:
        dist.broadcast(t, src=dist.get_global_rank(self.group, owner), group=self.group)
        return t
