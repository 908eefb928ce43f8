"""Pipeline parallelism: stage r owns a contiguous layer range, the hidden state ``[rows][H]`` hops
to the next stage once per forward, the token chosen by the last stage travels back to every stage.

Reference: multi-process PP (grimoire.cpp:2485-2499 ranks, pp_send_hidden/pp_recv_hidden
:4766-4887, pp_sync_token(s) :4621/:4889, chunked prefill so stages overlap, generation.hpp:193-257).
There the hop is fp32 over a Unix socket chain; here it is ``ncclSend/ncclRecv`` (torch.distributed
p2p) issued on a dedicated communication stream with event hand-off, double-buffered so a stage can
run one chunk ahead of its successor -- by design NOT fused into a kernel: one hop per stage per
step, overlapped with compute by chunking.  The payload is fp32 by default (token-identical to a
single process); ``wire_dtype=torch.bfloat16`` halves the bytes.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


class PipelineParallel:
    def __init__(self, group, device, wire_dtype: torch.dtype = torch.float32):
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.ranks = dist.get_process_group_ranks(group)
        self.wire_dtype = wire_dtype
        self.cuda = self.device.type == "cuda"
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.cuda else None
        self._stage = [None, None]          # double-buffered staging for sends
        self._flip = 0
        self._pending: list = []
        self.stats = {"sends": 0, "recvs": 0, "bytes": 0}

    @property
    def is_first(self) -> bool:
        return self.rank == 0

    @property
    def is_last(self) -> bool:
        return self.rank == self.world - 1

    def attach(self, model) -> None:
        model.pp = self

    # ---- stage boundary ----
    def send_hidden(self, h: torch.Tensor) -> None:
        dst = self.ranks[self.rank + 1]
        self.stats["sends"] += 1
        self.stats["bytes"] += h.numel() * torch.finfo(self.wire_dtype).bits // 8
        if not self.cuda:
            dist.send(h.to(self.wire_dtype).contiguous(), dst=dst, group=self.group)
            return
        # copy into a staging buffer on the compute stream, then hand the send to the comm stream so
        # the next chunk's kernels do not wait for the successor to post its receive
        i = self._flip
        self._flip ^= 1
        buf = self._stage[i]
        if buf is None or buf.shape != h.shape or buf.dtype != self.wire_dtype:
            buf = torch.empty_like(h, dtype=self.wire_dtype)
            self._stage[i] = buf
        cur = torch.cuda.current_stream(self.device)
        self.comm_stream.wait_stream(cur)          # earlier sends from this buffer finished before reuse
        cur.wait_stream(self.comm_stream)
        buf.copy_(h)
        ready = torch.cuda.Event()
        ready.record(cur)
        with torch.cuda.stream(self.comm_stream):
            self.comm_stream.wait_event(ready)
            dist.send(buf, dst=dst, group=self.group)

    def recv_hidden(self, h: torch.Tensor) -> None:
        src = self.ranks[self.rank - 1]
        self.stats["recvs"] += 1
        if self.wire_dtype == h.dtype:
            dist.recv(h, src=src, group=self.group)
            return
        tmp = torch.empty_like(h, dtype=self.wire_dtype)
        dist.recv(tmp, src=src, group=self.group)
        h.copy_(tmp)

    def broadcast_from_last(self, t: torch.Tensor) -> torch.Tensor:
        """The last stage's tensor (chosen tokens, last-token logits) to every stage."""
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.comm_stream)
        dist.broadcast(t, src=self.ranks[self.world - 1], group=self.group)
        return t


def stage_layers(n_layers: int, world: int, rank: int) -> tuple[int, int]:
    per, extra = divmod(n_layers, world)
    b = rank * per + min(rank, extra)
    return b, b + per + (1 if rank < extra else 0)
