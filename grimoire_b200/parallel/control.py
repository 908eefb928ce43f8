"""Rank lockstep: the front-end rank broadcasts every engine call so the worker ranks issue the
same kernels (and therefore the same collectives) in the same order.

Reference: PPRequest kinds 0 generate / 1 shutdown / 2 admit slot / 3 batch step / 4 cache sequence
/ 5 speculative batch step (grimoire.cpp:2834-2845), pp_send_request / pp_recv_request with length
validation (:4658-4734), grimoire_pp_worker_loop (:25040-25124), the per-token cancellation word
(include/b70/generation_control.hpp).  Here the descriptor is a small int64 tensor broadcast over a
gloo (CPU) group, so control traffic never touches the GPU stream; a cancelled job simply stops
appearing in later steps, and SHUTDOWN ends the worker loop.  A worker whose engine call raises
leaves the loop (the byte stream cannot be resynchronised), and a broadcast that times out ends it
with ``WorkerLost``.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

OPEN, RELEASE, PREFILL, STEP, ROLLBACK, COMMIT, SHUTDOWN, PREFIX_REUSE = range(8)
MAX_PAYLOAD = 1 << 22          # ints; anything larger is a corrupted header
HEADER = 4                     # kind, a, b, payload length


class WorkerLost(RuntimeError):
    pass


class ControlChannel:
    def __init__(self, group, src_rank: int = 0):
        self.group = group
        self.src = src_rank
        self.rank = dist.get_rank(group)
        self.is_root = self.rank == 0

    def send(self, kind: int, a: int = 0, b: int = 0, payload: Sequence[int] = ()) -> None:
        n = len(payload)
        if n > MAX_PAYLOAD:
            raise ValueError("control payload too large")
        head = torch.tensor([kind, a, b, n], dtype=torch.int64)
        try:
            dist.broadcast(head, src=self.src, group=self.group)
            if n:
                dist.broadcast(torch.tensor(list(payload), dtype=torch.int64), src=self.src, group=self.group)
        except RuntimeError as e:
            # a worker that left its loop (exception, exit) or stopped answering within the group timeout
            raise WorkerLost(f"control channel broken while sending kind={kind}: {e}") from None

    def recv(self):
        head = torch.zeros(HEADER, dtype=torch.int64)
        try:
            dist.broadcast(head, src=self.src, group=self.group)
        except RuntimeError as e:
            raise WorkerLost(f"control channel closed: {e}") from None
        kind, a, b, n = (int(v) for v in head)
        if not (0 <= kind <= PREFIX_REUSE) or n < 0 or n > MAX_PAYLOAD:
            raise WorkerLost(f"bad control header kind={kind} len={n}")      # validate before allocating
        payload = []
        if n:
            t = torch.zeros(n, dtype=torch.int64)
            dist.broadcast(t, src=self.src, group=self.group)
            payload = t.tolist()
        return kind, a, b, payload


class ControlledEngine:
    """Front-end side: same interface as ``Engine``; every call is announced before it runs."""

    def __init__(self, engine, channel: ControlChannel):
        self.engine, self.ch = engine, channel
        self.limits, self.device, self.cfg, self.kv, self.model = engine.limits, engine.device, engine.cfg, engine.kv, engine.model

    @property
    def prefix_cache(self):
        return self.engine.prefix_cache

    def open(self, slot: Optional[int] = None):
        seq = self.engine.open(slot)
        self.ch.send(OPEN, seq.slot)
        return seq

    def release(self, seq, cache: bool = False, head_logits=None) -> None:
        self.ch.send(RELEASE, seq.slot, 1 if cache else 0)
        self.engine.release(seq, cache, head_logits)

    def prefix_reuse(self, seq, prompt) -> int:
        self.ch.send(PREFIX_REUSE, seq.slot, 0, list(prompt))
        return self.engine.prefix_reuse(seq, prompt)

    def prefill(self, seq, tokens, want_logits: bool = True):
        toks = tokens.tolist() if torch.is_tensor(tokens) else list(tokens)
        self.ch.send(PREFILL, seq.slot, 0, toks)
        return self.engine.prefill(seq, toks, want_logits)

    def decode_rows(self, tokens, seqs, positions, use_graph: bool = True, return_logits: bool = False):
        M = len(tokens)
        self.ch.send(STEP, M, 1 if use_graph else 0, list(tokens) + [s.slot for s in seqs] + list(positions))
        return self.engine.decode_rows(tokens, seqs, positions, use_graph, return_logits)

    def commit_rows(self, seqs, tokens, positions) -> None:
        self.ch.send(COMMIT, len(tokens), 0, [s.slot for s in seqs] + list(tokens) + list(positions))
        self.engine.commit_rows(seqs, tokens, positions)

    def rollback(self, seq, length: int) -> None:
        self.ch.send(ROLLBACK, seq.slot, length)
        self.engine.rollback(seq, length)

    def enable_speculation(self) -> None:
        self.engine.enable_speculation()         # every rank switched at start-up (parallel/launch.py); local no-op then

    def sample_rows(self, logits, opts, positions):
        return self.engine.sample_rows(logits, opts, positions)      # every rank holds the same logits: the front end draws

    def can_prefill_batch(self) -> bool:
        return False                                                 # the control protocol announces one prompt per call

    def shutdown(self) -> None:
        self.ch.send(SHUTDOWN)


def worker_loop(engine, channel: ControlChannel) -> int:
    """Worker ranks: mirror the front end's engine calls until SHUTDOWN.  Returns calls served."""
    served = 0
    while True:
        kind, a, b, p = channel.recv()
        if kind == SHUTDOWN:
            return served
        served += 1
        if kind == OPEN:
            engine.open(a)
        elif kind == RELEASE:
            seq = engine.kv.slots.get(a)
            if seq is not None:
                engine.release(seq, bool(b))
        elif kind == PREFIX_REUSE:
            engine.prefix_reuse(engine.kv.slots[a], p)
        elif kind == PREFILL:
            engine.prefill(engine.kv.slots[a], p)
        elif kind == STEP:
            M = a
            toks, slots, pos = p[:M], p[M: 2 * M], p[2 * M: 3 * M]
            engine.decode_rows(toks, [engine.kv.slots[s] for s in slots], pos, use_graph=bool(b))
        elif kind == COMMIT:
            M = a
            slots, toks, pos = p[:M], p[M: 2 * M], p[2 * M: 3 * M]
            engine.commit_rows([engine.kv.slots[s] for s in slots], toks, pos)
        elif kind == ROLLBACK:
            engine.rollback(engine.kv.slots[a], b)
