"""Continuous-batching scheduler: one thread owns the engine, request threads submit jobs and
receive tokens.

Parity with the reference's GrimoireScheduler (grimoire.cpp:24271-25006): ``generate`` blocks the
calling (HTTP) thread and runs ``on_token`` on THAT thread; the scheduler thread admits prompts
(burst hold, batched / interleaved admission), steps every live conversation in one batched pass
(plain, or speculative with copy drafts and per-row longest-prefix acceptance), flushes the first
tokens of a round together, retires finished conversations into the prefix cache and cancels a job
at the next token when its callback returns False (client disconnect).  The policy lives in the
C++ core (csrc/host/sched_core.cpp); this file performs the engine calls the plan asks for.
"""
from __future__ import annotations

import ctypes
import itertools
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

import torch

from .. import _native
from ..engine.generation import CopyDrafter, FinishReason, SpecStats, first_token_of
from ..engine.kv import OutOfPages
from ..engine.sampling import SamplingOptions, sample_ref

PLAN_ADMIT, PLAN_STEP, PLAN_WAIT = 1, 2, 4


class _Plan(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("wait_ms", ctypes.c_double), ("n_admit", ctypes.c_int),
                ("admit_job", ctypes.c_int64 * 64), ("admit_slot", ctypes.c_int * 64), ("admit_from", ctypes.c_int * 64),
                ("admit_to", ctypes.c_int * 64), ("n_live", ctypes.c_int), ("live_job", ctypes.c_int64 * 64),
                ("live_slot", ctypes.c_int * 64), ("draft_depth", ctypes.c_int), ("n_retired", ctypes.c_int),
                ("retired_job", ctypes.c_int64 * 64), ("retired_slot", ctypes.c_int * 64)]


@dataclass
class SchedJob:
    id: int
    prompt: list[int]
    max_new: int
    eos: Optional[int]
    eos2: Optional[int]
    sampling: SamplingOptions
    q: "queue.Queue" = field(default_factory=queue.Queue)
    seq: object = None
    next_token: Optional[int] = None
    emitted: int = 0
    finish: Optional[str] = None
    submitted: float = 0.0
    first_token_at: Optional[float] = None
    stats: SpecStats = field(default_factory=SpecStats)
    last_logits: Optional[torch.Tensor] = None


class Scheduler:
    def __init__(self, engine, width: int = 8, interleave_chunk: int = 1024, prefill_chunk: int = 4096,
                 hold_ms: float = 8.0, hold_long_ms: float = 100.0, depths: Sequence[int] = (0,), spec_rows: int = 32,
                 copy_drafts: bool = False, use_graph: bool = True, clock: Callable[[], float] = time.monotonic, drafter=None):
        self.engine = engine
        self.lib = _native.host()
        self.lib.grm_sched_new.restype = ctypes.c_void_p
        darr = (ctypes.c_int * len(depths))(*depths)
        self.h = ctypes.c_void_p(self.lib.grm_sched_new(width, engine.limits.max_ctx, interleave_chunk, prefill_chunk, 32768,
                                                        4096, ctypes.c_double(hold_ms), ctypes.c_double(hold_long_ms), darr,
                                                        len(depths), spec_rows))
        if not self.h:
            raise ValueError("scheduler width must be in 1..64")
        self.width = width
        self.use_graph = use_graph
        self.clock = clock
        # any object with the Drafter protocol (engine/generation.py): the MTP head's drafter, or prompt-lookup copy drafts
        self.drafter = drafter if drafter is not None else (CopyDrafter() if copy_drafts else None)
        if self.drafter is not None and any(d > 0 for d in depths) and hasattr(engine, "enable_speculation"):
            engine.enable_speculation()
        self.jobs: dict[int, SchedJob] = {}
        self._ids = itertools.count(1)
        self._lock = threading.Lock()
        self._wake = threading.Condition(self._lock)
        self._inbox: list[SchedJob] = []
        self._cancel: list[int] = []
        self._stop = False
        self.metrics = {"steps": 0, "rows": 0, "tokens": 0, "admit_rows": 0, "spec_rounds": 0, "spec_accepted": 0,
                        "ttft_ms": [], "errors": 0}
        self.thread = threading.Thread(target=self._run, name="grimoire-scheduler", daemon=True)
        self.thread.start()

    # ------------------------------------------------------------------------------------------
    # request side
    # ------------------------------------------------------------------------------------------
    def generate(self, prompt: Sequence[int], max_new: int, eos: Optional[int] = None, eos2: Optional[int] = None,
                 on_token: Optional[Callable[[int], bool]] = None, sampling: Optional[SamplingOptions] = None):
        """Blocks until the request finishes; ``on_token`` runs on the calling thread.
        Returns (tokens, finish_reason, job)."""
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) >= self.engine.limits.max_ctx:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit the context of {self.engine.limits.max_ctx}")
        job = SchedJob(next(self._ids), list(prompt), max_new, eos, eos2, (sampling or SamplingOptions()).validate(),
                       submitted=self.clock())
        with self._wake:
            if self._stop:
                raise RuntimeError("scheduler is shut down")
            self._inbox.append(job)
            self._wake.notify_all()
        out: list[int] = []
        while True:
            item = job.q.get()
            if item is None:
                break
            if isinstance(item, BaseException):
                raise item
            out.append(item)
            if on_token is not None and on_token(item) is False:
                with self._wake:
                    self._cancel.append(job.id)
                    self._wake.notify_all()
                # drain until the scheduler acknowledges
                while True:
                    it = job.q.get()
                    if it is None or isinstance(it, BaseException):
                        break
                job.finish = FinishReason.CANCELLED
                break
        return out, job.finish or FinishReason.LENGTH, job

    def shutdown(self, timeout: float = 30.0) -> None:
        """Graceful stop: live generations end at the next token, the step in flight completes."""
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        self.thread.join(timeout)
        if self.h:
            self.lib.grm_sched_delete(self.h)
            self.h = None

    # ------------------------------------------------------------------------------------------
    # engine side
    # ------------------------------------------------------------------------------------------
    def _now_ms(self) -> float:
        return self.clock() * 1000.0

    def _finish(self, job: SchedJob, reason: str) -> None:
        if job.finish is None:
            job.finish = reason
        self.lib.grm_sched_on_tokens(self.h, ctypes.c_int64(job.id), 0, 1)
        job.q.put(None)

    def _emit(self, job: SchedJob, tok: int) -> bool:
        """Push one token to the request thread; returns False when the job is finished."""
        if job.first_token_at is None:
            job.first_token_at = self.clock()
            self.metrics["ttft_ms"].append((job.first_token_at - job.submitted) * 1000.0)
        job.emitted += 1
        self.metrics["tokens"] += 1
        job.q.put(tok)
        done = tok == job.eos or tok == job.eos2
        state = self.lib.grm_sched_on_tokens(self.h, ctypes.c_int64(job.id), 1, 1 if done else 0)
        if done:
            job.finish = FinishReason.STOP
            job.q.put(None)
            return False
        if state == 3:
            job.finish = FinishReason.LENGTH
            job.q.put(None)
            return False
        return True

    def _fail(self, job: SchedJob, err: Exception) -> None:
        """End one request with an error; the scheduler core retires it on the next plan."""
        self.metrics["errors"] += 1
        job.finish = FinishReason.ERROR
        self.lib.grm_sched_on_tokens(self.h, ctypes.c_int64(job.id), 0, 1)
        job.q.put(err)

    def _pick(self, job: SchedJob, logits: torch.Tensor, position: int) -> int:
        if job.sampling.greedy:
            return first_token_of(logits)
        dev = getattr(self.engine, "sample_rows", None)
        if dev is not None and torch.is_tensor(logits):
            # the device sampler: no logits row travels to the host (the options of the row go up, 4 bytes come back)
            return dev(logits.reshape(1, -1), [job.sampling], [position])[0]
        return sample_ref(logits, job.sampling, position)

    def _run(self) -> None:
        plan = _Plan()
        eng = self.engine
        while True:
            with self._wake:
                inbox, self._inbox = self._inbox, []
                cancels, self._cancel = self._cancel, []
                stopping = self._stop
            for job in inbox:
                reused = 0
                rc = self.lib.grm_sched_submit(self.h, ctypes.c_int64(job.id), len(job.prompt), job.max_new, reused,
                                               ctypes.c_double(self._now_ms()))
                if rc != 0:
                    job.q.put(ValueError("prompt does not fit the context"))
                    continue
                self.jobs[job.id] = job
            for jid in cancels:
                self.lib.grm_sched_cancel(self.h, ctypes.c_int64(jid))
            if stopping:
                for job in self.jobs.values():
                    self.lib.grm_sched_cancel(self.h, ctypes.c_int64(job.id))
            self.lib.grm_sched_plan(self.h, ctypes.c_double(self._now_ms()), ctypes.byref(plan))
            # ---- retire ----
            for i in range(plan.n_retired):
                job = self.jobs.pop(plan.retired_job[i], None)
                if job is None:
                    continue
                if job.seq is not None:
                    try:
                        eng.release(job.seq, cache=True) if getattr(eng, "prefix_cache", None) is not None else eng.release(job.seq)
                    except Exception:
                        self.metrics["errors"] += 1
                if job.finish is None:
                    job.finish = FinishReason.CANCELLED
                    job.q.put(None)
            if stopping and not self.jobs:
                return
            if plan.kind == 0 or plan.kind == PLAN_WAIT:
                with self._wake:
                    if not self._inbox and not self._cancel and not self._stop:
                        self._wake.wait(timeout=(plan.wait_ms / 1000.0) if plan.kind == PLAN_WAIT else 0.05)
                continue
            try:
                if plan.kind & PLAN_ADMIT:
                    self._admit(plan)
                if plan.kind & PLAN_STEP:
                    self._step(plan)
            except Exception as e:  # engine failure: fail the affected jobs, keep serving
                self.metrics["errors"] += 1
                for job in list(self.jobs.values()):
                    if job.finish is None:
                        job.finish = FinishReason.ERROR
                        self.lib.grm_sched_on_tokens(self.h, ctypes.c_int64(job.id), 0, 1)
                        job.q.put(e)

    def _admit(self, plan: _Plan) -> None:
        eng = self.engine
        firsts = []
        # whole prompts that start from an empty slot share ONE M-row pass (admit_batch, grimoire.cpp:12071-12146)
        batched = set()
        can = getattr(eng, "can_prefill_batch", None)
        if plan.n_admit > 1 and can is not None and can():
            cand = []
            for i in range(plan.n_admit):
                job = self.jobs.get(plan.admit_job[i])
                if job is not None and job.seq is None and plan.admit_from[i] == 0 and plan.admit_to[i] == len(job.prompt):
                    cand.append((i, job))
            room = eng._prefill_rows
            chosen = []
            for i, job in cand:
                if len(job.prompt) <= room and len(chosen) < eng._prefill_logit_rows:
                    chosen.append((i, job))
                    room -= len(job.prompt)
            if len(chosen) > 1:
                seqs, taken = [], []
                for i, job in chosen:
                    seq = eng.open()
                    reused = eng.prefix_reuse(seq, job.prompt) if hasattr(eng, "prefix_reuse") else 0
                    job.seq = seq
                    if reused == 0:
                        seqs.append(seq)
                        taken.append((i, job))       # prompts with a cached prefix take the single path below
                if len(taken) > 1:
                    logits = eng.prefill_batch(seqs, [job.prompt for _, job in taken])
                    for (i, job), lg in zip(taken, logits):
                        batched.add(i)
                        self.metrics["admit_rows"] += len(job.prompt)
                        state = self.lib.grm_sched_on_prefilled(self.h, ctypes.c_int64(job.id), len(job.prompt))
                        if state == 2:
                            firsts.append((job, self._pick(job, lg, job.seq.length)))
                    self.metrics["admit_batches"] = self.metrics.get("admit_batches", 0) + 1
        for i in range(plan.n_admit):
            if i in batched:
                continue
            job = self.jobs.get(plan.admit_job[i])
            if job is None:
                continue
            lo, hi = plan.admit_from[i], plan.admit_to[i]
            if job.seq is None:
                job.seq = eng.open()
                if lo == 0 and hasattr(eng, "prefix_reuse"):
                    eng.prefix_reuse(job.seq, job.prompt)
            if lo == 0 and job.seq.length:
                lo = min(job.seq.length, len(job.prompt))          # tokens served by the prefix cache
                if lo >= hi:
                    hi = min(len(job.prompt), max(hi, lo))
            lo = max(lo, job.seq.length)
            logits = eng.prefill(job.seq, job.prompt[lo:hi]) if hi > lo or lo >= len(job.prompt) else None
            self.metrics["admit_rows"] += max(0, hi - lo)
            state = self.lib.grm_sched_on_prefilled(self.h, ctypes.c_int64(job.id), hi)
            if state == 2 and logits is not None:
                firsts.append((job, self._pick(job, logits, job.seq.length)))
        # first tokens of the round are flushed together (grimoire.cpp:24670-24686)
        for job, tok in firsts:
            job.next_token = tok
            self._emit(job, tok)

    def _step(self, plan: _Plan) -> None:
        eng = self.engine
        live = [self.jobs[plan.live_job[i]] for i in range(plan.n_live) if plan.live_job[i] in self.jobs]
        live = [j for j in live if j.finish is None and j.next_token is not None]
        if not live:
            return
        depth = plan.draft_depth if self.drafter is not None else 0
        tokens, seqs, positions, spans, stepped = [], [], [], [], []
        for job in live:
            drafts = []
            if depth > 0 and job.sampling.greedy:
                room = self.lib.grm_sched_remaining(self.h, ctypes.c_int64(job.id)) - 1
                d = max(0, min(depth, room))
                if d:
                    drafts = list(self.drafter.propose(eng, job.seq, job.next_token, d))[:d]
            block = [job.next_token] + drafts
            pos0 = job.seq.length
            kv = getattr(eng, "kv", None)
            if kv is not None:
                # map the pages of this job's rows now: a pool that stays short after evicting cached prefixes fails
                # this request only, the others keep decoding
                try:
                    kv.ensure(job.seq, pos0 + len(block))
                except OutOfPages as e:
                    self._fail(job, e)
                    continue
            spans.append((len(tokens), len(block)))
            stepped.append(job)
            tokens += block
            seqs += [job.seq] * len(block)
            positions += list(range(pos0, pos0 + len(block)))
        live = stepped
        if not live:
            return
        need_logits = any(not j.sampling.greedy for j in live)
        res = eng.decode_rows(tokens, seqs, positions, use_graph=self.use_graph, return_logits=need_logits)
        chosen, logits = (res if need_logits else (res, None))
        self.metrics["steps"] += 1
        self.metrics["rows"] += len(tokens)
        for job, (o, n) in zip(live, spans):
            block = tokens[o: o + n]
            accepted = 0
            while accepted < n - 1 and block[accepted + 1] == int(chosen[o + accepted]):
                accepted += 1
            if n > 1:
                job.stats.rounds += 1
                job.stats.drafted += n - 1
                job.stats.accepted += accepted
                self.metrics["spec_rounds"] += 1
                self.metrics["spec_accepted"] += accepted
            keep = block[: accepted + 1]
            pos0 = positions[o]
            eng.commit_rows([job.seq] * len(keep), keep, list(range(pos0, pos0 + len(keep))))
            if n > 1 and hasattr(eng, "rollback"):
                eng.rollback(job.seq, pos0 + len(keep))
            if self.drafter is not None:
                self.drafter.observe(eng, job.seq, keep, row0=o)       # model drafters track the newest hidden state
            alive = True
            for d in block[1: accepted + 1]:
                alive = self._emit(job, d)
                if not alive:
                    break
            if not alive:
                continue
            if job.sampling.greedy:
                nxt = int(chosen[o + accepted])
            else:
                nxt = self._pick(job, logits[o + accepted], pos0 + accepted + 1)
            job.next_token = nxt
            self._emit(job, nxt)
