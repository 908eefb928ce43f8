"""Engine: one model on one device (one rank of a TP/PP group) with its KV pool, activation
buffers, chunked prefill, batched decode / verify and the replayable decode graph.

API parity with the reference's ``struct Grimoire`` (grimoire.cpp:2299-4500): ``prefill``,
``decode_batch``, ``decode_solo`` (= graph replay), ``argmax_token``, ``release``, slot admission,
``build_graph``/``step`` (grimoire.cpp:23640-23723: token / position live in device memory so the
recording stays valid).  The differences are structural: pooled 16-token int8 pages instead of
per-slot KV copies, one universal M-row forward, CUDA graphs instead of SYCL command graphs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..models.dense import Buffers, DenseModel, RowBatch
from ..ops import core as K
from ..ops.core import PAGE
from .kv import KvPool, OutOfPages, SeqSlot


@dataclass
class EngineLimits:
    max_slots: int = 8               # conversation slots (GRIMOIRE_SEQ_SLOTS / MAX_BATCH)
    max_ctx: int = 8192              # per-request context cap (--ctx)
    prefill_chunk: int = 4096        # GRIMOIRE_PREFILL_CHUNK
    max_decode_rows: int = 64        # rows of one batched decode / verify step
    kv_pages: int = 0                # 0 = max_slots * max_ctx / 16
    extra_kv_layers: int = 0         # KV layers beyond the model's own (1 for an MTP draft head)


class Engine:
    def __init__(self, model: DenseModel, limits: Optional[EngineLimits] = None):
        self.model = model
        self.cfg = model.cfg
        self.device = model.device
        self.limits = limits or EngineLimits()
        lim = self.limits
        K.apply_pdl_switch()
        n_attn = getattr(model, "kv_layer_count", len(model.layers)) + lim.extra_kv_layers   # attention layers of this stage
        self.mtp = None                  # models.mtp.MtpDrafter attaches itself here
        pages = lim.kv_pages or (lim.max_slots * ((lim.max_ctx + PAGE - 1) // PAGE))
        self.kv = KvPool(n_attn, model.geom.Hkv, model.geom.D, pages, lim.max_slots, lim.max_ctx, self.device)
        chunk = min(lim.prefill_chunk, lim.max_ctx)
        self.prefill_buf: Optional[Buffers] = None
        self._prefill_rows = chunk
        self._prefill_logit_rows = max(1, min(lim.max_slots, 64))
        self.decode_buf = model.make_buffers(lim.max_decode_rows, lim.max_decode_rows)
        # device-resident step inputs (graph replay reads these)
        i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=self.device)
        self.d_tokens, self.d_row_seq, self.d_row_pos = i32(lim.max_decode_rows), i32(lim.max_decode_rows), i32(lim.max_decode_rows)
        pin = self.device.type == "cuda"
        self.h_stage = torch.zeros(3, lim.max_decode_rows, dtype=torch.int32, pin_memory=pin)
        # verify blocks of a step as groups of rows for the one-pass verify attention: slot, first row, rows, first position
        self.h_groups = torch.zeros(4, lim.max_decode_rows, dtype=torch.int32, pin_memory=pin)
        self.d_groups = torch.zeros(4, lim.max_decode_rows, dtype=torch.int32, device=self.device)
        self.h_next = torch.zeros(lim.max_decode_rows, dtype=torch.int32, pin_memory=pin)
        self.prefix_cache = None
        self._verify: dict = {}           # slot -> (handle, first row, rows, first position) of its last verify block
        self._reused_head_logits = None
        self.graphs: dict[tuple, "torch.cuda.CUDAGraph"] = {}      # (rows, splits, distinct sequences)
        self.counters = {"prefill_rows": 0, "decode_steps": 0, "decode_rows": 0, "graph_replays": 0, "kernel_launches": 0}

    # ------------------------------------------------------------------------------------------
    # slots
    # ------------------------------------------------------------------------------------------
    def open(self, slot: Optional[int] = None) -> SeqSlot:
        seq = self.kv.open_slot(slot)
        if hasattr(self.model, "reset_slot"):
            self.model.reset_slot(seq.slot)        # recurrent state of hybrid models starts at zero
        return seq

    def release(self, seq: SeqSlot, cache: bool = False, head_logits=None) -> None:
        """Free the slot; with ``cache`` its KV stays resident in the prefix cache (cache_sequence,
        grimoire.cpp:12333) until evicted."""
        if cache and self.prefix_cache is not None:
            extra = None
            snap = getattr(self.model, "snapshot_slot", None)
            if snap is not None:
                # recurrent layers: the state after the last cached token travels with the entry; an entry whose token
                # record and cache length disagree cannot be resumed and is not kept
                if seq.length != len(seq.tokens):
                    self.kv.release(seq)
                    return
                extra = {"recurrent": snap(seq.slot)}
            self.prefix_cache.store(seq, head_logits, extra)
        self.kv.release(seq)

    def enable_prefix_cache(self, max_entries: int = 16):
        from .prefix_cache import PrefixCache

        self.prefix_cache = PrefixCache(self.kv, max_entries)
        return self.prefix_cache

    def prefix_reuse(self, seq: SeqSlot, prompt) -> int:
        """Attach the longest cached prefix of ``prompt`` to a fresh slot; returns tokens reused."""
        if self.prefix_cache is None:
            return 0
        n, logits = self.prefix_cache.reuse(seq, list(prompt))
        self._reused_head_logits = logits
        rec = self.prefix_cache.last_extra.get("recurrent") if n else None
        if rec is not None:
            self.model.load_slot(seq.slot, rec)
        return n

    def rollback(self, seq: SeqSlot, length: int) -> None:
        """Forget cached positions >= length (rows of a verify block past the accepted prefix); recurrent layers get
        their state of position ``length`` back (commit_spec_prefix, grimoire.cpp:12407-12482)."""
        v = self._verify.pop(seq.slot, None) if self._verify else None
        if v is not None:
            handle, row0, rows, pos0 = v
            self.model.commit_verify(handle, seq.slot, row0, length - pos0, rows, pos0, self.decode_buf)
        if seq.length > length or len(seq.pages) * PAGE > length + PAGE:
            self.kv.truncate(seq, length)

    # ------------------------------------------------------------------------------------------
    # prefill (one sequence, chunked)
    # ------------------------------------------------------------------------------------------
    def _ensure_prefill_buf(self):
        if self.prefill_buf is None:
            self.prefill_buf = self.model.make_buffers(self._prefill_rows, self._prefill_logit_rows,
                                                       dense_kv_tokens=max(self.limits.max_ctx, self._prefill_rows))

    def prefill(self, seq: SeqSlot, tokens: Sequence[int] | torch.Tensor, want_logits: bool = True) -> Optional[torch.Tensor]:
        """Append ``tokens`` to the sequence in chunks of ``prefill_chunk`` rows; returns the fp32
        logits of the last token (device tensor [V]) when ``want_logits``."""
        self._ensure_prefill_buf()
        if not torch.is_tensor(tokens):
            tokens = torch.tensor(list(tokens), dtype=torch.int32)
        tokens = tokens.to(torch.int32)
        n = int(tokens.shape[0])
        if n == 0:
            # an identical prompt was fully served by the prefix cache (prompt-head snapshot)
            lg, self._reused_head_logits = self._reused_head_logits, None
            return lg
        if self.prefix_cache is not None:
            self.prefix_cache.make_room((seq.length + n + PAGE - 1) // PAGE - len(seq.pages))
        if seq.length + n > self.limits.max_ctx:
            raise OutOfPages(f"prompt of {seq.length + n} tokens exceeds the context cap {self.limits.max_ctx}")
        self.kv.ensure(seq, seq.length + n)
        tok_dev = tokens.to(self.device, non_blocking=True)
        logits = None
        done = 0
        while done < n:
            m = min(self._prefill_rows, n - done)
            pos0 = seq.length
            rows = torch.arange(pos0, pos0 + m, dtype=torch.int32, device=self.device)
            rb = RowBatch(tok_dev[done: done + m], torch.full((m,), seq.slot, dtype=torch.int32, device=self.device), rows,
                          mode="prefill", q_pos0=pos0, seq_slot=seq.slot,
                          logits_rows=torch.tensor([m - 1], device=self.device))
            out = self.model.forward(rb, self.prefill_buf, self.kv.layers, self.kv.table)
            if self.mtp is not None:
                self.mtp.warm_chunk(seq, tok_dev, done, m, pos0, self.prefill_buf, last=(done + m == n))
            seq.length += m
            done += m
            self.counters["prefill_rows"] += m
            logits = out
        hook = getattr(self.model, "on_tokens", None)
        if hook is not None:
            hook(n)
        seq.tokens.extend(int(t) for t in tokens.tolist())
        pp = getattr(self.model, "pp", None)
        if pp is not None:
            # the last stage owns the logits; every stage needs the same first token
            row = logits[0] if logits is not None else torch.empty(self.cfg.vocab_size, dtype=torch.float32, device=self.device)
            logits = pp.broadcast_from_last(row)[None]
        return logits[0] if want_logits else None

    def can_prefill_batch(self) -> bool:
        """Several fresh prompts in one M-row pass: dense models without a draft head or pipeline stages."""
        return isinstance(self.model, DenseModel) and self.mtp is None and getattr(self.model, "pp", None) is None

    def prefill_batch(self, seqs: Sequence[SeqSlot], prompts: Sequence[Sequence[int]]) -> list[torch.Tensor]:
        """Read several whole prompts into fresh slots with ONE forward pass (admit_batch, grimoire.cpp:12071-12146): the
        projections run over the sum of the prompt lengths, attention per prompt.  Every sequence must be empty and the
        rows must fit one prefill chunk.  Returns the last-token logits of each prompt."""
        total = sum(len(p) for p in prompts)
        if not self.can_prefill_batch() or total > self._prefill_rows or any(s.length or s.pages for s in seqs) or \
                any(len(p) == 0 or len(p) > self.limits.max_ctx for p in prompts):
            raise ValueError("prefill_batch needs fresh slots, non-empty prompts and at most one chunk of rows in total")
        self._ensure_prefill_buf()
        if self.prefix_cache is not None:
            self.prefix_cache.make_room(sum((len(p) + PAGE - 1) // PAGE for p in prompts))
        toks, rs, rp, segs, last = [], [], [], [], []
        for s, p in zip(seqs, prompts):
            self.kv.ensure(s, len(p))
            segs.append((len(toks), len(p)))
            toks += [int(t) for t in p]
            rs += [s.slot] * len(p)
            rp += list(range(len(p)))
            last.append(len(toks) - 1)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32).to(self.device, non_blocking=True)
        rb = RowBatch(i32(toks), i32(rs), i32(rp), mode="prefill", q_pos0=0, seq_slot=seqs[0].slot, segments=segs,
                      logits_rows=torch.tensor(last, device=self.device))
        logits = self.model.forward(rb, self.prefill_buf, self.kv.layers, self.kv.table)
        for s, p in zip(seqs, prompts):
            s.length = len(p)
            s.tokens.extend(int(t) for t in p)
        self.counters["prefill_rows"] += total
        self.counters["prefill_batches"] = self.counters.get("prefill_batches", 0) + 1
        return [logits[i] for i in range(len(prompts))]

    # ------------------------------------------------------------------------------------------
    # batched decode / verify rows
    # ------------------------------------------------------------------------------------------
    def enable_speculation(self) -> None:
        """Speculative decoding is about to run on this engine: put every batch height on the batch-invariant projection
        kernels (ops/linear.py: set_batch_invariant), so that a token verified inside a block is the token plain greedy
        decoding would have produced, and drop decode graphs captured in the other mode."""
        from ..ops import linear as _lin

        if not _lin.BATCH_INVARIANT:
            _lin.set_batch_invariant(True)
            self.graphs.clear()

    def _stage_rows(self, tokens, slots, positions) -> int:
        M = len(tokens)
        st = self.h_stage
        st[0, :M] = torch.as_tensor(tokens, dtype=torch.int32)
        st[1, :M] = torch.as_tensor(slots, dtype=torch.int32)
        st[2, :M] = torch.as_tensor(positions, dtype=torch.int32)
        self.d_tokens[:M].copy_(st[0, :M], non_blocking=True)
        self.d_row_seq[:M].copy_(st[1, :M], non_blocking=True)
        self.d_row_pos[:M].copy_(st[2, :M], non_blocking=True)
        return M

    def _splits_for(self, M: int, max_len: int) -> int:
        return K.decode_splits(max_len, M, self.model.geom.Hkv)

    def _run_rows(self, M: int, splits: int, distinct: bool = False, runs=None, full_logits: bool = True, ngroups: int = 0) -> torch.Tensor:
        hs = getattr(self.model, "head_split", None)
        rb = RowBatch(self.d_tokens[:M], self.d_row_seq[:M], self.d_row_pos[:M], mode="decode", splits=splits, distinct=distinct, runs=runs,
                      full_logits=full_logits or hs is None, verify=(self.d_groups, ngroups) if ngroups else None)
        logits = self.model.forward(rb, self.decode_buf, self.kv.layers, self.kv.table)
        pp = getattr(self.model, "pp", None)
        if logits is not None and hs is not None and not rb.full_logits:
            # vocabulary-split head: the ranks exchange (value, index) candidates instead of logits rows
            self.model.tp.head_pick(logits, hs[0], hs[1], self.decode_buf.next_ids[:M])
        elif logits is not None:
            K.argmax_rows(logits, self.decode_buf.next_ids[:M])
        if pp is not None:
            pp.broadcast_from_last(self.decode_buf.next_ids[:M])     # token chosen by the last stage travels back
        return logits

    def decode_rows(self, tokens: Sequence[int], seqs: Sequence[SeqSlot], positions: Sequence[int],
                    use_graph: bool = True, return_logits: bool = False):
        """One step over M rows; row i appends ``tokens[i]`` at ``positions[i]`` of ``seqs[i]`` and
        returns the greedy next token per row (host list).  Rows of one sequence with consecutive
        positions form a speculative verify block."""
        M = len(tokens)
        if M == 0:
            return []
        if M > self.limits.max_decode_rows:
            raise ValueError("too many rows for one step")
        if not getattr(self.model, "supports_verify_rows", True) and len({s.slot for s in seqs}) != M:
            # recurrent layers advance one token per conversation per step: no multi-row verify blocks
            raise NotImplementedError("this model cannot score several rows of one conversation in one step")
        runs = None
        self._verify = {}
        if hasattr(self.model, "begin_verify") and len({s.slot for s in seqs}) != M:
            # verify blocks over recurrent layers: group the rows into runs and record what a rollback needs
            groups, i = [], 0
            while i < M:
                n = 1
                while i + n < M and seqs[i + n].slot == seqs[i].slot and positions[i + n] == positions[i] + n:
                    n += 1
                groups.append((seqs[i].slot, i, n, positions[i]))
                i += n
            if len({g[0] for g in groups}) != len(groups):
                raise ValueError("rows of one conversation must be consecutive positions in one block")
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=self.device)
            runs = (i32([g[0] for g in groups]), i32([g[1] for g in groups]), i32([g[2] for g in groups]))
            blocks = [g for g in groups if g[2] > 1]
            handle = self.model.begin_verify(i32([g[0] for g in blocks]), M)
            self._verify = {g[0]: (handle, g[1], g[2], g[3]) for g in blocks}
            use_graph = False
        max_len = 0
        for s, p in zip(seqs, positions):
            self.kv.ensure(s, p + 1)
            max_len = max(max_len, p + 1)
        if (runs is None and M > 1 and len({s.slot for s in seqs}) == 1 and max_len < K.VERIFY_ATTN_MIN_CTX
                and len({self._splits_for(1, p + 1) for p in positions}) > 1):
            # one conversation's verify block whose rows sit on both sides of a length at which the single-row split factor changes (once
            # per doubling of the context): score the rows one launch each, which is what plain decoding would do
            outs, lgs = [], []
            for t, s, p in zip(tokens, seqs, positions):
                r = self.decode_rows([t], [s], [p], use_graph=use_graph, return_logits=return_logits)
                if return_logits:
                    outs.append(r[0][0])
                    lgs.append(r[1][0].clone())
                else:
                    outs.append(r[0])
            return (outs, torch.stack(lgs)) if return_logits else outs
        self._stage_rows(tokens, [s.slot for s in seqs], positions)
        splits = self._splits_for(M, max_len)
        distinct = len({s.slot for s in seqs}) == M      # no verify block: the attention kernel may append K / V itself
        shape = ()
        if not distinct and max_len < K.VERIFY_ATTN_MIN_CTX:
            # Short contexts: every row of a verify block is scored exactly as a single-row step at its position would be
            # (the per-row kernel with the single-row split factor, whose page partition depends on the row's own length
            # only), so that speculative output reproduces plain greedy output bit for bit; the one-pass kernel is no
            # faster below this length anyway.
            splits = self._splits_for(1, max_len)
        elif not distinct and self.device.type == "cuda" and isinstance(self.model, DenseModel):
            # verify blocks: groups of consecutive rows of one conversation share one pass over its cache
            per = K.verify_rows_per_group(self.model.geom)
            if per >= 1:
                groups = K.verify_groups([s.slot for s in seqs], list(positions), per)
                n = len(groups)
                self.h_groups[:, :n] = torch.tensor(groups, dtype=torch.int32).t()
                self.d_groups[:, :n].copy_(self.h_groups[:, :n], non_blocking=True)
                shape = tuple(g[2] for g in groups)
                splits = K.decode_splits(max_len, n, self.model.geom.Hkv)
        tp = getattr(self.model, "tp", None)
        ep = getattr(self.model, "ep", None)
        if (tp is not None and not tp.fused) or (ep is not None and not ep.fused) or getattr(self.model, "pp", None) is not None:
            use_graph = False        # NCCL collectives / stage hops stay out of captured graphs
        full = return_logits or getattr(self.model, "head_split", None) is None
        if full and getattr(self.model, "head_split", None) is not None:
            use_graph = False        # whole logits rows of a split head are gathered by a library collective
        if not getattr(self.model, "graph_safe", True):
            use_graph = False        # the model does host work per step (n-gram ids from the step's tokens)
        if use_graph and self.device.type == "cuda":
            key = (M, splits, distinct) + ((shape,) if shape else ())
            g = self.graphs.get(key)
            if g is None:
                g = self._capture(M, splits, distinct, len(shape), key)
            g.replay()
            self.counters["graph_replays"] += 1
        else:
            self._run_rows(M, splits, distinct, runs, full_logits=full, ngroups=len(shape))
        if runs is not None:
            self.model.end_verify()
        self.h_next[:M].copy_(self.decode_buf.next_ids[:M], non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        self.counters["decode_steps"] += 1
        self.counters["decode_rows"] += M
        out = self.h_next[:M].tolist()
        if return_logits:
            return out, self.decode_buf.logits[:M]
        return out

    def sample_rows(self, logits: torch.Tensor, opts: Sequence, positions: Sequence[int]) -> list[int]:
        """Draw one token per logits row with per-row options (temperature / top-k / top-p / seed, the draw is a pure
        function of (seed, position): launch_sample_logits, src/sample_logits.hpp:41-134).  On a GPU the rows never leave
        the device: the options go up (a few bytes per row), the chosen ids come back (4 bytes per row)."""
        from .sampling import DeviceSampler, sample_ref

        n = logits.shape[0]
        if self.device.type != "cuda":
            self.counters["logits_d2h_bytes"] = self.counters.get("logits_d2h_bytes", 0)
            return [sample_ref(logits[i], opts[i], int(positions[i])) for i in range(n)]
        if getattr(self, "_sampler", None) is None:
            self._sampler = DeviceSampler(self.limits.max_decode_rows, self.device)
            self._sample_pos = torch.zeros(self.limits.max_decode_rows, dtype=torch.int32, device=self.device)
            self._sample_out = torch.zeros(self.limits.max_decode_rows, dtype=torch.int32, device=self.device)
        self._sampler.set_rows(list(opts))
        self._sample_pos[:n] = torch.tensor([int(p) for p in positions], dtype=torch.int32)
        self._sampler.sample(logits, self._sample_pos[:n], self._sample_out[:n])
        self.counters["sample_d2h_bytes"] = self.counters.get("sample_d2h_bytes", 0) + 4 * n
        return [int(v) for v in self._sample_out[:n].tolist()]

    def commit_rows(self, seqs: Sequence[SeqSlot], tokens: Sequence[int], positions: Sequence[int]) -> None:
        """Record that rows were appended (host bookkeeping after an accepted step)."""
        for s, t, p in zip(seqs, tokens, positions):
            if p == s.length:
                s.length += 1
                s.tokens.append(int(t))
        hook = getattr(self.model, "on_tokens", None)        # hybrid models flush their routing counts every few hundred tokens
        if hook is not None:
            hook(len(tokens))

    def _save_recurrent(self, M: int):
        fn = getattr(self.model, "save_recurrent", None)
        return fn(torch.unique(self.d_row_seq[:M])) if fn is not None else None

    def _restore_recurrent(self, saved) -> None:
        if saved is not None:
            self.model.restore_recurrent(saved)

    def _capture(self, M: int, splits: int, distinct: bool = False, ngroups: int = 0, key=None):
        # warm the allocator / workspace outside capture, then record; a model with recurrent state
        # must not keep the warm-up run's update
        saved = self._save_recurrent(M)
        full = getattr(self.model, "head_split", None) is None     # a split head is captured with its (value, index) pick
        self._run_rows(M, splits, distinct, full_logits=full, ngroups=ngroups)
        torch.cuda.current_stream().synchronize()
        self._restore_recurrent(saved)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._run_rows(M, splits, distinct, full_logits=full, ngroups=ngroups)
        self.graphs[key if key is not None else (M, splits, distinct)] = g
        return g

    # ------------------------------------------------------------------------------------------
    # self-feeding decode graph (token and position stay on the device between steps)
    # ------------------------------------------------------------------------------------------
    def build_step_graph(self, seqs: Sequence[SeqSlot], first_tokens: Sequence[int], steps_ahead: int):
        """Record one decode step for ``seqs`` that feeds its own arg-max back as the next input and
        bumps the positions on the device, so ``steps_ahead`` replays need no host round trip (the
        reference's build_graph/step contract, grimoire.cpp:23640-23723).  Pages for the next
        ``steps_ahead`` positions are mapped up front.  Returns the graph; tokens are read with
        ``read_next``."""
        M = len(seqs)
        max_len = 0
        for s in seqs:
            self.kv.ensure(s, s.length + steps_ahead + 1)
            max_len = max(max_len, s.length + steps_ahead + 1)
        self._stage_rows(first_tokens, [s.slot for s in seqs], [s.length for s in seqs])
        splits = self._splits_for(M, max_len)
        distinct = len({s.slot for s in seqs}) == M

        def body():
            self._run_rows(M, splits, distinct, full_logits=getattr(self.model, "head_split", None) is None)
            self.d_tokens[:M].copy_(self.decode_buf.next_ids[:M])
            self.d_row_pos[:M].add_(1)

        saved = (self.d_tokens[:M].clone(), self.d_row_pos[:M].clone())
        rec = self._save_recurrent(M)
        body()                       # warm-up outside capture (also sizes the workspace)
        torch.cuda.current_stream().synchronize()
        self.d_tokens[:M].copy_(saved[0]); self.d_row_pos[:M].copy_(saved[1])
        self._restore_recurrent(rec)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            body()
        self.d_tokens[:M].copy_(saved[0]); self.d_row_pos[:M].copy_(saved[1])
        torch.cuda.current_stream().synchronize()
        return g

    def read_next(self, M: int) -> list[int]:
        self.h_next[:M].copy_(self.decode_buf.next_ids[:M])
        torch.cuda.current_stream().synchronize()
        return self.h_next[:M].tolist()

    # ------------------------------------------------------------------------------------------
    # convenience: greedy generation for one sequence (CLI / tests)
    # ------------------------------------------------------------------------------------------
    def generate(self, prompt: Sequence[int], max_new: int, eos: Optional[int] = None, use_graph: bool = True,
                 collect_logits: bool = False):
        seq = self.open()
        out, logit_trace = [], []
        try:
            logits = self.prefill(seq, prompt)
            tok = int(K.ref.argmax_lowest(logits[None].float().cpu())[0]) if self.device.type != "cuda" else int(
                K.argmax_rows(logits[None], torch.zeros(1, dtype=torch.int32, device=self.device))[0])
            if collect_logits:
                logit_trace.append(logits.float().cpu().clone())
            for _ in range(max_new):
                out.append(tok)
                if eos is not None and tok == eos:
                    break
                if len(out) == max_new:
                    break
                pos = seq.length
                res = self.decode_rows([tok], [seq], [pos], use_graph=use_graph, return_logits=collect_logits)
                nxt = res[0] if collect_logits else res
                if collect_logits:
                    logit_trace.append(res[1][0].float().cpu().clone())
                self.commit_rows([seq], [tok], [pos])
                tok = int(nxt[0])
        finally:
            self.release(seq)
        return (out, logit_trace) if collect_logits else out
