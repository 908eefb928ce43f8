"""Single-request control loop: prefix reuse -> chunked prefill -> {emit; draft; verify; accept;
commit} with plain decoding as the fallback.

Same contract as the reference's ``generate_tokens<Engine>`` template (include/b70/generation.hpp:
82-432), which is written against an engine *concept* so host tests can drive it with fake engines
(tests/test_generation.cpp).  Here the concept is the ``EngineLike`` protocol: anything that offers
``open / release / prefill / decode_rows / commit_rows`` (and optionally ``draft`` / ``rollback`` /
``prefix_reuse``) can be driven -- the real ``Engine`` or the fakes of tests/test_generation.py.

Speculation: K draft tokens come from a drafter (MTP chain, copy / prompt-lookup, or none); ONE
verify pass scores the candidate block as K+1 rows of the same conversation; the longest prefix
whose drafts equal the target's greedy choices is accepted and the target's next choice after it is
the bonus token (grimoire.cpp:11597-11622).  Greedy speculative decoding reproduces plain greedy
tokens.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional, Protocol, Sequence


@dataclass
class SpecStats:
    """Accepted / drafted accounting per request (include/b70/generation.hpp:41-54)."""

    rounds: int = 0
    drafted: int = 0
    accepted: int = 0
    emitted: int = 0
    degraded_rounds: int = 0

    @property
    def accept_length(self) -> float:
        """Mean tokens emitted per verify round (accepted drafts + the bonus token)."""
        return (self.accepted + self.rounds) / self.rounds if self.rounds else 1.0

    def line(self) -> str:
        return (f"spec: rounds={self.rounds} drafted={self.drafted} accepted={self.accepted} "
                f"accept_len={self.accept_length:.2f} degraded={self.degraded_rounds}")


@dataclass
class GenerationOptions:
    max_new: int = 128
    eos: Optional[int] = None
    eos2: Optional[int] = None
    draft_depth: int = 0            # K; 0 disables speculation
    drafter: Optional["Drafter"] = None
    use_graph: bool = True
    stats: SpecStats = field(default_factory=SpecStats)


class FinishReason:
    STOP = "stop"
    LENGTH = "length"
    CANCELLED = "cancelled"
    ERROR = "error"


def generation_budget(prompt_len: int, max_tokens: int, ctx: int) -> int:
    """Tokens that may be generated for a prompt under the context cap; raises ValueError (HTTP 400
    upstream) when the prompt itself does not fit (include/b70/generation.hpp:62-69)."""
    if prompt_len <= 0:
        raise ValueError("empty prompt")
    if prompt_len >= ctx:
        raise ValueError(f"prompt of {prompt_len} tokens does not fit the context of {ctx}")
    return max(0, min(max_tokens, ctx - prompt_len))


class EngineLike(Protocol):
    def open(self, slot: Optional[int] = None): ...
    def release(self, seq) -> None: ...
    def prefill(self, seq, tokens, want_logits: bool = True): ...
    def decode_rows(self, tokens, seqs, positions, use_graph: bool = True, return_logits: bool = False): ...
    def commit_rows(self, seqs, tokens, positions) -> None: ...


class Drafter(Protocol):
    def propose(self, engine, seq, last_token: int, depth: int) -> list[int]: ...
    def observe(self, engine, seq, accepted_tokens: Sequence[int], row0: int = 0) -> None: ...


class CopyDrafter:
    """Prompt-lookup drafts: if the last ``n`` tokens occurred earlier in the conversation, propose
    what followed them (the reference's copy_propose, grimoire.cpp:24277; 646-687 tok/s on copy/edit
    tasks, README.md:291).  Needs no model."""

    def __init__(self, ngram: int = 3, min_ngram: int = 2):
        self.ngram, self.min_ngram = ngram, min_ngram

    def propose(self, engine, seq, last_token: int, depth: int) -> list[int]:
        hist = list(seq.tokens) + [last_token]
        for n in range(self.ngram, self.min_ngram - 1, -1):
            if len(hist) <= n:
                continue
            key = hist[-n:]
            # most recent earlier occurrence
            for start in range(len(hist) - n - 1, -1, -1):
                if hist[start: start + n] == key:
                    follow = hist[start + n: start + n + depth]
                    if follow:
                        return follow
                    break
        return []

    def observe(self, engine, seq, accepted_tokens, row0: int = 0) -> None:
        pass


class OracleDrafter:
    """Drafts with a dialled acceptance rate, for measuring the verify path on models whose real draft head predicts
    nothing useful (random weights): it knows the continuation plain greedy decoding produces (``truth`` = prompt +
    greedy output) and proposes it, replacing a draft by a wrong token with probability ``1 - accept`` per position
    (a deterministic hash of the position, so runs repeat).  The verified output is still the target's own."""

    def __init__(self, truth: Sequence[int], accept: float = 0.7, vocab: int = 1 << 30, seed: int = 0):
        self.truth, self.accept, self.vocab, self.seed = list(truth), float(accept), vocab, seed

    def _u(self, pos: int) -> float:
        x = (pos * 0x9E3779B97F4A7C15 + self.seed * 0xBF58476D1CE4E5B9 + 0x94D049BB133111EB) & ((1 << 64) - 1)
        x ^= x >> 31
        x = (x * 0xD6E8FEB86659FD93) & ((1 << 64) - 1)
        x ^= x >> 29
        return (x >> 11) / float(1 << 53)

    def propose(self, engine, seq, last_token: int, depth: int) -> list[int]:
        pos = seq.length + 1                      # index in ``truth`` of the token that follows ``last_token``
        out = []
        for j in range(depth):
            if pos + j >= len(self.truth):
                break
            t = self.truth[pos + j]
            if self._u(pos + j) >= self.accept:
                t = (t + 1) % self.vocab          # a wrong draft: everything after it is rejected too
            out.append(t)
        return out

    def observe(self, engine, seq, accepted_tokens, row0: int = 0) -> None:
        pass


def first_token_of(logits) -> int:
    """Greedy choice from a 1-D logits tensor, ties to the lowest index."""
    import torch

    lg = logits.float()
    mx = lg.max()
    return int(torch.nonzero(lg == mx)[0, 0])


def generate_tokens(engine: EngineLike, prompt: Sequence[int], opts: GenerationOptions,
                    on_token: Optional[Callable[[int], bool]] = None, seq=None):
    """Run one request to completion.  ``on_token(tok)`` returning False cancels at that token
    (client disconnect / stop signal).  Returns (tokens, finish_reason)."""
    own = seq is None
    if opts.draft_depth > 0 and opts.drafter is not None and hasattr(engine, "enable_speculation"):
        engine.enable_speculation()            # verify blocks and single rows on the same arithmetic from here on
    if own:
        seq = engine.open()
    out: list[int] = []
    reason = FinishReason.LENGTH
    try:
        reused = 0
        if hasattr(engine, "prefix_reuse"):
            reused = engine.prefix_reuse(seq, prompt)
        logits = engine.prefill(seq, list(prompt[reused:]))
        tok = first_token_of(logits)
        stats = opts.stats
        while len(out) < opts.max_new:
            out.append(tok)
            stats.emitted += 1
            if on_token is not None and on_token(tok) is False:
                reason = FinishReason.CANCELLED
                break
            if tok == opts.eos or tok == opts.eos2:
                reason = FinishReason.STOP
                break
            if len(out) >= opts.max_new:
                break
            pos = seq.length
            drafts: list[int] = []
            if opts.draft_depth > 0 and opts.drafter is not None:
                room = opts.max_new - len(out) - 1
                depth = max(0, min(opts.draft_depth, room))
                if depth:
                    drafts = list(opts.drafter.propose(engine, seq, tok, depth))[:depth]
            if not drafts:
                nxt = engine.decode_rows([tok], [seq], [pos], use_graph=opts.use_graph)
                engine.commit_rows([seq], [tok], [pos])
                if opts.drafter is not None:
                    opts.drafter.observe(engine, seq, [tok])      # a model drafter tracks the newest hidden state
                tok = int(nxt[0])
                continue
            # ---- verify: block [tok, d1..dK] as K+1 rows of this conversation ----
            block = [tok] + drafts
            try:
                verified = engine.decode_rows(block, [seq] * len(block), list(range(pos, pos + len(block))),
                                              use_graph=opts.use_graph)
            except NotImplementedError:
                # degraded round: the engine declined the batched verify -> plain step
                stats.degraded_rounds += 1
                nxt = engine.decode_rows([tok], [seq], [pos], use_graph=opts.use_graph)
                engine.commit_rows([seq], [tok], [pos])
                tok = int(nxt[0])
                continue
            accepted = 0
            while accepted < len(drafts) and drafts[accepted] == int(verified[accepted]):
                accepted += 1
            stats.rounds += 1
            stats.drafted += len(drafts)
            stats.accepted += accepted
            # commit tok + accepted drafts; rows past the accepted prefix are rolled back
            keep = block[: accepted + 1]
            engine.commit_rows([seq] * len(keep), keep, list(range(pos, pos + len(keep))))
            if hasattr(engine, "rollback"):
                engine.rollback(seq, pos + len(keep))
            opts.drafter.observe(engine, seq, keep)
            stop = False
            for d in drafts[:accepted]:
                out.append(d)
                stats.emitted += 1
                if on_token is not None and on_token(d) is False:
                    reason, stop = FinishReason.CANCELLED, True
                    break
                if d == opts.eos or d == opts.eos2:
                    reason, stop = FinishReason.STOP, True
                    break
                if len(out) >= opts.max_new:
                    stop = True
                    break
            if stop:
                break
            tok = int(verified[accepted])
    finally:
        if own:
            engine.release(seq)
    return out, reason
