"""Control-flow tests of the single-request loop with fake engines (tier T2 of the reference's
strategy, tests/test_generation.cpp:29-140): deterministic "next = prev + 1" engines, injectable
draft rejection, a verify that declines, cancellation, budget checks."""
import pytest
import torch

from grimoire_b200.engine.generation import (CopyDrafter, FinishReason, GenerationOptions, SpecStats, generate_tokens,
                                             generation_budget)

V = 1000


class FakeSeq:
    def __init__(self):
        self.length, self.tokens, self.slot, self.pages = 0, [], 0, []


class FakeEngine:
    """next token = (prev + 1) % V; verify rows are scored independently."""

    def __init__(self, decline_verify=False):
        self.decline_verify = decline_verify
        self.calls, self.rolled_back, self.released = [], [], 0

    def open(self, slot=None):
        return FakeSeq()

    def release(self, seq):
        self.released += 1

    def prefill(self, seq, tokens, want_logits=True):
        seq.tokens.extend(tokens)
        seq.length += len(tokens)
        lg = torch.zeros(V)
        lg[(tokens[-1] + 1) % V] = 1.0
        return lg

    def decode_rows(self, tokens, seqs, positions, use_graph=True, return_logits=False):
        if len(tokens) > 1 and self.decline_verify:
            raise NotImplementedError
        self.calls.append(len(tokens))
        # rows of a verify block must sit at consecutive positions after the cached prefix
        assert list(positions) == list(range(positions[0], positions[0] + len(tokens)))
        return [(t + 1) % V for t in tokens]

    def commit_rows(self, seqs, tokens, positions):
        for s, t, p in zip(seqs, tokens, positions):
            assert p == s.length
            s.length += 1
            s.tokens.append(t)

    def rollback(self, seq, length):
        self.rolled_back.append(length)


class ScriptedDrafter:
    """Proposes the right continuation but corrupts the draft at ``bad_at`` (0-based) every round."""

    def __init__(self, bad_at=None):
        self.bad_at, self.seen = bad_at, []

    def propose(self, engine, seq, last_token, depth):
        d = [(last_token + 1 + i) % V for i in range(depth)]
        if self.bad_at is not None and self.bad_at < depth:
            d[self.bad_at] = (d[self.bad_at] + 7) % V
        return d

    def observe(self, engine, seq, accepted_tokens):
        self.seen.append(list(accepted_tokens))


def test_plain_greedy():
    e = FakeEngine()
    out, why = generate_tokens(e, [5, 6, 7], GenerationOptions(max_new=6))
    assert out == [8, 9, 10, 11, 12, 13] and why == FinishReason.LENGTH and e.released == 1


def test_eos_stops():
    out, why = generate_tokens(FakeEngine(), [5], GenerationOptions(max_new=50, eos=9))
    assert out == [6, 7, 8, 9] and why == FinishReason.STOP


@pytest.mark.parametrize("bad_at,accepted_per_round", [(None, 3), (0, 0), (1, 1), (2, 2)])
def test_speculation_reproduces_plain_tokens(bad_at, accepted_per_round):
    plain, _ = generate_tokens(FakeEngine(), [1, 2, 3], GenerationOptions(max_new=17))
    e = FakeEngine()
    st = SpecStats()
    d = ScriptedDrafter(bad_at)
    out, why = generate_tokens(e, [1, 2, 3], GenerationOptions(max_new=17, draft_depth=3, drafter=d, stats=st))
    assert out == plain and why == FinishReason.LENGTH
    assert st.rounds > 0 and st.emitted == 17
    full_rounds = [s for s in d.seen if len(s) == accepted_per_round + 1]
    assert len(full_rounds) >= st.rounds - 1        # the last round may be clipped by the budget
    assert abs(st.accept_length - (accepted_per_round + 1)) < 0.6
    # every round rolls back to exactly the committed length
    assert all(a <= b for a, b in zip(e.rolled_back, e.rolled_back[1:]))


def test_declined_verify_degrades_to_plain_steps():
    st = SpecStats()
    e = FakeEngine(decline_verify=True)
    out, _ = generate_tokens(e, [1], GenerationOptions(max_new=5, draft_depth=3, drafter=ScriptedDrafter(), stats=st))
    assert out == [2, 3, 4, 5, 6] and st.degraded_rounds > 0 and st.rounds == 0


def test_cancel_from_callback_and_eos_inside_accepted_block():
    seen = []
    out, why = generate_tokens(FakeEngine(), [1], GenerationOptions(max_new=50), on_token=lambda t: (seen.append(t), len(seen) < 3)[1])
    assert why == FinishReason.CANCELLED and out == [2, 3, 4]
    out, why = generate_tokens(FakeEngine(), [1], GenerationOptions(max_new=50, eos=6, draft_depth=4, drafter=ScriptedDrafter()))
    assert out == [2, 3, 4, 5, 6] and why == FinishReason.STOP


def test_copy_drafter_finds_repeats():
    s = FakeSeq()
    s.tokens = [10, 11, 12, 13, 14, 20, 21, 10, 11]
    d = CopyDrafter(ngram=3, min_ngram=2)
    assert d.propose(None, s, 12, 3) == [13, 14, 20]
    assert d.propose(None, s, 99, 3) == []


def test_generation_budget():
    assert generation_budget(100, 50, 1024) == 50
    assert generation_budget(1000, 50, 1024) == 24
    with pytest.raises(ValueError):
        generation_budget(1024, 10, 1024)
    with pytest.raises(ValueError):
        generation_budget(0, 10, 1024)
