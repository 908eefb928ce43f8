"""Hybrid DeltaNet + MoE decoder on the CPU path: end-to-end identities on a tiny configuration
(3 GDN : 1 gated-attention layers, 16 experts top-4 + shared) and op oracles."""
import math

import pytest
import torch

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.models.config import tiny_hybrid_moe
from grimoire_b200.models.hybrid import HybridModel
from grimoire_b200.ref import gdn_ref, moe_ref


@pytest.fixture(scope="module")
def eng():
    cfg = tiny_hybrid_moe(4)
    model = HybridModel.random(cfg, "cpu", seed=1, max_slots=4)
    return Engine(model, EngineLimits(max_slots=4, max_ctx=160, prefill_chunk=32, max_decode_rows=8))


def _prompt(n, seed=3):
    return torch.randint(0, 4096, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_generate_and_slot_state_is_reset(eng):
    a = eng.generate(_prompt(20), 8)
    b = eng.generate(_prompt(20), 8)          # same slot reused: state must have been zeroed
    assert a == b and len(a) == 8
    assert eng.kv.pages_used() == 0


def test_chunked_prefill_carries_recurrent_state(eng):
    p = _prompt(70)
    s1 = eng.open()
    a = eng.prefill(s1, p).clone()            # chunks of 32: state and conv ring cross chunk borders
    eng.release(s1)
    big = Engine(eng.model, EngineLimits(max_slots=4, max_ctx=160, prefill_chunk=128, max_decode_rows=8))
    s2 = big.open()
    b = big.prefill(s2, p).clone()
    big.release(s2)
    assert float((a - b).abs().max()) < 0.05 * max(1.0, float(b.abs().max())) and int(a.argmax()) == int(b.argmax())


def test_batched_decode_equals_solo(eng):
    sa, sb = eng.open(), eng.open()
    la, lb = eng.prefill(sa, _prompt(11, 5)), eng.prefill(sb, _prompt(37, 6))
    ta, tb = int(la.argmax()), int(lb.argmax())
    st = eng.model.state.clone(), eng.model.ring.clone()
    both, lg = eng.decode_rows([ta, tb], [sa, sb], [sa.length, sb.length], return_logits=True)
    lg = lg.clone()
    eng.model.state.copy_(st[0]); eng.model.ring.copy_(st[1])      # undo the step, then decode b alone
    solo, l1 = eng.decode_rows([tb], [sb], [sb.length], return_logits=True)
    assert both[1] == solo[0] and torch.allclose(lg[1], l1[0], atol=5e-3)      # CPU BLAS blocks differ per M
    eng.release(sa), eng.release(sb)


@pytest.mark.parametrize("keep", [1, 2, 3])
def test_verify_block_then_rollback_equals_sequential_decode(eng, keep):
    """A block of three rows of one conversation runs through the recurrent layers as one run; rolling back to ``keep``
    rows must leave KV, conv tails and DeltaNet state exactly where ``keep`` single steps leave them."""
    p = _prompt(29, 8)
    # sequential path: three single-row steps, logits of each
    s = eng.open()
    tok = int(eng.prefill(s, p).argmax())
    seq_tokens, seq_logits = [tok], []
    for _ in range(4):
        nxt, lg = eng.decode_rows([seq_tokens[-1]], [s], [s.length], use_graph=False, return_logits=True)
        seq_logits.append(lg[0].clone())
        eng.commit_rows([s], [seq_tokens[-1]], [s.length])
        seq_tokens.append(int(nxt[0]))
    eng.release(s)
    # block path: the same three tokens as one verify block, then keep only the first ``keep``
    s = eng.open()
    assert int(eng.prefill(s, p).argmax()) == tok
    pos0 = s.length
    block = seq_tokens[:3]
    if keep < 3:
        block = block[:keep] + [(seq_tokens[keep] + 1) % 4096] + block[keep + 1:]        # a wrong draft right after the kept rows
    nxt, lg = eng.decode_rows(block, [s] * 3, [pos0, pos0 + 1, pos0 + 2], use_graph=False, return_logits=True)
    for i in range(keep):
        assert int(nxt[i]) == seq_tokens[i + 1]
        assert float((lg[i] - seq_logits[i]).abs().max()) < 5e-3
    eng.commit_rows([s] * keep, block[:keep], list(range(pos0, pos0 + keep)))
    eng.rollback(s, pos0 + keep)
    assert s.length == pos0 + keep
    nxt2, lg2 = eng.decode_rows([seq_tokens[keep]], [s], [s.length], use_graph=False, return_logits=True)
    assert int(nxt2[0]) == seq_tokens[keep + 1]
    assert float((lg2[0] - seq_logits[keep]).abs().max()) < 5e-3
    eng.release(s)


def test_speculation_on_the_hybrid_model_keeps_greedy_tokens(eng):
    """Drafts with a mix of right and wrong tokens through verify blocks: the emitted stream equals plain greedy and
    some drafts are accepted (the reference's hybrid + MTP path, tools/test_spec_e2e.cpp: spec == plain)."""
    from grimoire_b200.engine.generation import GenerationOptions, OracleDrafter, SpecStats, generate_tokens

    prompt = _prompt(23, 9)
    plain, _ = generate_tokens(eng, prompt, GenerationOptions(max_new=18, use_graph=False))
    st = SpecStats()
    drafter = OracleDrafter(prompt + plain, accept=0.6, vocab=4096, seed=3)
    spec, _ = generate_tokens(eng, prompt, GenerationOptions(max_new=18, draft_depth=3, drafter=drafter, stats=st, use_graph=False))
    assert spec == plain
    assert st.rounds > 0 and 0 < st.accepted < st.drafted


def test_gdn_oracle_properties():
    torch.manual_seed(0)
    Hk, Hv, D = 1, 2, 8
    S = torch.zeros(Hv, D, D)
    k = gdn_ref.l2norm(torch.randn(Hk, D))
    v = torch.randn(Hv, D)
    # a = 1, beta = 1 from a zero state stores v k^T: reading with q = k returns v / sqrt(D)
    o = gdn_ref.gdn_step(S, k, k, v, torch.ones(Hv), torch.ones(Hv))
    assert torch.allclose(o, v / math.sqrt(D), atol=1e-5)
    # writing the same pair again changes nothing (delta rule: v - S k = 0)
    S2 = S.clone()
    gdn_ref.gdn_step(S2, k, k, v, torch.ones(Hv), torch.ones(Hv))
    assert torch.allclose(S, S2, atol=1e-5)
    y, ring = gdn_ref.conv4_silu(torch.ones(2, 3), torch.tensor([[0., 0., 0., 1.]] * 3), torch.zeros(3, 3))
    assert torch.allclose(y, torch.nn.functional.silu(torch.ones(2, 3))) and torch.equal(ring[:, -1], torch.ones(3))


def test_moe_oracle_route_and_shared_gate():
    torch.manual_seed(1)
    lg = torch.randn(4, 8)
    ids, w = moe_ref.route(lg, 3)
    assert torch.allclose(w.sum(-1), torch.ones(4)) and (w[:, :-1] >= w[:, 1:]).all()
    assert torch.equal(ids[:, 0], lg.argmax(-1))
