"""Qwen4-Exp mechanisms as operators: HyperConnections, sparse-attention selection and gather attention, the n-gram
embedding's ids / gate / convolution.  The oracles (ref/qwen4_exp_ref.py) are checked against the properties the reference
spells out in include/b70/qwen4_exp.hpp and tests/test_qwen4_exp.cpp; the device operators (ops/qwen4_exp.py,
csrc/kernels/qwen4_exp_ops.cu) against the oracles."""
import math

import pytest
import torch

from grimoire_b200.ref import qwen4_exp_ref as R


def test_hyperconnection_oracle_properties():
    g = torch.Generator().manual_seed(0)
    hc, H, low = 4, 32, 8
    hyper = torch.randn(3, hc * H, generator=g)
    w = torch.zeros(hc * H)
    normed = R.hc_norm(hyper, w, hc, 1e-6)
    # each stream on its own variance: scaling one stream leaves the others' normed values alone
    h2 = hyper.clone(); h2[:, :H] *= 9
    assert torch.allclose(R.hc_norm(h2, w, hc, 1e-6)[:, H:], normed[:, H:], atol=1e-5)
    assert torch.allclose(normed.reshape(3, hc, H).pow(2).mean(-1), torch.ones(3, hc), atol=1e-3)
    # an untrained injection is the identity residual: inj = 0 -> 2 sigmoid(0) = 1
    block = torch.randn(3, H, generator=g)
    out = R.hc_combine(hyper, normed, block, torch.zeros(hc, hc * H), hc)
    assert torch.allclose(out.reshape(3, hc, H), hyper.reshape(3, hc, H) + block[:, None, :], atol=1e-6)
    # mix with up = 0: every gate is sigmoid(0) = 1/2 -> half the mean of the normed streams
    mix = R.hc_mix(normed, torch.randn(low, hc * H, generator=g), torch.zeros(hc * H, low), hc)
    assert torch.allclose(mix, 0.5 * normed.reshape(3, hc, H).mean(1), atol=1e-6)
    # the division by hc is inside the silu
    down, up = torch.randn(low, hc * H, generator=g) * 0.2, torch.randn(hc * H, low, generator=g) * 0.2
    a = R.hc_mix(normed, down, up, hc)
    wrong = (torch.sigmoid((torch.nn.functional.silu(normed @ down.t()) / hc) @ up.t()) * normed).reshape(3, hc, H).mean(1)
    assert float((a - wrong).abs().max()) > 1e-4


def test_qsa_oracle_properties():
    g = torch.Generator().manual_seed(1)
    q, keys = torch.randn(4, 16, generator=g), torch.randn(10, 16, generator=g)
    lg = R.qsa_index_logits(q, keys, visible=7)
    assert torch.isinf(lg[7:]).all() and (lg[:7] >= 0).all()
    want = torch.relu(q @ keys.t()).sum(0) / 4.0                       # relu per head, then the sum, then the scale
    assert torch.allclose(lg[:7], want[:7], atol=1e-6)
    assert not torch.allclose(lg[:7], torch.relu((q @ keys.t()).sum(0))[:7] / 4.0)
    assert R.qsa_topk_blocks(torch.tensor([0.5, 2.0, 2.0, 1.0]), 4, 3) == [1, 2, 3]
    assert R.qsa_topk_blocks(torch.tensor([0.5, 2.0]), 2, 4) == [1, 0, -1, -1]      # holes, never block 0 again
    # expand: ratio 4, budget 8, query at position 9 (seq_len 10): blocks 1 then 0, tail = tokens 8, 9 (+ one hole)
    idx = R.qsa_expand_blocks([1, 0], 4, 8, seq_len=10, query_pos=9)
    assert idx == [4, 5, 6, 7, 0, 1, 2, 3, 8, 9, -1]
    assert R.qsa_expand_blocks([-1, -1], 4, 8, seq_len=2, query_pos=1) == [-1] * 8 + [0, 1, -1]
    # gather attention == dense attention when the list is the whole visible range, and holes change nothing
    k, v = torch.randn(2, 12, 16, generator=g), torch.randn(2, 12, 16, generator=g)
    full = list(range(10))
    o = R.qsa_attention(q, k, v, full, 0.25)
    o2 = R.qsa_attention(q, k, v, [3, -1] + [i for i in full if i != 3] + [-1], 0.25)
    assert torch.allclose(o, o2, atol=1e-6)
    ref = torch.stack([torch.softmax((k[h // 2, :10] @ q[h]) * 0.25, 0) @ v[h // 2, :10] for h in range(4)])
    assert torch.allclose(o, ref, atol=1e-6)


def test_ple_oracle_properties():
    sizes, offsets, total = R.ngram_vocab_layout(1000, 4, layer_id=0)
    assert sizes == [1009, 1013, 1019, 1021] and offsets == [0, 1009, 2022, 3041] and total == 4062     # consecutive primes above the base
    assert R.ngram_vocab_layout(1000, 2, layer_id=1)[0] == [1019, 1021]                                   # the layer id continues the sequence
    mult = R.ngram_multipliers(3, 151936, 1234, 0)
    assert all(m % 2 == 1 and 0 < m for m in mult) and all(151935 * m < (1 << 63) for m in mult)
    assert R.ngram_multipliers(3, 151936, 1234, 1) != mult and R.ngram_multipliers(3, 151936, 99, 0) != mult
    eos, hp = 7, 2
    ids = R.ple_ngram_ids(50, [11, 12, 13], mult, sizes, offsets, context_len=2, heads_per_ngram=hp, eos=eos)
    assert all(offsets[h] <= ids[h] < offsets[h] + sizes[h] for h in range(4))
    # heads 0-1 are bigrams: they do not see the token two back; heads 2-3 are trigrams and do
    ids2 = R.ple_ngram_ids(50, [11, 99, 13], mult, sizes, offsets, 2, hp, eos)
    assert ids2[:2] == ids[:2] and ids2[2:] != ids[2:]
    # sticky EOS: anything older than an EOS reads as EOS, and before the sequence is EOS too
    a = R.ple_ngram_ids(50, [11, 12, eos], mult, sizes, offsets, 2, hp, eos)
    b = R.ple_ngram_ids(50, [11, 99, eos], mult, sizes, offsets, 2, hp, eos)
    assert a == b == R.ple_ngram_ids(50, [], mult, sizes, offsets, 2, hp, eos)
    # gate: per stream; value gated into every stream; conv input is the norm of the gated rows
    g = torch.Generator().manual_seed(2)
    hc, H = 2, 16
    key, query, value = torch.randn(3, hc * H, generator=g), torch.randn(3, hc * H, generator=g), torch.randn(3, H, generator=g)
    z = torch.zeros(hc * H)
    gated, conv_in = R.ple_gate(key, value, query, z, z, z, hc, 1e-6)
    gs = gated.reshape(3, hc, H) / value[:, None, :]
    assert torch.allclose(gs, gs[..., :1].expand_as(gs), atol=1e-5) and (gs > 0).all() and (gs < 1).all()
    assert torch.allclose(conv_in.reshape(3, hc, H).pow(2).mean(-1), torch.ones(3, hc), atol=1e-3)
    k2 = key.clone(); k2[:, :H] = -k2[:, :H]                               # flipping one stream's key flips only that stream's gate side
    g2, _ = R.ple_gate(k2, value, query, z, z, z, hc, 1e-6)
    assert torch.allclose(g2[:, H:], gated[:, H:], atol=1e-6) and not torch.allclose(g2[:, :H], gated[:, :H], atol=1e-4)
    # conv: both residuals are added; taps before the sequence read zero; dilation spaces the taps
    T, C = 6, hc * H
    ci, gt, hd = torch.randn(T, C, generator=g), torch.randn(T, C, generator=g), torch.randn(T, C, generator=g)
    w = torch.randn(C, 2, generator=g)
    out = R.ple_conv(ci, gt, hd, w, dilation=3)
    assert torch.allclose(out[0], hd[0] + gt[0] + torch.nn.functional.silu(w[:, 1] * ci[0]), atol=1e-6)
    assert torch.allclose(out[4], hd[4] + gt[4] + torch.nn.functional.silu(w[:, 1] * ci[4] + w[:, 0] * ci[1]), atol=1e-6)


def _hc(device, g, hc=4, H=128, low=32):
    from grimoire_b200.ops.qwen4_exp import HyperConnection

    nw = torch.randn(hc * H, generator=g) * 0.1
    down, up, inj = torch.randn(low, hc * H, generator=g) * 0.1, torch.randn(hc * H, low, generator=g) * 0.3, torch.randn(hc, hc * H, generator=g) * 0.1
    return HyperConnection(nw, down, up, inj, hc, 1e-6, device), (nw, down, up, inj)


def test_device_classes_on_cpu_follow_the_oracles():
    from grimoire_b200.ops.qwen4_exp import PleNgram, QsaSelector, qsa_gather_attention

    g = torch.Generator().manual_seed(3)
    hcm, (nw, down, up, inj) = _hc("cpu", g)
    hyper = torch.randn(3, 4 * 128, generator=g)
    out = torch.zeros(3, 128)
    hcm.mix(hyper, out)
    normed = R.hc_norm(hyper, nw, 4, 1e-6).bfloat16().float()
    assert torch.allclose(out, R.hc_mix(normed, down.bfloat16().float(), up.bfloat16().float(), 4), atol=1e-5)
    block = torch.randn(3, 128, generator=g)
    want = R.hc_combine(hyper, normed, block, inj.bfloat16().float(), 4)
    hcm.combine(hyper, block)
    assert torch.allclose(hyper, want, atol=1e-5)
    sel = QsaSelector(heads=4, head_dim=32, budget=16, ratio=4, device="cpu")
    q = torch.randn(2, 4, 32, generator=g).bfloat16()
    keys = torch.randn(9, 32, generator=g).bfloat16()
    idx = sel.select(q, keys, torch.tensor([37, 5], dtype=torch.int32), torch.tensor([38, 6], dtype=torch.int32))
    assert idx.shape == (2, 19) and idx[0, 16:].tolist() == [36, 37, -1] and idx[1, 16:].tolist() == [4, 5, -1]
    assert sorted(t for t in idx[1, :16].tolist() if t >= 0) == [0, 1, 2, 3]            # one complete block is all a 6-token sequence has
    k, v = torch.randn(2, 40, 32, generator=g).bfloat16(), torch.randn(2, 40, 32, generator=g).bfloat16()
    o = torch.zeros(2, 4, 32, dtype=torch.bfloat16)
    qsa_gather_attention(q, k, v, idx, o, 0.2)
    assert torch.allclose(o[0].float(), R.qsa_attention(q[0], k, v, idx[0].tolist(), 0.2), atol=1e-2)
    table = torch.randn(5000, 8, generator=g)
    ple = PleNgram(table, vocab_base=1000, vocab_size=4096, ngram_size=3, heads_per_ngram=2, seed=1234, layer_id=0, eos=7, device="cpu")
    ids = ple.ids([50, 51], history=[11, 12])
    assert ids.shape == (2, 4) and ids[0].tolist() == R.ple_ngram_ids(50, [11, 12], ple.mult, ple.sizes, ple.offsets, 2, 2, 7)
    assert ids[1].tolist() == R.ple_ngram_ids(51, [11, 12, 50], ple.mult, ple.sizes, ple.offsets, 2, 2, 7)
    assert ple.gather(ids).shape == (2, 32) and torch.equal(ple.gather(ids)[0, :8], table[ids[0, 0]])


@pytest.mark.gpu
def test_qwen4_exp_kernels_match_oracles():
    from grimoire_b200.ops import core as K
    from grimoire_b200.ops.qwen4_exp import QsaSelector, ple_conv, ple_gate, qsa_gather_attention

    g = torch.Generator().manual_seed(4)
    hcm, (nw, down, up, inj) = _hc("cuda", g, hc=4, H=256, low=64)
    for M in (1, 5):
        hyper = torch.randn(M, 4 * 256, generator=g)
        normed = R.hc_norm(hyper, nw, 4, 1e-6).bfloat16().float()
        for dt in (torch.float32, torch.bfloat16):
            out = torch.zeros(M, 256, dtype=dt, device="cuda")
            hcm.mix(hyper.cuda(), out)
            want = R.hc_mix(normed, down.bfloat16().float(), up.bfloat16().float(), 4)
            assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), float((out.float().cpu() - want).abs().max())
        block = torch.randn(M, 256, generator=g)
        hy = hyper.cuda()
        hcm.combine(hy, block.cuda())
        want = R.hc_combine(hyper, normed, block, inj.bfloat16().float(), 4)
        assert torch.allclose(hy.cpu(), want, atol=2e-2, rtol=2e-2), float((hy.cpu() - want).abs().max())
    sel_g, sel_c = QsaSelector(8, 64, 64, 16, "cuda"), QsaSelector(8, 64, 64, 16, "cpu")
    q = torch.randn(3, 8, 64, generator=g).bfloat16()
    keys = torch.randn(20, 64, generator=g).bfloat16()
    pos, sl = torch.tensor([300, 47, 15], dtype=torch.int32), torch.tensor([301, 48, 16], dtype=torch.int32)
    ig = sel_g.select(q.cuda(), keys.cuda(), pos.cuda(), sl.cuda()).cpu()
    ic = sel_c.select(q, keys, pos, sl)
    for r in range(3):                     # the same SET of tokens; near-equal logits may order two blocks differently
        assert sorted(ig[r].tolist()) == sorted(ic[r].tolist()), r
        assert ig[r, 64:].tolist() == ic[r, 64:].tolist()
    k, v = torch.randn(2, 320, 64, generator=g).bfloat16(), torch.randn(2, 320, 64, generator=g).bfloat16()
    o = torch.zeros(3, 8, 64, dtype=torch.bfloat16, device="cuda")
    qsa_gather_attention(q.cuda(), k.cuda(), v.cuda(), ig.cuda(), o, 0.125)
    for r in range(3):
        want = R.qsa_attention(q[r], k, v, ig[r].tolist(), 0.125)
        assert torch.allclose(o[r].float().cpu(), want, atol=2e-2, rtol=2e-2), (r, float((o[r].float().cpu() - want).abs().max()))
    hc, H = 4, 256
    key, query, value = torch.randn(5, hc * H, generator=g), torch.randn(5, hc * H, generator=g), torch.randn(5, H, generator=g)
    nk, nq, ncw = (torch.randn(hc * H, generator=g) * 0.1 for _ in range(3))
    gt, ci = ple_gate(key.cuda(), value.cuda(), query.cuda(), nk.cuda(), nq.cuda(), ncw.cuda(), hc, 1e-6)
    wg, wc = R.ple_gate(key, value, query, nk, nq, ncw, hc, 1e-6)
    assert torch.allclose(gt.cpu(), wg, atol=1e-4, rtol=1e-3) and torch.allclose(ci.cpu(), wc, atol=1e-3, rtol=1e-3)
    T, C, t0 = 7, hc * H, 4
    conv_in, gated, hidden = torch.randn(t0 + T, C, generator=g), torch.randn(T, C, generator=g), torch.randn(T, C, generator=g)
    w = torch.randn(C, 3, generator=g)
    out = ple_conv(conv_in.cuda(), gated.cuda(), hidden.cuda(), w.cuda(), dilation=3, t0=t0)
    want = ple_conv(conv_in, gated, hidden, w, dilation=3, t0=t0)
    assert torch.allclose(out.cpu(), want, atol=1e-4, rtol=1e-4)
    assert K.status_read()[0] == 0
