"""The DFlash block drafter (models/dflash_drafter.py): its block math against a plain restatement written here, the
context caches kept in step with the target through prefill chunks, plain steps and verified blocks, and speculative
generation with it through the public entry point (a random drafter is rarely right, so the point is that the output
stays the plain greedy output while blocks are drafted and verified).  Reference: dflash_draft,
src/grimoire.cpp:16516-17289; tools/ref_qwen3_dflash.py for the layer math."""
import json
import math

import pytest
import torch
import torch.nn.functional as F

from grimoire_b200.api import Grimoire
from grimoire_b200.config import EngineConfig
from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.engine.generation import GenerationOptions, generate_tokens
from grimoire_b200.formats.safetensors_io import save_file
from grimoire_b200.models.config import ModelConfig
from grimoire_b200.models.dense import DenseModel
from grimoire_b200.models.dflash import resolve_dflash_config
from grimoire_b200.models.dflash_drafter import DFlashDrafter, DFlashModel, random_dflash_state_dict
from grimoire_b200.models.synthetic import random_state_dict

from .fixtures.mini_model import write_checkpoint

TARGET = ModelConfig(hidden_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                     vocab_size=4096, intermediate_size=512, tie_word_embeddings=True, rope_theta=1e6)
DRAFT_JSON = json.dumps({"num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2,
                         "head_dim": 32, "intermediate_size": 256, "vocab_size": 4096, "rope_theta": 10000.0,
                         "layer_types": ["full_attention", "sliding_attention"], "sliding_window": 24,
                         "dflash_config": {"mask_token_id": 4095, "target_layer_ids": [0, 2], "block_size": 8}})


def _rms(x, w, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, theta):                       # x [rows][heads][D], NeoX halves
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = pos.float()[:, None] * inv[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def _naive_block(st, sd, taps, ids, L):
    """Everything from scratch in fp32 over bf16-rounded weights: context rows 0..L-1 from ``taps``, block ``ids`` at L.."""
    w = lambda n: sd[n].bfloat16().float()
    lin = lambda x, n: x.bfloat16().float() @ w(n).t()
    Hq, Hkv, D = st.n_heads, st.n_kv_heads, st.head_dim
    M = len(ids)
    ctx = lin(taps.reshape(L, -1), "fc.weight")
    cn = _rms(ctx, sd["hidden_norm.weight"])
    cpos, bpos = torch.arange(L), torch.arange(L, L + M)
    h = w("embed_tokens.weight")[torch.tensor(ids)]
    for i in range(st.n_layers):
        p = f"layers.{i}."
        kn, qn = sd[p + "self_attn.k_norm.weight"], sd[p + "self_attn.q_norm.weight"]
        ck = _rope(_rms(lin(cn, p + "self_attn.k_proj.weight").reshape(L, Hkv, D), kn), cpos, st.rope_theta).bfloat16().float()
        cv = lin(cn, p + "self_attn.v_proj.weight").reshape(L, Hkv, D).bfloat16().float()
        x = _rms(h, sd[p + "input_layernorm.weight"])
        q = _rope(_rms(lin(x, p + "self_attn.q_proj.weight").reshape(M, Hq, D), qn), bpos, st.rope_theta)
        k = _rope(_rms(lin(x, p + "self_attn.k_proj.weight").reshape(M, Hkv, D), kn), bpos, st.rope_theta)
        v = lin(x, p + "self_attn.v_proj.weight").reshape(M, Hkv, D)
        keys, vals, kpos = torch.cat([ck, k]), torch.cat([cv, v]), torch.cat([cpos, bpos])
        o = torch.zeros(M, Hq, D)
        for m in range(M):
            for hq in range(Hq):
                g = hq // (Hq // Hkv)
                sc = (keys[:, g] @ q[m, hq]) / math.sqrt(D)
                vis = torch.ones(L + M, dtype=torch.bool)
                if st.layers[i].causal:
                    vis &= kpos <= bpos[m]
                if st.layers[i].window > 0:
                    vis &= kpos > bpos[m] - st.layers[i].window
                sc = sc.masked_fill(~vis, float("-inf"))
                o[m, hq] = torch.softmax(sc, 0) @ vals[:, g]
        h = h + lin(o.reshape(M, Hq * D), p + "self_attn.o_proj.weight")
        x = _rms(h, sd[p + "post_attention_layernorm.weight"])
        h = h + lin(F.silu(lin(x, p + "mlp.gate_proj.weight")) * lin(x, p + "mlp.up_proj.weight"), p + "mlp.down_proj.weight")
    return _rms(h, sd["norm.weight"])


def test_block_math_matches_a_plain_restatement():
    st = resolve_dflash_config(DRAFT_JSON)
    assert not st.error and st.target_layers == [0, 2] and st.layers[1].window == 24 and st.layers[1].causal and not st.layers[0].causal
    sd = random_dflash_state_dict(st, TARGET.hidden_size, seed=3)
    m = DFlashModel(st, sd, "cpu", TARGET.hidden_size)
    L, M = 37, 6
    g = torch.Generator().manual_seed(1)
    taps = torch.randn(L, 2, TARGET.hidden_size, generator=g)
    ids = [17] + [st.mask_token] * (M - 1)
    pos = torch.arange(L, L + M)
    # context ingested in three pieces, as prefill chunks and committed steps would
    ck = [torch.zeros(64, m.Hkv, m.D, dtype=torch.bfloat16) for _ in m.layers]
    cv = [torch.zeros(64, m.Hkv, m.D, dtype=torch.bfloat16) for _ in m.layers]
    for a, b in ((0, 20), (20, 36), (36, 37)):
        for li, (k, v) in enumerate(m.context_kv(m.combine(taps[a:b]), torch.arange(a, b))):
            ck[li][a:b], cv[li][a:b] = k.bfloat16(), v.bfloat16()
    got = m.block(m.embed_block(torch.tensor(ids), m.embed), pos, list(zip(ck, cv)), L)
    want = _naive_block(st, sd, taps, ids, L)
    assert float((got - want).abs().max()) < 2e-2 * max(1.0, float(want.abs().max()))     # the drafter keeps bf16 products


def _engine():
    model = DenseModel.from_state_dict(TARGET, random_state_dict(TARGET, seed=0), "cpu")
    return Engine(model, EngineLimits(max_slots=2, max_ctx=160, prefill_chunk=32, max_decode_rows=16))


def test_drafter_keeps_context_in_step_and_output_stays_greedy():
    prompt = torch.randint(0, 4000, (45,), generator=torch.Generator().manual_seed(2)).tolist()
    plain, _ = generate_tokens(_engine(), prompt, GenerationOptions(max_new=20))
    eng = _engine()
    st = resolve_dflash_config(DRAFT_JSON)
    d = DFlashDrafter(eng, DFlashModel(st, random_dflash_state_dict(st, TARGET.hidden_size, seed=3), "cpu", TARGET.hidden_size), block_rows=5)
    assert eng.model.tap_index == {0: 0, 2: 1} and eng.decode_buf.taps.shape[1:] == (2, TARGET.hidden_size)
    seq = eng.open()
    opts = GenerationOptions(max_new=20, draft_depth=4, drafter=d)
    out, _ = generate_tokens(eng, prompt, opts, seq=seq)
    assert out == plain
    assert d.stats["blocks"] >= 3 and opts.stats.drafted >= 3 * 4
    # every committed position has context rows, ingested exactly once, and nothing beyond them
    assert d.have[seq.slot] == seq.length and d.stats["ctx_rows"] == seq.length
    # the cached context equals a from-scratch projection of the taps of a fresh single pass over the same tokens
    eng2 = _engine()
    eng2.model.set_taps(st.target_layers)
    eng2.model.add_tap_rows(eng2.decode_buf)
    s2 = eng2.open()
    toks = (prompt + out)[: seq.length]
    taps = []
    for a in range(0, len(toks), 32):
        eng2.prefill(s2, toks[a: a + 32])
        taps.append(eng2.prefill_buf.taps[: len(toks[a: a + 32])].clone())
    taps = torch.cat(taps)
    fresh = d.m.context_kv(d.m.combine(taps), torch.arange(len(toks)))
    for li, (k, v) in enumerate(fresh):
        assert torch.allclose(d.ck[li][seq.slot, : len(toks)].float(), k, atol=3e-2, rtol=3e-2)
        assert torch.allclose(d.cv[li][seq.slot, : len(toks)].float(), v, atol=3e-2, rtol=3e-2)


def test_dflash_model_flag_loads_a_drafter_directory(tmp_path):
    write_checkpoint(tmp_path / "target", TARGET, seed=0)
    st = resolve_dflash_config(DRAFT_JSON)
    dd = tmp_path / "draft"
    dd.mkdir()
    (dd / "config.json").write_text(DRAFT_JSON)
    save_file({k: v.bfloat16() for k, v in random_dflash_state_dict(st, TARGET.hidden_size, seed=3).items()}, dd / "model.safetensors")
    base = dict(ctx=160, seq_slots=2, prefill_chunk=32, prefix_cache=0, copy_drafts=0, proj="bf16")
    plain = Grimoire.load(EngineConfig(model=str(tmp_path / "target"), **base), device="cpu")
    spec = Grimoire.load(EngineConfig(model=str(tmp_path / "target"), dflash_model=str(dd), **base), device="cpu")
    assert isinstance(spec.drafter, DFlashDrafter) and spec.drafter.block_rows == 8
    prompt = list(range(100, 140))
    a, _ = plain.generate(prompt, 16)
    b, _ = spec.generate(prompt, 16, draft_depth=7)
    assert a == b and spec.drafter.stats["blocks"] > 0
    plain.close(), spec.close()


@pytest.mark.gpu
def test_drafter_on_gpu_keeps_greedy_output_with_graphs():
    from grimoire_b200.models.config import small_dense
    from grimoire_b200.ops import core as K

    cfg = small_dense(layers=4)
    sd = random_state_dict(cfg, seed=0)
    lim = EngineLimits(max_slots=2, max_ctx=256, prefill_chunk=64, max_decode_rows=16)
    prompt = torch.randint(0, cfg.vocab_size, (90,), generator=torch.Generator().manual_seed(2)).tolist()
    plain_eng = Engine(DenseModel.from_state_dict(cfg, sd, "cuda"), lim)
    plain_eng.enable_speculation()             # same (batch-invariant) arithmetic as the speculative run
    plain, _ = generate_tokens(plain_eng, prompt, GenerationOptions(max_new=24))
    eng = Engine(DenseModel.from_state_dict(cfg, sd, "cuda"), lim)
    js = json.loads(DRAFT_JSON)
    js["vocab_size"] = cfg.vocab_size
    js["dflash_config"]["mask_token_id"] = cfg.vocab_size - 1
    js["dflash_config"]["target_layer_ids"] = [0, 1, 2]
    st = resolve_dflash_config(json.dumps(js))
    d = DFlashDrafter(eng, DFlashModel(st, random_dflash_state_dict(st, cfg.hidden_size, seed=3), "cuda", cfg.hidden_size))
    seq = eng.open()
    opts = GenerationOptions(max_new=24, draft_depth=7, drafter=d, use_graph=True)
    out, _ = generate_tokens(eng, prompt, opts, seq=seq)
    assert out == plain
    assert d.stats["blocks"] >= 3 and d.have[seq.slot] == seq.length
    assert K.status_read()[0] == 0


DRAFT2_JSON = json.dumps({"num_hidden_layers": 2, "hidden_size": 128, "num_attention_heads": 4, "num_key_value_heads": 2,
                          "head_dim": 32, "intermediate_size": 256, "vocab_size": 4096, "rope_theta": 10000.0,
                          "dflash_config": {"mask_token_id": 4095, "target_layer_ids": [0, 2], "block_size": 8, "conv_kernel_size": 3,
                                            "conv_group_size": 32, "selector_rank": 16, "selector_top_k": 4,
                                            "input_embedding_scale": 1.5, "output_multiplier": 0.5, "final_logit_softcapping": 20.0}})


def _naive_conv(x, delta, base, taps, gs):
    rows, H = x.shape
    out = torch.zeros_like(x)
    for r in range(rows):
        for tap in range(taps):
            if r - tap < 0:
                continue
            for c in range(H):
                out[r, c] += (base[tap, c] + delta[r, tap, c // gs]) * x[r - tap, c]
    return out


def test_second_generation_convolutions_and_selector_match_a_plain_restatement():
    from grimoire_b200.models.dflash_drafter import GroupedConv

    st = resolve_dflash_config(DRAFT2_JSON)
    assert not st.error and st.conv_kernel_size == 3 and st.conv_group_size == 32 and st.selector_top_k == 4 and st.selector_rank == 16
    assert st.input_embedding_scale == 1.5 and st.output_multiplier == 0.5 and st.final_logit_softcapping == 20.0
    sd = random_dflash_state_dict(st, TARGET.hidden_size, seed=5)
    m = DFlashModel(st, sd, "cpu", TARGET.hidden_size)
    assert m.selector is not None and all(L.attn_conv is not None and L.mlp_conv is not None for L in m.layers)
    # the grouped convolution alone
    g = torch.Generator().manual_seed(2)
    x = torch.randn(6, 128, generator=g)
    cv = m.layers[0].attn_conv
    y, co = cv.prepare(x, m._lin)
    delta = m._lin(x, cv.proj).reshape(6, 2, 3, 4)
    assert torch.allclose(y, _naive_conv(x, delta[:, 0], cv.base[0], 3, 32), atol=1e-5)
    assert torch.allclose(cv.finish(x, co), _naive_conv(x, delta[:, 1], cv.base[1], 3, 32), atol=1e-5)
    # row 0 of a block never sees an earlier row: the same rows as a block of their own start afresh
    y2, _ = cv.prepare(x[2:], m._lin)
    assert torch.allclose(y2[0], (cv.base[0][0] + delta[2, 0, 0].repeat_interleave(32)) * x[2], atol=1e-5)
    # the selector: pair scores and the greedy walk, restated the way the reference's two kernels do it
    hidden = torch.randn(5, 128, generator=g)
    head = m.head
    got = m.select(hidden, head, anchor=77)
    lg = m.logits(hidden, head)
    assert float(lg.abs().max()) <= 20.0
    unary, cand = torch.topk(lg, 4, dim=-1)
    pred, succ, proj = (t.float() for t in m.selector)
    hp = (hidden.bfloat16() @ m.selector[2].t()).float()
    previous, want = 0, []
    for step in range(5):
        pid = 77 if step == 0 else int(cand[step - 1, previous])
        best, pick = -float("inf"), 0
        for c in range(4):
            gated = (pred[pid] * hp[step]).bfloat16().float()
            s = float(unary[step, c]) + float((gated * succ[int(cand[step, c])]).sum().bfloat16())
            if s > best:
                best, pick = s, c
        want.append(int(cand[step, pick]))
        previous = pick
    assert [int(t) for t in got] == want
    # and through the engine: the output stays the plain greedy output
    prompt = torch.randint(0, 4000, (45,), generator=torch.Generator().manual_seed(2)).tolist()
    plain, _ = generate_tokens(_engine(), prompt, GenerationOptions(max_new=12))
    eng = _engine()
    d = DFlashDrafter(eng, m, block_rows=5)
    out, _ = generate_tokens(eng, prompt, GenerationOptions(max_new=12, draft_depth=4, drafter=d))
    assert out == plain and d.stats["blocks"] >= 2


def test_block_drafter_under_the_continuous_batching_scheduler():
    """Two conversations decoded together by the scheduler with the block drafter attached: per-conversation context caches
    stay in step through interleaved verify blocks, and every conversation's output equals its plain greedy output."""
    import threading

    from grimoire_b200.sched.scheduler import Scheduler

    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, 4000, (n,), generator=g).tolist() for n in (21, 40)]
    alone = [generate_tokens(_engine(), p, GenerationOptions(max_new=12))[0] for p in prompts]
    eng = _engine()
    st = resolve_dflash_config(DRAFT_JSON)
    d = DFlashDrafter(eng, DFlashModel(st, random_dflash_state_dict(st, TARGET.hidden_size, seed=3), "cpu", TARGET.hidden_size), block_rows=4)
    s = Scheduler(eng, width=2, interleave_chunk=32, prefill_chunk=32, hold_ms=20.0, depths=(3, 3), spec_rows=16, drafter=d)
    res = [None, None]

    def work(i):
        res[i] = s.generate(prompts[i], 12)

    ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    [t.start() for t in ts]
    [t.join(timeout=180) for t in ts]
    s.shutdown()
    for i in range(2):
        assert res[i] is not None and res[i][0] == alone[i], (i, res[i], alone[i])
    assert d.stats["blocks"] >= 2


def test_block_drafter_taps_a_sandwich_norm_target():
    """The reference taps Muse-Glimmer and Gemma-4 targets for its block drafter (forward_muse / forward_gemma4 store the
    taps): the sandwich decoder keeps the same residual taps, so the drafter attaches to it unchanged."""
    from grimoire_b200.models.config import tiny_muse
    from grimoire_b200.models.gemma4 import MuseModel
    from grimoire_b200.models.synthetic import random_gemma4_state_dict

    cfg = tiny_muse()
    sd = random_gemma4_state_dict(cfg, 3)
    lim = EngineLimits(max_slots=2, max_ctx=160, prefill_chunk=32, max_decode_rows=16)
    prompt = torch.randint(0, 4000, (45,), generator=torch.Generator().manual_seed(2)).tolist()
    plain, _ = generate_tokens(Engine(MuseModel.from_state_dict(cfg, sd, "cpu"), lim), prompt, GenerationOptions(max_new=10))
    eng = Engine(MuseModel.from_state_dict(cfg, sd, "cpu"), lim)
    st = resolve_dflash_config(DRAFT_JSON)
    d = DFlashDrafter(eng, DFlashModel(st, random_dflash_state_dict(st, cfg.hidden_size, seed=3), "cpu", cfg.hidden_size), block_rows=4)
    seq = eng.open()
    out, _ = generate_tokens(eng, prompt, GenerationOptions(max_new=10, draft_depth=3, drafter=d), seq=seq)
    assert out == plain and d.stats["blocks"] >= 2 and d.have[seq.slot] == seq.length
    assert float(eng.decode_buf.taps.abs().max()) > 0
