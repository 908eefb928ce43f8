"""Qwen4-Exp as a whole model: config parsing and refusals, loading by the family's tensor names, and the served logits
(chunked prompt, token-by-token decode, both sides of the sparse-attention budget, two conversations at once) against the
fp32 whole-model oracle that strings the operator oracles around the hybrid family's block oracles."""
import dataclasses

import pytest
import torch

from grimoire_b200.api import Grimoire
from grimoire_b200.config import EngineConfig
from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.models.config import ModelConfig, tiny_qwen4_exp
from grimoire_b200.models.qwen4_exp import Qwen4ExpModel
from grimoire_b200.ref import qwen4_exp_model_ref as oracle

from .fixtures.mini_model import write_qwen4_exp_checkpoint


def _ec(model, **kw):
    return EngineConfig(model=str(model), ctx=128, seq_slots=2, prefill_chunk=16, **kw)


def _ids(n, seed, vocab):
    return torch.randint(3, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.fixture(scope="module")
def ckpt(tmp_path_factory):
    cfg = tiny_qwen4_exp()
    d = tmp_path_factory.mktemp("q4e")
    sd = write_qwen4_exp_checkpoint(d, cfg, seed=3)
    return cfg, sd, d


def test_config_keys_defaults_and_refusals(ckpt):
    cfg, _, d = ckpt
    got = ModelConfig.from_dir(d)
    assert got.is_qwen4_exp and got.eos_token_id == cfg.eos_token_id               # first entry of the list
    for f in ("hc_count", "hc_lowrank", "ple_layer_ids", "ple_embed_dim", "ple_conv_kernel_size", "ngram_size", "heads_per_ngram",
              "ngram_vocab_size_base", "ngram_seed", "indexer_n_heads", "indexer_head_dim", "indexer_budget", "indexer_compress_ratio",
              "layer_types", "attn_output_gate", "norm_zero_centered", "partial_rotary_factor"):
        assert getattr(got, f) == getattr(cfg, f), f
    base = {"model_type": "qwen4_exp_text", "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 2, "vocab_size": 64}
    d0 = ModelConfig.from_hf(base)                                                  # the family's own defaults
    assert (d0.hc_count, d0.hc_lowrank, d0.ngram_size, d0.heads_per_ngram, d0.ple_embed_dim, d0.ngram_seed) == (4, 320, 3, 8, 128, 1234)
    assert d0.indexer_n_heads == 0 and d0.ple_layer_ids == []
    with pytest.raises(ValueError, match="together"):
        ModelConfig.from_hf(dict(base, indexer_n_heads=4, indexer_head_dim=64))
    with pytest.raises(ValueError, match="sigmoid"):
        ModelConfig.from_hf(dict(base, output_gate_type="sigmoid"))
    with pytest.raises(ValueError, match="1-based"):
        ModelConfig.from_hf(dict(base, ple_layer_ids=[0]))
    with pytest.raises(ValueError, match="hc_count"):
        ModelConfig.from_hf(dict(base, hc_count=1))


def test_served_logits_match_the_whole_model_oracle(ckpt):
    cfg, sd, d = ckpt
    g = Grimoire.load(_ec(d), device="cpu")
    assert isinstance(g.model, Qwen4ExpModel) and g.engine.prefix_cache is None
    ids = _ids(41, 1, cfg.vocab_size)
    q = lambda w: quantize(w.bfloat16().float(), Fmt.FP8_BLOCK).dequant().float()
    lists = {}
    want = oracle.forward_logits(cfg, {k: v.bfloat16().float() for k, v in sd.items()}, ids, weight_fn=q, trace=lists)
    # the sparse attention really drops tokens on the late rows (budget 16 + the block being filled), and keeps all on the early ones
    assert sorted(lists) == [i for i in range(cfg.num_hidden_layers) if cfg.is_attention_layer(i)]
    late = [t for t in lists[1][40] if t >= 0]
    assert len(late) == cfg.indexer_budget + 1 and 40 in late
    assert sorted(t for t in lists[1][13] if t >= 0) == list(range(14))
    got = g.score_ids(ids)                                   # one row per step: dense attention below the budget, selection above
    err = float((got - want).abs().max())
    assert err < 0.06 * float(want.abs().max()), (err, float(want.abs().max()))
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.9
    # chunked prompt (16-token chunks: the first below the budget, the others above it) ends on the same row
    picked, select = [], g.model.selector.select
    g.model.selector.select = lambda *a: picked.append(select(*a)) or picked[-1]
    s = g.engine.open()
    last = g.engine.prefill(s, ids).float()
    g.engine.release(s)
    g.model.selector.select = select
    # chunks 2 and 3 of both attention layers went through the selection, and the lists are the oracle's
    assert [tuple(p.shape) for p in picked] == [(16, 19), (16, 19), (9, 19), (9, 19)]
    assert picked[2][-1].tolist() == lists[1][40] and picked[3][-1].tolist() == lists[3][40]
    assert picked[0][0].tolist() == lists[1][16]
    assert float((last - want[-1]).abs().max()) < 0.06 * float(want.abs().max())
    assert float((last - got[-1]).abs().max()) < 0.03 * float(want.abs().max())
    # greedy continuation agrees with scoring the continued sequence
    out, _ = g.generate(ids, 5)
    full = g.score_ids(ids + out)
    assert [int(full[len(ids) - 1 + j].argmax()) for j in range(5)] == out
    g.close()


def test_two_conversations_keep_their_own_history(ckpt):
    """n-gram history, convolution tails, indexer caches and recurrent state are per conversation: interleaved decoding of
    two prompts gives each the tokens it gets alone."""
    cfg, _, d = ckpt
    g = Grimoire.load(_ec(d), device="cpu")
    a, b = _ids(23, 5, cfg.vocab_size), _ids(30, 6, cfg.vocab_size)
    alone = [g.generate(p, 6)[0] for p in (a, b)]
    eng = g.engine
    sa, sb = eng.open(), eng.open()
    ta, tb = int(eng.prefill(sa, a).argmax()), int(eng.prefill(sb, b).argmax())
    outs = ([ta], [tb])
    for _ in range(5):
        nxt = eng.decode_rows([outs[0][-1], outs[1][-1]], [sa, sb], [sa.length, sb.length])
        eng.commit_rows([sa, sb], [outs[0][-1], outs[1][-1]], [sa.length, sb.length])
        outs[0].append(int(nxt[0])), outs[1].append(int(nxt[1]))
    assert [outs[0], outs[1]] == alone
    with pytest.raises(NotImplementedError):
        eng.decode_rows([1, 2], [sa, sa], [sa.length, sa.length + 1])          # no verify blocks for this family
    eng.release(sa), eng.release(sb)
    # a slot that is reused starts from nothing
    again = g.generate(a, 6)[0]
    assert again == alone[0]
    # the continuous-batching scheduler serves the family too (no speculation: one row per conversation and step)
    out, why, job = g.scheduler().generate(b, 6)
    assert out == alone[1]
    g.close()


def test_dense_attention_variant_without_indexer_or_ngram_layers():
    """The family's keys are optional apart from the streams: no indexer -> dense attention, no ple_layer_ids -> no n-gram layers."""
    cfg = dataclasses.replace(tiny_qwen4_exp(2), indexer_n_heads=0, indexer_head_dim=0, indexer_budget=0, indexer_compress_ratio=0,
                              ple_layer_ids=[])
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.hybrid import _DictSource
    from grimoire_b200.models.synthetic import random_qwen4_exp_state_dict

    sd = random_qwen4_exp_state_dict(cfg, 2)
    m = Qwen4ExpModel.from_checkpoint(_DictSource(cfg, sd), "cpu")
    assert m.selector is None and all(x.ple is None and x.indexer is None for x in m.extra)
    ids = _ids(20, 2, cfg.vocab_size)
    q = lambda w: quantize(w.bfloat16().float(), Fmt.FP8_BLOCK).dequant().float()
    want = oracle.forward_logits(cfg, {k: v.bfloat16().float() for k, v in sd.items()}, ids, weight_fn=q)
    eng = Engine(m, EngineLimits(max_slots=2, max_ctx=64, prefill_chunk=8, max_decode_rows=4))
    last = eng.prefill(eng.open(), ids).float()
    assert float((last - want[-1]).abs().max()) < 0.06 * float(want.abs().max())
