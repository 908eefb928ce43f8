"""Every way a model reaches the engine through ``Grimoire.load``: synthetic presets of both families, HF checkpoints of
the hybrid family (per-expert and fused expert tensors) checked against the fp32 whole-model oracle, the checkpoint's
MTP draft head, and the pre-quantised artifact round trip (CPU path; the reference's counterpart is the model-matrix
gate, tools/test_model_matrix.cpp, over tools/mini_model.hpp fixtures)."""
import dataclasses

import pytest
import torch

from grimoire_b200.api import Grimoire, UnsupportedModel
from grimoire_b200.config import EngineConfig
from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.models.config import tiny_dense, tiny_hybrid_moe
from grimoire_b200.models.hybrid import HybridModel
from grimoire_b200.ref import hybrid_reference

from .fixtures.mini_model import write_checkpoint, write_hybrid_checkpoint


def _ec(model, **kw):
    base = dict(model=str(model), ctx=192, seq_slots=4, prefill_chunk=64, prefix_cache=0, mtp=0, copy_drafts=0)
    base.update(kw)
    return EngineConfig(**base)


def _prompt(n, seed=3, vocab=4096):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def test_synthetic_presets_dispatch_by_family():
    g = Grimoire.load(_ec("synthetic:tiny_hybrid_moe"), device="cpu")
    assert isinstance(g.model, HybridModel)
    out, why = g.generate(_prompt(12), 5)
    assert len(out) == 5
    g.close()
    g = Grimoire.load(_ec("synthetic:tiny_dense"), device="cpu")
    assert not isinstance(g.model, HybridModel)
    g.close()
    with pytest.raises(UnsupportedModel):
        Grimoire.load(_ec("synthetic:tiny_hybrid_moe", tp_world=2, tp_rank=0), device="cpu")


@pytest.fixture(scope="module")
def hybrid_dirs(tmp_path_factory):
    cfg = tiny_hybrid_moe(4)
    a, b = tmp_path_factory.mktemp("hyb_split"), tmp_path_factory.mktemp("hyb_fused")
    sd = write_hybrid_checkpoint(a, cfg, seed=5, fused_experts=False)
    write_hybrid_checkpoint(b, cfg, seed=5, fused_experts=True)
    return cfg, sd, a, b


def test_hybrid_checkpoint_matches_fp32_oracle(hybrid_dirs):
    cfg, sd, split_dir, fused_dir = hybrid_dirs
    g = Grimoire.load(_ec(split_dir), device="cpu")
    assert isinstance(g.model, HybridModel) and len(g.model.layers) == 4
    ids = _prompt(21, 9)
    got = g.score_ids(ids)
    # like with like: the oracle sees the same bf16 storage and block-fp8 round trip of every projection
    q = lambda w: quantize(w.bfloat16().float(), Fmt.FP8_BLOCK).dequant().float()
    want = hybrid_reference.forward_logits(cfg, {k: v.bfloat16().float() for k, v in sd.items()}, ids, weight_fn=q)
    err = float((got - want).abs().max())
    assert err < 0.06 * float(want.abs().max()), (err, float(want.abs().max()))
    agree = (got.argmax(-1) == want.argmax(-1)).float().mean()
    assert float(agree) >= 0.9
    g2 = Grimoire.load(_ec(fused_dir), device="cpu")
    got2 = g2.score_ids(ids)
    assert torch.allclose(got, got2, atol=1e-5), float((got - got2).abs().max())
    g.close(), g2.close()


@pytest.mark.parametrize("preset", ["tiny_hybrid_dense", "tiny_moe"])
def test_hybrid_family_neighbours_match_fp32_oracle(preset, tmp_path):
    """The 27B-style hybrid with a dense FFN (int4 projections) and a Qwen3-MoE-style decoder (plain attention, no shared
    expert) load through the same class and agree with the fp32 oracle under their own weight round trip; greedy
    continuation through the engine (prefill + decode steps, recurrent state included) follows the oracle's argmax."""
    from grimoire_b200.models.config import PRESETS

    cfg = PRESETS[preset]()
    sd = write_hybrid_checkpoint(tmp_path / preset, cfg, seed=9)
    g = Grimoire.load(_ec(tmp_path / preset), device="cpu")
    assert isinstance(g.model, HybridModel)
    dense_ffn = not cfg.is_moe
    assert g.model.proj == ("int4" if dense_ffn else "fp8")
    assert all((l.moe is None) == dense_ffn for l in g.model.layers)
    if not dense_ffn:
        assert all(l.moe.shared_gu is None and l.kind == "attn" for l in g.model.layers) and not g.model.geom.q_gated
    ids = _prompt(23, 11)
    got = g.score_ids(ids)
    fmt = Fmt.INT4 if dense_ffn else Fmt.FP8_BLOCK
    q = lambda w: quantize(w.bfloat16().float(), fmt).dequant().float()
    want = hybrid_reference.forward_logits(cfg, {k: v.bfloat16().float() for k, v in sd.items()}, ids, weight_fn=q)
    err = float((got - want).abs().max())
    assert err < 0.06 * float(want.abs().max()), (err, float(want.abs().max()))
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.9
    out, _ = g.generate(ids, 4)
    full = g.score_ids(ids + out)
    assert [int(full[len(ids) - 1 + j].argmax()) for j in range(4)] == out
    g.close()


def test_qwen3_moe_with_dense_layers_on_the_sparse_step(tmp_path):
    """Qwen3-MoE's ``mlp_only_layers`` / ``decoder_sparse_step``: dense and MoE feed-forwards in one model."""
    import dataclasses

    from grimoire_b200.models.config import ModelConfig, tiny_moe

    cfg = dataclasses.replace(tiny_moe(4), intermediate_size=384, mlp_only_layers=[0], decoder_sparse_step=2)
    assert [cfg.layer_is_sparse(i) for i in range(4)] == [False, True, False, True]
    sd = write_hybrid_checkpoint(tmp_path / "m", cfg, seed=3)
    parsed = ModelConfig.from_dir(tmp_path / "m")
    assert parsed.mlp_only_layers == [0] and parsed.decoder_sparse_step == 2
    g = Grimoire.load(_ec(tmp_path / "m"), device="cpu")
    assert [L.moe is not None for L in g.model.layers] == [False, True, False, True]
    ids = _prompt(19, 4)
    got = g.score_ids(ids)
    q = lambda w: quantize(w.bfloat16().float(), Fmt.FP8_BLOCK).dequant().float()
    want = hybrid_reference.forward_logits(cfg, {k: v.bfloat16().float() for k, v in sd.items()}, ids, weight_fn=q)
    assert float((got - want).abs().max()) < 0.06 * float(want.abs().max())
    g.close()


def test_k2_horizon_checkpoint_matches_fp32_oracle(tmp_path):
    """K2-Horizon: dense first layer, sparse layers with the routed value projection and the sigmoid / selection-bias router,
    two-group norms, softplus attention gate, ungated shared expert -- config parsing, loading by the family's tensor names,
    logits against the fp32 oracle, greedy continuation following the model's own scores."""
    from grimoire_b200.models.config import ModelConfig, tiny_k2

    cfg = tiny_k2()
    # (with random routers a token whose two best experts score within the engine-vs-oracle rounding difference picks another
    # expert, and a flipped VALUE expert moves every later row; this seed has no such near-tie, so the comparison is strict)
    sd = write_hybrid_checkpoint(tmp_path / "k2", cfg, seed=14)
    parsed = ModelConfig.from_dir(tmp_path / "k2")
    for f in ("norm_groups", "attn_gate_proj", "router_sigmoid", "router_scale", "num_shared_experts", "shared_expert_intermediate_size",
              "mova_experts", "mova_top_k", "mlp_only_layers", "decoder_sparse_step", "qk_norm", "norm_zero_centered"):
        assert getattr(parsed, f) == getattr(cfg, f), f
    assert [parsed.layer_is_sparse(i) for i in range(3)] == [False, True, True]
    g = Grimoire.load(_ec(tmp_path / "k2"), device="cpu")
    assert isinstance(g.model, HybridModel)
    assert [(L.moe is not None, L.mova is not None, L.gate_proj is not None, L.router_bias is not None) for L in g.model.layers] == \
        [(False, False, True, False), (True, True, True, True), (True, True, True, True)]
    ids = _prompt(23, 12)
    got = g.score_ids(ids)
    q = lambda w: quantize(w.bfloat16().float(), Fmt.FP8_BLOCK).dequant().float()
    want = hybrid_reference.forward_logits(cfg, {k: v.bfloat16().float() for k, v in sd.items()}, ids, weight_fn=q)
    err = float((got - want).abs().max())
    assert err < 0.06 * float(want.abs().max()), (err, float(want.abs().max()))
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.9
    out, _ = g.generate(ids, 4)
    full = g.score_ids(ids + out)
    assert [int(full[len(ids) - 1 + j].argmax()) for j in range(4)] == out
    g.close()


def test_hybrid_prefix_cache_restores_recurrent_state(hybrid_dirs):
    _, _, split_dir, _ = hybrid_dirs
    g = Grimoire.load(_ec(split_dir, prefix_cache=1), device="cpu")
    eng = g.engine
    p1 = _prompt(37, 21)
    s = eng.open()
    lg = eng.prefill(s, p1)
    first = int(lg.argmax())
    eng.release(s, cache=True)
    # a prompt that extends the cached conversation resumes from its KV pages AND its DeltaNet / conv state
    p2 = p1 + [first] + _prompt(9, 22)
    s2 = eng.open()
    n = eng.prefix_reuse(s2, p2)
    assert n == len(p1)
    a = eng.prefill(s2, p2[n:]).clone()
    eng.release(s2)
    eng.prefix_cache.entries.clear()
    s3 = eng.open()
    assert eng.prefix_reuse(s3, p2) == 0
    b = eng.prefill(s3, p2).clone()
    eng.release(s3)
    assert int(a.argmax()) == int(b.argmax()) and float((a - b).abs().max()) < 0.05 * max(1.0, float(b.abs().max()))
    # a prompt that diverges inside the cached entry cannot use its end-of-sequence state
    s4 = eng.open()
    s5 = eng.open()
    eng.prefill(s4, p1)
    eng.release(s4, cache=True)
    assert eng.prefix_reuse(s5, p1[:20] + _prompt(10, 23)) == 0
    eng.release(s5)
    g.close()


def test_mtp_head_from_checkpoint_drafts_and_keeps_greedy(tmp_path):
    cfg = dataclasses.replace(tiny_dense(), tie_word_embeddings=False)
    write_checkpoint(tmp_path, cfg, seed=2, mtp=True)
    plain = Grimoire.load(_ec(tmp_path), device="cpu")
    assert plain.drafter is None
    ids = _prompt(30, 4)
    want, _ = plain.generate(ids, 16)
    plain.close()
    g = Grimoire.load(_ec(tmp_path, mtp=1), device="cpu")
    assert g.drafter is not None and len(g.engine.kv.layers) == cfg.num_hidden_layers + 1
    from grimoire_b200.engine.generation import SpecStats

    st = SpecStats()
    got, _ = g.generate(ids, 16, draft_depth=3, stats=st)
    assert got == want and st.rounds > 0 and st.drafted > 0
    out, why, job = g.scheduler().generate(ids, 16)
    assert out == want
    g.close()


def test_artifact_round_trip_serves_same_logits(tmp_path):
    from grimoire_b200.formats.artifact import quantize_checkpoint

    cfg = dataclasses.replace(tiny_dense(), tie_word_embeddings=False)
    src = tmp_path / "src"
    write_checkpoint(src, cfg, seed=7, tokenizer=False, mtp=True)
    out = tmp_path / "bundle"
    stats = quantize_checkpoint(src, out, Fmt.INT4, policy="linear", bundle=True)
    assert stats["quantized"] > 0 and (out / "model-v3.grm").exists() and (out / "config.json").exists()
    ids = _prompt(17, 8)
    a = Grimoire.load(_ec(src), device="cpu")
    la = a.score_ids(ids)
    a.close()
    b = Grimoire.load(_ec(out), device="cpu")                       # the bundle directory
    lb = b.score_ids(ids)
    b.close()
    c = Grimoire.load(_ec(out / "model-v3.grm", mtp=1), device="cpu")   # the file itself, with its draft head
    assert c.drafter is not None
    lc = c.score_ids(ids)
    c.close()
    assert torch.allclose(la, lb, atol=1e-4), float((la - lb).abs().max())
    assert torch.allclose(lb, lc, atol=1e-6)


def test_expert_placement_from_heat_file_keeps_logits_and_balances_ranks(hybrid_dirs, tmp_path, monkeypatch):
    """A routing-heat file (models/expert_placement.py) permutes expert ownership at load: the experts' weights and the
    router rows move together, so the logits do not change, and the hot experts spread over the expert-parallel ranks."""
    from grimoire_b200.models.expert_placement import ExpertHeat, rank_loads

    cfg, _, split_dir, _ = hybrid_dirs
    ids = _prompt(21, 9)
    g = Grimoire.load(_ec(split_dir), device="cpu")
    base = g.score_ids(ids)
    g.close()
    heat = ExpertHeat(cfg.num_hidden_layers, cfg.num_experts)
    gen = torch.Generator().manual_seed(2)
    for l in range(cfg.num_hidden_layers):
        # skewed traffic: the first quarter of the experts takes most of it
        hot = torch.randint(0, cfg.num_experts // 4, (400,), generator=gen).tolist()
        cold = torch.randint(0, cfg.num_experts, (100,), generator=gen).tolist()
        heat.credit(l, hot + cold)
    path = str(tmp_path / "hits.json")
    heat.save(path)
    monkeypatch.setenv("GRIMOIRE_EXPERT_HEAT", path)
    g = Grimoire.load(_ec(split_dir), device="cpu")            # one rank: the file is read, the placement is the identity
    assert g.model.expert_perm is not None and g.model.expert_perm[0] == list(range(cfg.num_experts))
    g.close()
    # any placement leaves the logits alone (bit for bit: the experts' weights and the router rows move together)
    from grimoire_b200.engine.engine import Engine, EngineLimits

    def last_logits(perms):
        m = HybridModel.from_checkpoint(split_dir, "cpu", max_slots=2, expert_perm=perms)
        eng = Engine(m, EngineLimits(max_slots=2, max_ctx=64, prefill_chunk=32, max_decode_rows=4))
        return eng.prefill(eng.open(), ids).float()

    perms = [torch.randperm(cfg.num_experts, generator=gen).tolist() for _ in range(cfg.num_hidden_layers)]
    assert torch.equal(last_logits(perms), last_logits(None))
    # the same file, two ranks: each rank's share of the recorded traffic is close to half (identity order: ~0.85 / 0.15)
    m = HybridModel(cfg, "cpu", max_slots=2)
    m.ep_rank, m.ep_world = 0, 2
    assert m.set_expert_placement(path)
    h2 = ExpertHeat(cfg.num_hidden_layers, cfg.num_experts)
    assert h2.load(path)
    loads = rank_loads(h2.h[0], m.expert_perm[0], 2)
    ident = rank_loads(h2.h[0], list(range(cfg.num_experts)), 2)
    assert max(loads) / sum(loads) < 0.56 < max(ident) / sum(ident)


def test_mtp_head_on_a_dense_ffn_hybrid_target_keeps_greedy(tmp_path):
    """The 27B-style hybrid (Gated DeltaNet + gated attention, dense FFN) with its checkpoint's one-layer draft head:
    speculative decoding returns the plain greedy tokens, the head's KV layer sits after the target's attention layers,
    and rejected rows leave the recurrent state as plain decoding would."""
    from grimoire_b200.engine.generation import SpecStats
    from grimoire_b200.models.config import tiny_hybrid_dense

    cfg = tiny_hybrid_dense(4)
    write_hybrid_checkpoint(tmp_path, cfg, seed=6, mtp=True)
    plain = Grimoire.load(_ec(tmp_path), device="cpu")
    assert plain.drafter is None
    ids = _prompt(45, 8)
    want, _ = plain.generate(ids, 20)
    plain.close()
    g = Grimoire.load(_ec(tmp_path, mtp=1), device="cpu")
    assert isinstance(g.model, HybridModel) and g.drafter is not None
    assert len(g.engine.kv.layers) == cfg.num_attention_layers() + 1
    st = SpecStats()
    got, _ = g.generate(ids, 20, draft_depth=3, stats=st)
    assert got == want and st.rounds > 0 and st.drafted > 0
    out, why, job = g.scheduler().generate(ids, 20)
    assert out == want
    g.close()


def test_live_routing_counts_land_in_the_hit_file(hybrid_dirs, tmp_path, monkeypatch):
    """``GRIMOIRE_EXPERT_HITS``: a serving process counts its routing decisions per (layer, expert) and adds them to the hit
    file; a second process adds to the same file; counts are per logical expert whatever placement the model was loaded
    with; the file is the one the placement reads at the next load."""
    import json

    from grimoire_b200.engine.engine import Engine, EngineLimits

    cfg, _, split_dir, _ = hybrid_dirs
    path = tmp_path / "hits.json"
    monkeypatch.setenv("GRIMOIRE_EXPERT_HITS", str(path))
    ids = _prompt(40, 5)
    g = Grimoire.load(_ec(split_dir), device="cpu")
    out, _ = g.generate(ids, 8)
    g.close()
    first = torch.tensor(json.loads(path.read_text())["hits"])
    k = cfg.num_experts_per_tok
    rows = len(ids) + len(out) - 1                         # every prompt row and every decode step but the last token's
    assert first.shape == (cfg.num_hidden_layers, cfg.num_experts)
    assert all(int(first[l].sum()) == rows * k for l in range(cfg.num_hidden_layers)), first.sum(1)
    g = Grimoire.load(_ec(split_dir), device="cpu")
    g.generate(ids, 8)
    g.close()
    assert torch.equal(torch.tensor(json.loads(path.read_text())["hits"]), 2 * first)
    # a permuted placement routes the same logical experts
    gen = torch.Generator().manual_seed(4)
    perms = [torch.randperm(cfg.num_experts, generator=gen).tolist() for _ in range(cfg.num_hidden_layers)]
    counted = []
    for tag, pm in (("plain", None), ("perm", perms)):
        p2 = tmp_path / f"{tag}.json"
        m = HybridModel.from_checkpoint(split_dir, "cpu", max_slots=2, expert_perm=pm)
        m.record_expert_hits(str(p2), every=16)
        eng = Engine(m, EngineLimits(max_slots=2, max_ctx=64, prefill_chunk=32, max_decode_rows=4))
        eng.generate(ids, 8)
        assert p2.exists()                                  # flushed on the way, every 16 tokens
        m.save_expert_hits()
        counted.append(torch.tensor(json.loads(p2.read_text())["hits"]))
    assert torch.equal(counted[0], counted[1]) and int(counted[0].sum()) > 0
    monkeypatch.delenv("GRIMOIRE_EXPERT_HITS")
    monkeypatch.setenv("GRIMOIRE_EXPERT_HEAT", str(path))
    g = Grimoire.load(_ec(split_dir), device="cpu")
    assert g.model.expert_perm is not None
    g.close()


def test_host_resident_experts_give_the_same_logits(hybrid_dirs, tmp_path, monkeypatch):
    """The RAM tier: with ``GRIMOIRE_EXPERT_VRAM_PER_LAYER`` experts per layer on the device the others stay in host memory
    as the same fp8 blocks and the CPU pool computes their routes -- same logits and tokens as the all-device model; with a
    heat file the hottest experts are the resident ones, so fewer routes leave the device."""
    import json

    from grimoire_b200.ops.cpu_experts import CpuExperts

    cfg, _, split_dir, _ = hybrid_dirs
    ids = _prompt(70, 13)                                  # longer than a decode block: prompt rows go through the sorted path
    g = Grimoire.load(_ec(split_dir), device="cpu")
    base = g.score_ids(ids[:24])
    s = g.engine.open()
    base_last = g.engine.prefill(s, ids).float()
    g.engine.release(s)
    want, _ = g.generate(ids, 6)
    g.close()
    hits = tmp_path / "hits.json"
    monkeypatch.setenv("GRIMOIRE_EXPERT_HITS", str(hits))
    g = Grimoire.load(_ec(split_dir), device="cpu")
    g.generate(ids, 6)
    g.close()
    monkeypatch.delenv("GRIMOIRE_EXPERT_HITS")
    served = {}
    for tag, heat in (("first", ""), ("hot", str(hits))):
        monkeypatch.setenv("GRIMOIRE_EXPERT_VRAM_PER_LAYER", "4")
        if heat:
            monkeypatch.setenv("GRIMOIRE_EXPERT_HEAT", heat)
        g = Grimoire.load(_ec(split_dir), device="cpu")
        pools = [L.cx for L in g.model.layers]
        assert all(isinstance(c, CpuExperts) and c.n == cfg.num_experts - 4 for c in pools)
        assert all(L.moe.gate_up.shape[0] == 4 for L in g.model.layers) and g.model.graph_safe is False
        got = g.score_ids(ids[:24])
        assert float((got - base).abs().max()) < 1e-2 * float(base.abs().max()), float((got - base).abs().max())   # summation order differs; bf16 activations and the int8 cache amplify it
        s = g.engine.open()
        last = g.engine.prefill(s, ids).float()
        g.engine.release(s)
        assert float((last - base_last).abs().max()) < 1e-2 * float(base_last.abs().max())
        assert float((got.argmax(-1) == base.argmax(-1)).float().mean()) >= 0.95
        out, _ = g.generate(ids, 6)
        assert out[0] == want[0] and len(out) == 6              # a random model's near-ties may part later tokens
        served[tag] = sum(c.rows_served for c in pools)
        g.close()
    assert 0 < served["hot"] < served["first"], served
    total = json.loads(hits.read_text())["hits"]
    assert sum(map(sum, total)) > 0


def test_run_time_expert_swaps_follow_the_traffic(hybrid_dirs, tmp_path, monkeypatch):
    """``GRIMOIRE_EXPERT_SWAPS``: the heat of the routes the host sees promotes hot host experts into device slots at step
    boundaries -- weights, scales, router rows and the placement move together, so the logits stay, fewer routes leave the
    device on the same traffic, and the routing counts still name logical experts."""
    import json

    cfg, _, split_dir, _ = hybrid_dirs
    ids = _prompt(48, 21)
    ref_hits = tmp_path / "ref.json"
    monkeypatch.setenv("GRIMOIRE_EXPERT_HITS", str(ref_hits))
    g = Grimoire.load(_ec(split_dir), device="cpu")
    base = g.score_ids(ids[:20])
    g.close()
    hits = tmp_path / "hits.json"
    monkeypatch.setenv("GRIMOIRE_EXPERT_HITS", str(hits))
    monkeypatch.setenv("GRIMOIRE_EXPERT_VRAM_PER_LAYER", "6")
    monkeypatch.setenv("GRIMOIRE_EXPERT_SWAPS", "4")
    g = Grimoire.load(_ec(split_dir), device="cpu")
    m = g.model
    assert m.heat is not None and m.expert_perm[0] == list(range(cfg.num_experts))
    pools = [L.cx for L in m.layers]
    served = []
    for _ in range(4):                                   # the same traffic again and again: the placement adapts to it
        before = sum(c.rows_served for c in pools)
        s = g.engine.open()
        g.engine.prefill(s, ids)
        g.engine.release(s)
        served.append(sum(c.rows_served for c in pools) - before)
    assert m.swaps_done > 0 and any(p != list(range(cfg.num_experts)) for p in m.expert_perm)
    assert all(sorted(p) == list(range(cfg.num_experts)) for p in m.expert_perm)
    assert served[-1] < served[0], served
    got = g.score_ids(ids[:20])
    assert float((got - base).abs().max()) < 1e-2 * float(base.abs().max())
    assert float((got.argmax(-1) == base.argmax(-1)).float().mean()) >= 0.95
    with pytest.raises(ValueError):
        m.swap_experts(0, m.expert_perm[0][0], m.expert_perm[0][1])           # both on the device
    g.close()
    # counts per logical expert: 4 prompt passes + one scoring pass here against one scoring pass of the all-device model
    a, b = torch.tensor(json.loads(hits.read_text())["hits"]), torch.tensor(json.loads(ref_hits.read_text())["hits"])
    assert int(a.sum()) == (4 * len(ids) + 20) * cfg.num_experts_per_tok * cfg.num_hidden_layers
    assert int(b.sum()) == 20 * cfg.num_experts_per_tok * cfg.num_hidden_layers
    assert float(torch.corrcoef(torch.stack([a.float().flatten(), b.float().flatten()]))[0, 1]) > 0.5


def test_agnes_checkpoint_names_and_parallel_ffn_fold(tmp_path):
    """Agnes: ``agnes_delta_attention`` / ``agnes_global_attention`` layer types, ``delta_attn`` / ``global_attn`` tensor names
    and a second SwiGLU inside every mlp that is folded into the main one at load -- the served logits are those of the
    oracle that adds the two SwiGLUs separately; an unknown layer type and a missing parallel projection are refused."""
    import json

    from safetensors.torch import save_file

    from grimoire_b200.models.config import ModelConfig, tiny_hybrid_dense

    base = tiny_hybrid_dense(4)
    I, P, H = 384, 128, base.hidden_size
    cfg = dataclasses.replace(base, intermediate_size=I + P)
    from grimoire_b200.models.synthetic import random_hybrid_state_dict

    folded = random_hybrid_state_dict(cfg, seed=8)            # the equivalent model with one wide SwiGLU per layer
    sd = {}
    for k, v in folded.items():
        k2 = k.replace(".linear_attn.", ".delta_attn.").replace(".self_attn.", ".global_attn.")
        if k.endswith("mlp.gate_proj.weight") or k.endswith("mlp.up_proj.weight"):
            sd[k2], sd[k2.replace("mlp.", "mlp.parallel_ffn.")] = v[:I].clone(), v[I:].clone()
        elif k.endswith("mlp.down_proj.weight"):
            sd[k2], sd[k2.replace("mlp.", "mlp.parallel_ffn.")] = v[:, :I].clone(), v[:, I:].clone()
        else:
            sd[k2] = v
    tc = {"model_type": "agnes_text", "hidden_size": H, "num_hidden_layers": 4, "num_attention_heads": cfg.num_attention_heads,
          "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "vocab_size": cfg.vocab_size, "intermediate_size": I,
          "parallel_ffn_intermediate_size": P, "rms_norm_eps": cfg.rms_norm_eps,
          "rope_parameters": {"rope_theta": cfg.rope_theta, "partial_rotary_factor": cfg.partial_rotary_factor, "mrope_section": [11, 11, 10]},
          "layer_types": ["agnes_delta_attention" if t != "full_attention" else "agnes_global_attention" for t in cfg.layer_types],
          "linear_num_key_heads": cfg.linear_num_key_heads, "linear_num_value_heads": cfg.linear_num_value_heads,
          "linear_key_head_dim": cfg.linear_key_head_dim, "linear_value_head_dim": cfg.linear_value_head_dim,
          "linear_conv_kernel_dim": cfg.linear_conv_kernel_dim}
    d = tmp_path / "agnes"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"model_type": "agnes", "tie_word_embeddings": False, "text_config": tc}))
    save_file({k: v.bfloat16() for k, v in sd.items()}, d / "model.safetensors", {"format": "pt"})
    got_cfg = ModelConfig.from_dir(d)
    assert got_cfg.is_agnes and got_cfg.intermediate_size == I + P and got_cfg.parallel_ffn_intermediate_size == P
    assert got_cfg.layer_types == cfg.layer_types and got_cfg.attn_output_gate and got_cfg.norm_zero_centered
    g = Grimoire.load(_ec(d), device="cpu")
    assert isinstance(g.model, HybridModel)
    ids = _prompt(26, 5)
    got = g.score_ids(ids)
    q = lambda w: quantize(w.bfloat16().float(), Fmt.INT4).dequant().float()
    want = hybrid_reference.forward_logits(cfg, {k: v.bfloat16().float() for k, v in folded.items()}, ids, weight_fn=q)
    err = float((got - want).abs().max())
    assert err < 0.06 * float(want.abs().max()), (err, float(want.abs().max()))
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.9
    g.close()
    with pytest.raises(ValueError, match="neither a known"):
        ModelConfig.from_hf(dict(tc, layer_types=["agnes_delta_attention", "windowed_mixer", "x", "y"]))
    with pytest.raises(ValueError, match="DeltaNet geometry"):
        ModelConfig.from_hf({k: v for k, v in tc.items() if not k.startswith("linear_num")})
    (tmp_path / "broken").mkdir()
    (tmp_path / "broken" / "config.json").write_text((d / "config.json").read_text())
    save_file({k: v.bfloat16() for k, v in sd.items() if "layers.2.mlp.parallel_ffn.up_proj" not in k}, tmp_path / "broken" / "model.safetensors",
              {"format": "pt"})
    with pytest.raises(KeyError, match="parallel_ffn.up_proj"):
        Grimoire.load(_ec(tmp_path / "broken"), device="cpu")


def test_route_trace_file_lists_the_experts_in_order(hybrid_dirs, tmp_path, monkeypatch):
    """``GRIMOIRE_ROUTE_TRACE``: one record per MoE call -- layer, rows, top_k, kind -- followed by the routed expert ids."""
    import struct

    cfg, _, split_dir, _ = hybrid_dirs
    path = tmp_path / "routes.bin"
    monkeypatch.setenv("GRIMOIRE_ROUTE_TRACE", str(path))
    g = Grimoire.load(_ec(split_dir), device="cpu")
    ids = _prompt(9, 2)
    out, _ = g.generate(ids, 3)
    g.close()
    blob, at, recs = path.read_bytes(), 0, []
    while at < len(blob):
        layer, rows, k, kind = struct.unpack_from("<4i", blob, at)
        at += 16
        e = struct.unpack_from(f"<{rows * k}i", blob, at)
        at += 4 * rows * k
        recs.append((layer, rows, k, kind))
        assert k == cfg.num_experts_per_tok and all(0 <= v < cfg.num_experts for v in e)
    L = cfg.num_hidden_layers
    assert recs[:L] == [(l, 9, cfg.num_experts_per_tok, 1) for l in range(L)]               # the prompt, layer by layer
    assert recs[L:] == [(l, 1, cfg.num_experts_per_tok, 2) for _ in range(2) for l in range(L)]   # two decode steps after the first token
