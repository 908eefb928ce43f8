"""Gemma-4 text decoder (models/gemma4.py) against the fp32 oracle written from the checkpoint names
(ref/gemma4_reference.py): sandwich norms, GeGLU, sliding and global layers with their own RoPE (proportional on the global
ones), v taken from k on global layers, weightless v norm, scaling 1.0, embedding scale, layer scalars, logit soft cap;
greedy generation through the engine follows the model's own scores; the head geometry the kernels cannot serve is refused
by name.  Reference gate: tools/test_model_matrix.cpp, tools/test_gemma4_prefill.cpp."""
import dataclasses
import json

import pytest
import torch

from grimoire_b200.api import Grimoire, UnsupportedModel
from grimoire_b200.config import EngineConfig
from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.formats.safetensors_io import save_file
from grimoire_b200.models.config import ModelConfig, tiny_gemma4
from grimoire_b200.models.gemma4 import Gemma4Model, proportional_inv_freq
from grimoire_b200.models.synthetic import random_gemma4_state_dict
from grimoire_b200.ref import gemma4_reference


def _hf_config(cfg: ModelConfig) -> dict:
    return {"model_type": "gemma4_text", "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_hidden_layers,
            "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "vocab_size": cfg.vocab_size, "intermediate_size": cfg.intermediate_size, "rms_norm_eps": cfg.rms_norm_eps,
            "tie_word_embeddings": True, "sliding_window": cfg.sliding_window, "final_logit_softcapping": cfg.logit_softcap,
            "attention_k_eq_v": cfg.k_eq_v, "hidden_activation": "gelu_pytorch_tanh",
            "layer_types": ["sliding_attention" if s else "full_attention" for s in cfg.sliding_layers],
            "rope_parameters": {"sliding_attention": {"rope_type": "default", "rope_theta": cfg.rope_theta},
                                "full_attention": {"rope_type": "proportional", "rope_theta": cfg.global_rope_theta,
                                                   "partial_rotary_factor": cfg.global_partial_rotary}}}


def _write(path, cfg, seed=0):
    path.mkdir(parents=True, exist_ok=True)
    sd = random_gemma4_state_dict(cfg, seed)
    (path / "config.json").write_text(json.dumps(_hf_config(cfg)))
    save_file({k: v.bfloat16() for k, v in sd.items()}, path / "model.safetensors", {"format": "pt"})
    return sd


def _ec(model, **kw):
    base = dict(model=str(model), ctx=192, seq_slots=2, prefill_chunk=32, prefix_cache=0, mtp=0, copy_drafts=0)
    base.update(kw)
    return EngineConfig(**base)


def test_proportional_table_leaves_the_tail_unrotated():
    inv = proportional_inv_freq(64, 1e6, 0.25)
    assert inv.shape == (32,) and torch.all(inv[8:] == 0) and inv[0] == 1.0
    assert abs(float(inv[1]) - 1e6 ** (-2 / 64)) < 1e-7          # exponent over the WHOLE head, not over the rotated part


def test_hf_config_is_parsed_by_layer_type():
    cfg = ModelConfig.from_hf(_hf_config(tiny_gemma4()))
    want = tiny_gemma4()
    for f in ("sliding_layers", "sliding_window", "logit_softcap", "k_eq_v", "global_rope_theta", "global_partial_rotary",
              "global_rope_proportional", "embed_scale", "geglu", "sandwich_norms", "softmax_scale", "rope_theta"):
        assert getattr(cfg, f) == getattr(want, f), f
    assert cfg.is_gemma4 and cfg.norm_offset == 0.0


def test_checkpoint_matches_fp32_oracle_and_generation_follows_scores(tmp_path):
    cfg = tiny_gemma4()
    sd = _write(tmp_path / "g4", cfg, seed=4)
    g = Grimoire.load(_ec(tmp_path / "g4"), device="cpu")
    assert isinstance(g.model, Gemma4Model)
    assert [L.is_global for L in g.model.layers] == [False, False, False, True] and g.model.layers[3].k_eq_v
    ids = torch.randint(0, 4096, (45,), generator=torch.Generator().manual_seed(7)).tolist()       # longer than the window and the chunk
    got = g.score_ids(ids)
    q = lambda w: quantize(w.bfloat16().float(), Fmt.INT4).dequant().float()
    want = gemma4_reference.forward_logits(cfg, {k: v.bfloat16().float() for k, v in sd.items()}, ids, weight_fn=q)
    err = float((got - want).abs().max())
    assert err < 0.06 * float(want.abs().max()), (err, float(want.abs().max()))
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.9
    assert float(got.abs().max()) <= cfg.logit_softcap + 1e-3
    out, _ = g.generate(ids, 5)
    full = g.score_ids(ids + out)
    assert [int(full[len(ids) - 1 + j].argmax()) for j in range(5)] == out
    g.close()


def test_synthetic_preset_and_refusal_of_per_type_geometry(tmp_path):
    g = Grimoire.load(_ec("synthetic:tiny_gemma4"), device="cpu")
    assert isinstance(g.model, Gemma4Model) and len(g.generate(list(range(9, 30)), 4)[0]) == 4
    g.close()
    cfg = tiny_gemma4()
    hf = _hf_config(cfg)
    hf.update(global_head_dim=512, num_global_key_value_heads=1)
    d = tmp_path / "g4big"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(hf))
    with pytest.raises(UnsupportedModel, match="geometry"):
        Grimoire.load(_ec(d), device="cpu")


def _muse_hf_config(cfg: ModelConfig) -> dict:
    return {"model_type": "muse_glimmer", "text_config": {
        "model_type": "muse_glimmer_text", "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_hidden_layers,
        "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
        "vocab_size": cfg.vocab_size, "intermediate_size": cfg.intermediate_size, "rms_norm_eps": cfg.rms_norm_eps,
        "tie_word_embeddings": False, "sliding_window": cfg.sliding_window, "scale_query_by": 0.5, "rope_theta": cfg.rope_theta,
        "layer_types": ["sliding_attention" if s else "full_attention" for s in cfg.sliding_layers]}}


def test_muse_checkpoint_matches_fp32_oracle(tmp_path):
    """Muse-Glimmer switches of the sandwich decoder: normalised embeddings, weightless q / k norms, RoPE on the sliding
    layers only, sigmoid output gate projection, SwiGLU, (1 + w) norms, query prescale in the softmax scale."""
    from grimoire_b200.models.config import tiny_muse
    from grimoire_b200.models.gemma4 import MuseModel

    cfg = tiny_muse()
    path = tmp_path / "muse"
    path.mkdir()
    sd = random_gemma4_state_dict(cfg, 8)
    (path / "config.json").write_text(json.dumps(_muse_hf_config(cfg)))
    save_file({k: v.bfloat16() for k, v in sd.items()}, path / "model.safetensors", {"format": "pt"})
    parsed = ModelConfig.from_dir(path)
    for f in ("sliding_layers", "sliding_window", "softmax_scale", "embed_norm", "qk_norm_weightless", "global_nope", "attn_gate_proj",
              "norm_zero_centered", "geglu", "rope_theta", "tie_word_embeddings"):
        assert getattr(parsed, f) == getattr(cfg, f), f
    g = Grimoire.load(_ec(path), device="cpu")
    assert isinstance(g.model, MuseModel) and all(L.gate is not None for L in g.model.layers)
    assert float(g.model.inv_freq_global.abs().max()) == 0.0
    ids = torch.randint(0, 4096, (45,), generator=torch.Generator().manual_seed(7)).tolist()
    got = g.score_ids(ids)
    q = lambda w: quantize(w.bfloat16().float(), Fmt.INT4).dequant().float()
    want = gemma4_reference.forward_logits(cfg, {k: v.bfloat16().float() for k, v in sd.items()}, ids, weight_fn=q)
    err = float((got - want).abs().max())
    assert err < 0.06 * float(want.abs().max()), (err, float(want.abs().max()))
    assert float((got.argmax(-1) == want.argmax(-1)).float().mean()) >= 0.9
    out, _ = g.generate(ids, 5)
    full = g.score_ids(ids + out)
    assert [int(full[len(ids) - 1 + j].argmax()) for j in range(5)] == out
    g.close()
    g = Grimoire.load(_ec("synthetic:tiny_muse"), device="cpu")
    assert isinstance(g.model, MuseModel) and len(g.generate(list(range(9, 30)), 3)[0]) == 3
    g.close()


@pytest.mark.gpu
@pytest.mark.parametrize("family", ["gemma4", "muse"])
def test_gemma4_gpu_matches_cpu_path_and_graph_replay(family):
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import tiny_muse
    from grimoire_b200.models.gemma4 import MuseModel
    from grimoire_b200.ops import core as K

    if family == "muse":
        cfg = dataclasses.replace(tiny_muse(), hidden_size=512, head_dim=128, intermediate_size=1024, softmax_scale=0.5 / 128 ** 0.5)
        cls = MuseModel
    else:
        cfg = dataclasses.replace(tiny_gemma4(), hidden_size=512, head_dim=128, intermediate_size=1024, embed_scale=512 ** 0.5)
        cls = Gemma4Model
    sd = random_gemma4_state_dict(cfg, seed=2)
    lim = dict(max_slots=2, max_ctx=256, prefill_chunk=64, max_decode_rows=8)
    gpu = Engine(cls.from_state_dict(cfg, sd, "cuda"), EngineLimits(**lim))
    cpu = Engine(cls.from_state_dict(cfg, sd, "cpu"), EngineLimits(**lim))
    prompt = torch.randint(0, 4096, (90,), generator=torch.Generator().manual_seed(5)).tolist()
    sg, sc = gpu.open(), cpu.open()
    lg, lc = gpu.prefill(sg, prompt).float().cpu(), cpu.prefill(sc, prompt).float()
    scale = max(1.0, float(lc.abs().max()))
    assert float((lg - lc).abs().max()) < 0.06 * scale, float((lg - lc).abs().max())
    tok = int(lc.argmax())
    for _ in range(3):
        pos = sc.length
        _, l2c = cpu.decode_rows([tok], [sc], [pos], return_logits=True)
        _, l2g = gpu.decode_rows([tok], [sg], [pos], use_graph=False, return_logits=True)
        assert float((l2g[0].float().cpu() - l2c[0]).abs().max()) < 0.06 * scale
        cpu.commit_rows([sc], [tok], [pos]); gpu.commit_rows([sg], [tok], [pos])
        tok = int(l2c[0].argmax())
    gpu.release(sg); cpu.release(sc)
    assert gpu.generate(prompt, 8, use_graph=False) == gpu.generate(prompt, 8, use_graph=True)
    assert K.status_read()[0] == 0


def test_gemma4_gguf_file_loads_and_matches_the_safetensors_load(tmp_path):
    """The family's GGUF adapter: ``gemma4.*`` metadata (per-type key lengths and RoPE bases, per-layer kv heads and sliding
    pattern, ``rope_freqs.weight`` marking the rotated pairs) and the converter's tensor names; same logits as the HF load."""
    from grimoire_b200.formats import gguf as G

    from .test_gguf import _write_gguf

    cfg = tiny_gemma4()
    sd = _write(tmp_path / "hf", cfg, seed=6)
    L, D = cfg.num_hidden_layers, cfg.head_dim
    names = {"input_layernorm": "attn_norm", "post_attention_layernorm": "post_attention_norm", "pre_feedforward_layernorm": "ffn_norm",
             "post_feedforward_layernorm": "post_ffw_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k",
             "self_attn.v_proj": "attn_v", "self_attn.o_proj": "attn_output", "self_attn.q_norm": "attn_q_norm",
             "self_attn.k_norm": "attn_k_norm", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up", "mlp.down_proj": "ffn_down"}
    tensors = {}
    f32 = lambda name, t: tensors.__setitem__(name, (0, tuple(reversed(t.shape)), t.bfloat16().float().contiguous().numpy().tobytes()))
    f32("token_embd.weight", sd["model.embed_tokens.weight"])
    f32("output_norm.weight", sd["model.norm.weight"])
    rot = int(cfg.global_partial_rotary * D // 2)
    f32("rope_freqs.weight", torch.cat([torch.ones(rot), torch.full((D // 2 - rot,), 1e30)]))
    for i in range(L):
        for hf, gg in names.items():
            t = sd.get(f"model.layers.{i}.{hf}.weight")
            if t is not None:
                f32(f"blk.{i}.{gg}.weight", t)
        f32(f"blk.{i}.layer_output_scale.weight", sd[f"model.layers.{i}.layer_scalar"])
    toks = [chr(0x100 + i) for i in range(cfg.vocab_size)]
    kv = {"general.architecture": (8, "gemma4"), "gemma4.block_count": (4, L), "gemma4.embedding_length": (4, cfg.hidden_size),
          "gemma4.feed_forward_length": (4, cfg.intermediate_size), "gemma4.attention.head_count": (4, cfg.num_attention_heads),
          "gemma4.attention.key_length": (4, D), "gemma4.attention.key_length_swa": (4, D), "gemma4.attention.value_length": (4, D),
          "gemma4.attention.value_length_swa": (4, D), "gemma4.rope.dimension_count": (4, D), "gemma4.rope.dimension_count_swa": (4, D),
          "gemma4.attention.sliding_window": (4, cfg.sliding_window), "gemma4.attention.shared_kv_layers": (4, 0),
          "gemma4.embedding_length_per_layer_input": (4, 0), "gemma4.context_length": (4, 8192),
          "gemma4.rope.freq_base": (6, cfg.global_rope_theta), "gemma4.rope.freq_base_swa": (6, cfg.rope_theta),
          "gemma4.attention.layer_norm_rms_epsilon": (6, cfg.rms_norm_eps), "gemma4.final_logit_softcapping": (6, cfg.logit_softcap),
          "gemma4.attention.head_count_kv": (9, (4, [cfg.num_key_value_heads] * L)),
          "gemma4.attention.sliding_window_pattern": (9, (4, [1 if s else 0 for s in cfg.sliding_layers])),
          "tokenizer.ggml.model": (8, "gpt2"), "tokenizer.ggml.tokens": (9, (8, toks)), "tokenizer.ggml.merges": (9, (8, [])),
          "tokenizer.ggml.token_type": (9, (5, [1] * cfg.vocab_size))}
    path = tmp_path / "g4.gguf"
    _write_gguf(path, kv, tensors)
    gf = G.GGUFFile(path)
    got = G.config_from_gguf(gf)
    for f in ("sliding_layers", "sliding_window", "logit_softcap", "k_eq_v", "global_rope_theta", "global_partial_rotary", "rope_theta",
              "head_dim", "num_key_value_heads", "global_head_dim", "embed_scale"):
        assert getattr(got, f) == pytest.approx(getattr(cfg, f)) if isinstance(getattr(cfg, f), float) else getattr(got, f) == getattr(cfg, f), f
    gf.close()
    ids = torch.randint(0, 4096, (30,), generator=torch.Generator().manual_seed(3)).tolist()
    a = Grimoire.load(_ec(path), device="cpu")
    b = Grimoire.load(_ec(tmp_path / "hf"), device="cpu")
    assert isinstance(a.model, Gemma4Model)
    la, lb = a.score_ids(ids), b.score_ids(ids)
    assert torch.allclose(la, lb, atol=1e-4), float((la - lb).abs().max())
    a.close(), b.close()
