"""Loading synthetic HF checkpoints through the real reader: bf16 and GPTQ forms, sharded index,
name prefixes; the served tokens must equal a model built from the same tensors in memory."""
import json

import pytest
import torch

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.formats.checkpoint import Checkpoint
from grimoire_b200.formats.quantize import QuantWeight
from grimoire_b200.models.config import ModelConfig, tiny_dense
from grimoire_b200.models.dense import DenseModel
from tests.fixtures.mini_model import write_checkpoint

LIM = EngineLimits(max_slots=2, max_ctx=128, prefill_chunk=64, max_decode_rows=8)


def _prompt():
    return torch.randint(0, 4096, (12,), generator=torch.Generator().manual_seed(5)).tolist()


@pytest.mark.parametrize("quant,shards", [("bf16", 1), ("gptq", 1), ("gptq", 3)])
def test_checkpoint_roundtrip_serves_same_tokens(tmp_path, quant, shards):
    cfg = tiny_dense()
    cfg.tie_word_embeddings = False
    sd = write_checkpoint(tmp_path / "m", cfg, seed=2, quant=quant, shards=shards)
    ck = Checkpoint(tmp_path / "m")
    assert ck.cfg.hidden_size == 256 and ck.cfg.num_key_value_heads == 2 and ck.prefix == "model."
    lin = ck.linear("model.layers.0.self_attn.q_proj")
    if quant == "gptq":
        assert isinstance(lin, QuantWeight) and lin.group == 128      # group derived from the scales shape
    else:
        assert torch.equal(lin, sd["model.layers.0.self_attn.q_proj.weight"].bfloat16().float())
    a = Engine(DenseModel.from_checkpoint(tmp_path / "m", "cpu"), LIM).generate(_prompt(), 10)
    # the in-memory twin sees bf16-rounded weights in the bf16 case, the same int4 codes in the GPTQ case
    sd2 = {k: (v.bfloat16().float() if quant == "bf16" else v) for k, v in sd.items()}
    b = Engine(DenseModel.from_state_dict(cfg, sd2, "cpu"), LIM).generate(_prompt(), 10)
    assert a == b


def test_hf_config_parsing_nested_text_config_and_hybrid_fields():
    raw = {"text_config": {"model_type": "qwen3_next", "hidden_size": 2048, "num_hidden_layers": 4, "num_attention_heads": 16,
                           "num_key_value_heads": 2, "head_dim": 256, "vocab_size": 1000, "rms_norm_eps": 1e-6,
                           "rope_parameters": {"rope_theta": 5e6, "partial_rotary_factor": 0.25},
                           "layer_types": ["linear_attention", "linear_attention", "linear_attention", "full_attention"],
                           "linear_num_key_heads": 16, "linear_num_value_heads": 32, "linear_key_head_dim": 128,
                           "linear_value_head_dim": 128, "num_experts": 512, "num_experts_per_tok": 10,
                           "moe_intermediate_size": 512, "shared_expert_intermediate_size": 512}, "tie_word_embeddings": False}
    c = ModelConfig.from_hf(raw)
    assert c.rope_theta == 5e6 and c.rot_dim == 64 and c.attn_output_gate and c.norm_zero_centered
    assert c.num_attention_layers() == 1 and c.is_moe and c.linear_num_value_heads == 32


def test_int8_embedding_side_form_rounds_like_its_source_model(tmp_path):
    """``embed_tokens.weight`` as int8 codes with a per-row ``weight_scale``: the served row is bf16(code * bf16(scale))."""
    from safetensors.torch import save_file

    cfg = tiny_dense()
    write_checkpoint(tmp_path, cfg, seed=1)
    from safetensors.torch import load_file

    sd = load_file(tmp_path / "model.safetensors")
    emb = sd["model.embed_tokens.weight"].float()
    scale = (emb.abs().amax(dim=1) / 127).clamp_min(1e-8) * 1.0003            # not a bf16 number on purpose
    codes = torch.round(emb / scale[:, None]).clamp(-127, 127).to(torch.int8)
    sd["model.embed_tokens.weight"], sd["model.embed_tokens.weight_scale"] = codes, scale.float()
    save_file(sd, tmp_path / "model.safetensors", {"format": "pt"})
    got = Checkpoint(tmp_path).embedding()
    want = (codes.float() * scale.bfloat16().float()[:, None]).bfloat16().float()
    assert torch.equal(got, want) and not torch.equal(got, codes.float() * scale[:, None])
