"""Hybrid DeltaNet + MoE decoder on the GPU against its own CPU path (same weights), plus graph
replay == eager and batch invariance of a decode step."""
import pytest
import torch

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.models.config import FULL_ATTN, LINEAR_ATTN, ModelConfig
from grimoire_b200.models.hybrid import HybridModel
from grimoire_b200.ops import core as K

pytestmark = pytest.mark.gpu


def _cfg(kind: str = "moe"):
    lt = [LINEAR_ATTN, LINEAR_ATTN, LINEAR_ATTN, FULL_ATTN]
    if kind == "dense_ffn":       # the 27B-style hybrid: dense SwiGLU FFN, int4 projections
        return ModelConfig(model_type="qwen3_5", hidden_size=512, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                           head_dim=128, vocab_size=4096, intermediate_size=1024, partial_rotary_factor=0.5, attn_output_gate=True,
                           qk_norm=True, norm_zero_centered=True, layer_types=lt, linear_num_key_heads=2, linear_num_value_heads=4,
                           linear_key_head_dim=128, linear_value_head_dim=128, quant="int4")
    if kind == "plain_moe":       # Qwen3-MoE style: plain attention everywhere, no shared expert
        return ModelConfig(model_type="qwen3_moe", hidden_size=512, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                           head_dim=128, vocab_size=4096, intermediate_size=0, qk_norm=True, num_experts=16, num_experts_per_tok=4,
                           moe_intermediate_size=128, shared_expert_intermediate_size=0, quant="fp8_block")
    return ModelConfig(model_type="qwen3_next", hidden_size=512, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                       head_dim=128, vocab_size=4096, intermediate_size=0, partial_rotary_factor=0.5, attn_output_gate=True, qk_norm=True,
                       norm_zero_centered=True, layer_types=lt, linear_num_key_heads=2, linear_num_value_heads=4,
                       linear_key_head_dim=128, linear_value_head_dim=128, num_experts=16, num_experts_per_tok=4,
                       moe_intermediate_size=128, shared_expert_intermediate_size=128, quant="fp8_block")


LIM = dict(max_slots=3, max_ctx=256, prefill_chunk=64, max_decode_rows=8)


@pytest.mark.parametrize("kind", ["moe", "dense_ffn", "plain_moe"])
def test_hybrid_gpu_matches_cpu_path_and_graph_replay(kind):
    cfg = _cfg(kind)
    gpu = Engine(HybridModel.random(cfg, "cuda", seed=2, max_slots=3, gen_device="cpu"), EngineLimits(**LIM))
    cpu = Engine(HybridModel.random(cfg, "cpu", seed=2, max_slots=3), EngineLimits(**LIM))
    prompt = torch.randint(0, 4096, (90,), generator=torch.Generator().manual_seed(5)).tolist()
    sg, sc = gpu.open(), cpu.open()
    lg, lc = gpu.prefill(sg, prompt).float().cpu(), cpu.prefill(sc, prompt).float()
    scale = float(lc.abs().max())
    assert float((lg - lc).abs().max()) < 0.06 * max(scale, 1.0), (float((lg - lc).abs().max()), scale)
    tok = int(lc.argmax())
    for _ in range(4):
        pos = sc.length
        _, l2c = cpu.decode_rows([tok], [sc], [pos], return_logits=True)
        _, l2g = gpu.decode_rows([tok], [sg], [pos], use_graph=False, return_logits=True)
        assert float((l2g[0].float().cpu() - l2c[0]).abs().max()) < 0.06 * max(scale, 1.0)
        cpu.commit_rows([sc], [tok], [pos]); gpu.commit_rows([sg], [tok], [pos])
        tok = int(l2c[0].argmax())
    gpu.release(sg); cpu.release(sc)
    a = gpu.generate(prompt, 10, use_graph=False)
    b = gpu.generate(prompt, 10, use_graph=True)
    assert a == b
    assert K.status_read()[0] == 0


def test_k2_horizon_layers_on_gpu():
    """K2-Horizon layer mix on the GPU (grouped norms, routed value projection, softplus gate, sigmoid router with selection
    bias: csrc/kernels/k2_ops.cu) against the CPU path of the same weights.  The routers are random, so a near-tie may pick
    another expert on the two devices; the bound is therefore looser than for the other families (exactness against the fp32
    oracle is pinned on the CPU path, tests/test_load_paths.py), while graph replay must equal eager execution exactly."""
    cfg = ModelConfig(model_type="k2_horizon", hidden_size=512, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                      head_dim=128, vocab_size=4096, intermediate_size=1024, qk_norm=True, attn_gate_proj="softplus", num_experts=16,
                      num_experts_per_tok=4, moe_intermediate_size=128, shared_expert_intermediate_size=128, num_shared_experts=1,
                      norm_groups=2, router_sigmoid=True, router_scale=2.5, mova_experts=8, mova_top_k=2, mlp_only_layers=[0],
                      quant="fp8_block")
    gpu = Engine(HybridModel.random(cfg, "cuda", seed=14, max_slots=3), EngineLimits(**LIM))
    cpu = Engine(HybridModel.random(cfg, "cpu", seed=14, max_slots=3), EngineLimits(**LIM))
    assert [(L.moe is not None, L.mova is not None) for L in gpu.model.layers] == [(False, False), (True, True), (True, True)]
    prompt = torch.randint(0, 4096, (90,), generator=torch.Generator().manual_seed(5)).tolist()
    sg, sc = gpu.open(), cpu.open()
    lg, lc = gpu.prefill(sg, prompt).float().cpu(), cpu.prefill(sc, prompt).float()
    scale = max(1.0, float(lc.abs().max()))
    assert float((lg - lc).abs().max()) < 0.15 * scale, (float((lg - lc).abs().max()), scale)
    tok = int(lc.argmax())
    pos = sc.length
    _, l2c = cpu.decode_rows([tok], [sc], [pos], return_logits=True)
    _, l2g = gpu.decode_rows([tok], [sg], [pos], use_graph=False, return_logits=True)
    assert float((l2g[0].float().cpu() - l2c[0]).abs().max()) < 0.15 * scale
    gpu.release(sg); cpu.release(sc)
    assert gpu.generate(prompt, 8, use_graph=False) == gpu.generate(prompt, 8, use_graph=True)
    assert K.status_read()[0] == 0


@pytest.mark.parametrize("keep", [1, 2, 4])
def test_hybrid_verify_block_rollback_equals_sequential_gpu(keep):
    """A four-row verify block through the DeltaNet layers, rolled back to ``keep`` rows: the next single step must see the
    state that ``keep`` single steps leave (conv tail, delta-rule state and KV)."""
    cfg = _cfg()
    eng = Engine(HybridModel.random(cfg, "cuda", seed=4, max_slots=3), EngineLimits(**LIM))
    p = torch.randint(0, 4096, (41,), generator=torch.Generator().manual_seed(8)).tolist()
    s = eng.open()
    tok = int(eng.prefill(s, p).argmax())
    toks, logits = [tok], []
    for _ in range(5):
        nxt, lg = eng.decode_rows([toks[-1]], [s], [s.length], use_graph=False, return_logits=True)
        logits.append(lg[0].float().clone())
        eng.commit_rows([s], [toks[-1]], [s.length])
        toks.append(int(nxt[0]))
    eng.release(s)
    s = eng.open()
    assert int(eng.prefill(s, p).argmax()) == tok
    pos0 = s.length
    block = toks[:4]
    if keep < 4:
        block = block[:keep] + [(toks[keep] + 1) % 4096] + block[keep + 1:]
    nxt, lg = eng.decode_rows(block, [s] * 4, list(range(pos0, pos0 + 4)), use_graph=False, return_logits=True)
    scale = float(logits[0].abs().max())
    for i in range(keep):
        assert float((lg[i].float() - logits[i]).abs().max()) < 0.03 * scale
    eng.commit_rows([s] * keep, block[:keep], list(range(pos0, pos0 + keep)))
    eng.rollback(s, pos0 + keep)
    nxt2, lg2 = eng.decode_rows([toks[keep]], [s], [s.length], use_graph=False, return_logits=True)
    assert float((lg2[0].float() - logits[keep]).abs().max()) < 0.03 * scale
    eng.release(s)
    assert K.status_read()[0] == 0
