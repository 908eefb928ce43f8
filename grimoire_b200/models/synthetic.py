"""Synthetic checkpoints: random-init weights under the HF tensor names the loaders resolve
(model.layers.N.self_attn.q_proj.weight ...), the same role as the reference's test fixture
writer tools/mini_model.hpp:18-110 ("random, never zero, weights for every architecture")."""
from __future__ import annotations

import torch

from .config import ModelConfig


def random_state_dict(cfg: ModelConfig, seed: int = 0, std: float = 0.02, device="cpu") -> dict[str, torch.Tensor]:
    """fp32 logical weights of a dense decoder, N(0, std) drawn from ``seed``."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    H, D = cfg.hidden_size, cfg.head_dim
    qrows = cfg.num_attention_heads * D * (2 if cfg.attn_output_gate else 1)

    def rnd(*shape):
        return torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * std

    norm_w = (lambda n: torch.zeros(n, device=device)) if cfg.norm_zero_centered else (lambda n: torch.ones(n, device=device))
    sd = {"model.embed_tokens.weight": rnd(cfg.vocab_size, H), "model.norm.weight": norm_w(H)}
    if not cfg.tie_word_embeddings:
        sd["lm_head.weight"] = rnd(cfg.vocab_size, H)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"] = norm_w(H)
        sd[p + "post_attention_layernorm.weight"] = norm_w(H)
        sd[p + "self_attn.q_proj.weight"] = rnd(qrows, H)
        sd[p + "self_attn.k_proj.weight"] = rnd(cfg.kv_size, H)
        sd[p + "self_attn.v_proj.weight"] = rnd(cfg.kv_size, H)
        sd[p + "self_attn.o_proj.weight"] = rnd(H, cfg.num_attention_heads * D)
        if cfg.qk_norm:
            sd[p + "self_attn.q_norm.weight"] = norm_w(D)
            sd[p + "self_attn.k_norm.weight"] = norm_w(D)
        sd[p + "mlp.gate_proj.weight"] = rnd(cfg.intermediate_size, H)
        sd[p + "mlp.up_proj.weight"] = rnd(cfg.intermediate_size, H)
        sd[p + "mlp.down_proj.weight"] = rnd(H, cfg.intermediate_size)
    return sd
