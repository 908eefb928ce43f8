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


def random_hybrid_state_dict(cfg: ModelConfig, seed: int = 0, std: float = 0.02, fused_experts: bool = False,
                             mtp: bool = False) -> dict[str, torch.Tensor]:
    """fp32 logical weights of a hybrid (Gated DeltaNet + gated attention, MoE FFN) decoder under the tensor names the
    reference's loader resolves (src/qwen35_loader.cpp:1149-1169, :1320-1380): ``linear_attn.*`` with ``conv1d.weight``
    as [C][1][K], ``mlp.gate`` (router), ``mlp.shared_expert*`` and either per-expert ``mlp.experts.N.*_proj`` or the fused
    ``mlp.experts.gate_up_proj`` / ``down_proj``."""
    g = torch.Generator().manual_seed(seed)
    H, D = cfg.hidden_size, cfg.head_dim
    E, I, Is = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
    Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    C = 2 * Hk * Dk + Hv * Dv

    def rnd(*shape, scale=std):
        return torch.randn(*shape, generator=g, dtype=torch.float32) * scale

    nw = (lambda n: rnd(n, scale=0.05)) if cfg.norm_zero_centered else (lambda n: 1.0 + rnd(n, scale=0.05))
    sd = {"model.embed_tokens.weight": rnd(cfg.vocab_size, H), "model.norm.weight": nw(H)}
    if not cfg.tie_word_embeddings:
        sd["lm_head.weight"] = rnd(cfg.vocab_size, H)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = nw(H), nw(H)
        if cfg.is_attention_layer(i):
            a = p + "self_attn."
            sd[a + "q_proj.weight"] = rnd(cfg.q_size, H)
            sd[a + "k_proj.weight"], sd[a + "v_proj.weight"] = rnd(cfg.kv_size, H), rnd(cfg.kv_size, H)
            sd[a + "o_proj.weight"] = rnd(H, cfg.num_attention_heads * D)
            if cfg.qk_norm:
                sd[a + "q_norm.weight"], sd[a + "k_norm.weight"] = nw(D), nw(D)
        else:
            a = p + "linear_attn."
            sd[a + "in_proj_qkv.weight"], sd[a + "in_proj_z.weight"] = rnd(C, H), rnd(Hv * Dv, H)
            sd[a + "in_proj_a.weight"], sd[a + "in_proj_b.weight"] = rnd(Hv, H, scale=0.2), rnd(Hv, H, scale=0.2)
            sd[a + "conv1d.weight"] = rnd(C, 1, cfg.linear_conv_kernel_dim, scale=0.4)
            sd[a + "A_log"], sd[a + "dt_bias"] = rnd(Hv, scale=0.5), rnd(Hv, scale=0.5)
            sd[a + "norm.weight"] = 1.0 + rnd(Dv, scale=0.05)
            sd[a + "out_proj.weight"] = rnd(H, Hv * Dv)
        if cfg.attn_gate_proj and cfg.is_attention_layer(i):
            sd[p + "self_attn.gate_proj.weight"] = rnd(cfg.num_attention_heads * D, H)
        if cfg.mova_experts and cfg.layer_is_sparse(i) and cfg.is_attention_layer(i):
            # K2 sparse layer: the value projection is a routed bank of experts with its own sigmoid router
            sd.pop(p + "self_attn.v_proj.weight", None)
            sd[p + "self_attn.v_router.weight"] = rnd(cfg.mova_experts, H, scale=0.1)      # sigmoid scores: keep the logits off saturation
            sd[p + "self_attn.v_router.bias"] = rnd(cfg.mova_experts, scale=0.2)
            for e in range(cfg.mova_experts):
                sd[p + f"self_attn.v_experts.{e}.weight"] = rnd(cfg.kv_size, H, scale=0.1)
        m = p + "mlp."
        if not cfg.layer_is_sparse(i):             # dense FFN (the 27B hybrid; the mlp-only layers of an MoE model)
            sd[m + "gate_proj.weight"], sd[m + "up_proj.weight"] = rnd(cfg.intermediate_size, H), rnd(cfg.intermediate_size, H)
            sd[m + "down_proj.weight"] = rnd(H, cfg.intermediate_size)
            continue
        sd[m + "gate.weight"] = rnd(E, H, scale=0.1 if cfg.router_sigmoid else 0.5)
        if cfg.is_k2:
            sd[m + "gate.bias"] = rnd(E, scale=0.2)
            if Is:
                sd[m + "shared_experts.gate_proj.weight"], sd[m + "shared_experts.up_proj.weight"] = rnd(Is, H), rnd(Is, H)
                sd[m + "shared_experts.down_proj.weight"] = rnd(H, Is)
        elif Is:
            sd[m + "shared_expert_gate.weight"] = rnd(1, H, scale=0.5)
            sd[m + "shared_expert.gate_proj.weight"], sd[m + "shared_expert.up_proj.weight"] = rnd(Is, H), rnd(Is, H)
            sd[m + "shared_expert.down_proj.weight"] = rnd(H, Is)
        gu, dn = rnd(E, 2 * I, H), rnd(E, H, I)
        if fused_experts:
            sd[m + "experts.gate_up_proj"], sd[m + "experts.down_proj"] = gu, dn
        else:
            for e in range(E):
                x = m + f"experts.{e}."
                sd[x + "gate_proj.weight"], sd[x + "up_proj.weight"], sd[x + "down_proj.weight"] = gu[e, :I], gu[e, I:], dn[e]
    if mtp:
        sd.update(random_mtp_state_dict(cfg, seed, std))       # the draft layer: full attention + dense FFN under mtp.*
    return sd


def random_mtp_state_dict(cfg: ModelConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    """The dense family's one-layer multi-token-prediction head under its checkpoint names (``mtp.fc`` [H][2H], the three
    norms, ``mtp.layers.0.*``; src/grimoire.cpp:8603-8618)."""
    g = torch.Generator().manual_seed(seed + 4242)
    H, D = cfg.hidden_size, cfg.head_dim
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=torch.float32) * std
    nw = (lambda n: torch.zeros(n)) if cfg.norm_zero_centered else (lambda n: torch.ones(n))
    sd = {"mtp.fc.weight": rnd(H, 2 * H) + torch.cat([torch.eye(H), torch.eye(H)], dim=1) * 0.5,
          "mtp.pre_fc_norm_hidden.weight": nw(H), "mtp.pre_fc_norm_embedding.weight": nw(H), "mtp.norm.weight": nw(H)}
    p = "mtp.layers.0."
    sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = nw(H), nw(H)
    sd[p + "self_attn.q_proj.weight"] = rnd(cfg.q_size, H)
    sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"] = rnd(cfg.kv_size, H), rnd(cfg.kv_size, H)
    sd[p + "self_attn.o_proj.weight"] = rnd(H, cfg.num_attention_heads * D)
    if cfg.qk_norm:
        sd[p + "self_attn.q_norm.weight"], sd[p + "self_attn.k_norm.weight"] = nw(D), nw(D)
    sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = rnd(cfg.intermediate_size, H), rnd(cfg.intermediate_size, H)
    sd[p + "mlp.down_proj.weight"] = rnd(H, cfg.intermediate_size)
    return sd


def random_gemma4_state_dict(cfg: ModelConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    """fp32 logical weights of a sandwich-norm decoder (Gemma-4 or Muse-Glimmer style) under its checkpoint names (src/qwen35_loader.cpp:1172-1240): the four
    layer norms, q / k norms, ``layer_scalar``, no ``v_proj`` on global layers when the config sets attention_k_eq_v."""
    g = torch.Generator().manual_seed(seed)
    H, D, I = cfg.hidden_size, cfg.head_dim, cfg.intermediate_size
    rnd = lambda *shape, scale=std: torch.randn(*shape, generator=g, dtype=torch.float32) * scale
    nw = (lambda n: rnd(n, scale=0.05)) if cfg.norm_zero_centered else (lambda n: 1.0 + rnd(n, scale=0.05))
    sd = {"model.embed_tokens.weight": rnd(cfg.vocab_size, H), "model.norm.weight": nw(H)}
    if not cfg.tie_word_embeddings:
        sd["lm_head.weight"] = rnd(cfg.vocab_size, H)
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        for n in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            sd[p + n + ".weight"] = nw(H)
        a = p + "self_attn."
        sd[a + "q_proj.weight"], sd[a + "k_proj.weight"] = rnd(cfg.num_attention_heads * D, H), rnd(cfg.num_key_value_heads * D, H)
        if not (cfg.k_eq_v and not cfg.sliding_layers[i]):
            sd[a + "v_proj.weight"] = rnd(cfg.num_key_value_heads * D, H)
        sd[a + "o_proj.weight"] = rnd(H, cfg.num_attention_heads * D)
        # the softmax scale is 1.0 and q, k are normalised per head: norm weights near 1 would give scores of ~sqrt(D) and a
        # near one-hot, chaotic softmax; trained checkpoints keep them small, so the synthetic ones do too
        sd[a + "q_norm.weight"], sd[a + "k_norm.weight"] = 0.25 * (1.0 + rnd(D, scale=0.05)), 0.25 * (1.0 + rnd(D, scale=0.05))
        if cfg.attn_gate_proj:
            sd[a + "gate_proj.weight"] = rnd(cfg.num_attention_heads * D, H)
        sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"], sd[p + "mlp.down_proj.weight"] = rnd(I, H), rnd(I, H), rnd(H, I)
        if cfg.layer_scalar:
            sd[p + "layer_scalar"] = torch.tensor([1.0 + 0.1 * ((i % 3) - 1)])
    return sd


def random_qwen4_exp_state_dict(cfg: ModelConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    """fp32 logical weights of a Qwen4-Exp decoder under its checkpoint names (src/qwen35_loader.cpp:1060-1145): the hybrid
    family's blocks without any layernorm, two hyper-connections per layer and the tail mixer, an indexer on every attention
    layer and the n-gram embedding layers of ``ple_layer_ids`` (table sized by the prime layout of that layer's heads)."""
    from ..ref import qwen4_exp_ref as R

    sd = random_hybrid_state_dict(cfg, seed, std)
    for k in [k for k in sd if k.endswith("layernorm.weight") or k == "model.norm.weight"]:
        del sd[k]
    g = torch.Generator().manual_seed(seed + 9090)
    rnd = lambda *shape, scale=std: torch.randn(*shape, generator=g, dtype=torch.float32) * scale
    H, hc, low = cfg.hidden_size, cfg.hc_count, cfg.hc_lowrank
    wide = hc * H

    def connection(p: str, inject: bool):
        sd[p + "hc_norm.weight"] = rnd(wide, scale=0.05)
        sd[p + "input_mix_weight_down.weight"] = rnd(low, wide, scale=0.1)
        sd[p + "input_mix_weight_up.weight"] = rnd(wide, low, scale=0.3)
        if inject:
            sd[p + "block_inject_weight.weight"] = rnd(hc, wide, scale=0.1)

    ple_ids = sorted(set(cfg.ple_layer_ids))
    heads = (cfg.ngram_size - 1) * cfg.heads_per_ngram
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        connection(p + "attn_hyper_connection.", True)
        connection(p + "mlp_hyper_connection.", True)
        if cfg.is_attention_layer(i) and cfg.indexer_n_heads:
            ix, d = p + "self_attn.indexer.", cfg.indexer_head_dim
            sd[ix + "index_qk_proj.weight"] = rnd((cfg.indexer_n_heads + 1) * d, H, scale=0.3)
            sd[ix + "q_layernorm.weight"], sd[ix + "k_layernorm.weight"] = rnd(d, scale=0.05), rnd(d, scale=0.05)
        if (i + 1) in ple_ids:
            pl = p + "ple."
            _, _, total = R.ngram_vocab_layout(cfg.ngram_vocab_size_base, heads, ple_ids.index(i + 1))
            sd[pl + "ple_embedding.ngram_embedding.weight"] = rnd(total, cfg.ple_embed_dim // heads, scale=0.5)
            sd[pl + "key_proj.weight"], sd[pl + "value_proj.weight"] = rnd(wide, cfg.ple_embed_dim, scale=0.2), rnd(H, cfg.ple_embed_dim, scale=0.05)
            for k in ("norm_key", "norm_query", "norm_conv"):
                sd[pl + k + ".weight"] = rnd(wide, scale=0.05)
            sd[pl + "conv1d.weight"] = rnd(wide, 1, cfg.ple_conv_kernel_size, scale=0.3)
    connection("model.hyper_connection_mixer.", False)
    return sd
