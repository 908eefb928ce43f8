"""fp32 whole-model oracle of the hybrid family (Gated DeltaNet and / or full attention, gated or plain; MoE FFN with or
without a shared expert, or a dense FFN), written against the HF
tensor names: one sequence, all positions at once for attention, token by token for the recurrence.  It is the
host-side counterpart of the reference engine's model-matrix gate (tools/test_model_matrix.cpp) and of its per-family
forward (src/grimoire.cpp:15105-15453); ``HybridModel`` must agree with it up to its weight / KV quantisation."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..models.config import ModelConfig
from . import gdn_ref, k2_ref, moe_ref
from ..ops import ref


def _bf(t):
    return t.bfloat16().float()


def attention_delta(cfg: ModelConfig, sd: dict, p: str, x: torch.Tensor, pos, inv_freq, scale: float, wf, attend=None) -> torch.Tensor:
    """What the attention block of layer prefix ``p`` adds to the residual for the normed input rows ``x``.  ``attend``
    (q, k, v roped [T][heads][D]) -> [T][Hq][D] replaces the causal attention (sparse-attention families)."""
    bf, eps, off = _bf, cfg.rms_norm_eps, cfg.norm_offset
    D, Hq, Hkv, T = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, x.shape[0]
    a = p + "self_attn."
    if cfg.attn_output_gate:
        qg = (x @ wf(sd[a + "q_proj.weight"]).t()).reshape(T, Hq, 2 * D)
        q, gate = qg[..., :D], qg[..., D:].reshape(T, Hq * D)
    else:
        q, gate = (x @ wf(sd[a + "q_proj.weight"]).t()).reshape(T, Hq, D), None
    k = (x @ wf(sd[a + "k_proj.weight"]).t()).reshape(T, Hkv, D)
    if a + "v_router.weight" in sd:          # K2 sparse layer: routed value projection
        ex = torch.stack([wf(sd[a + f"v_experts.{e}.weight"]) for e in range(cfg.mova_experts)])
        v = k2_ref.mova_value(x, bf(sd[a + "v_router.weight"]), sd.get(a + "v_router.bias"), ex, cfg.mova_top_k).reshape(T, Hkv, D)
    else:
        v = (x @ wf(sd[a + "v_proj.weight"]).t()).reshape(T, Hkv, D)
    qn, kn = sd.get(a + "q_norm.weight"), sd.get(a + "k_norm.weight")
    q = ref.apply_rope(ref.head_rmsnorm(bf(q), None if qn is None else qn.float(), eps, off), pos, inv_freq, cfg.rot_dim)
    k = ref.apply_rope(ref.head_rmsnorm(bf(k), None if kn is None else kn.float(), eps, off), pos, inv_freq, cfg.rot_dim)
    if attend is None:
        o = ref.attention_rows(q, k, bf(v), pos, scale, cfg.sliding_window).reshape(T, Hq * D)
    else:
        o = attend(q, k, bf(v)).reshape(T, Hq * D)
    if gate is not None:
        o = o * torch.sigmoid(bf(gate))
    if cfg.attn_gate_proj == "softplus":     # K2: a separate gate projection of the normed layer input, softplus(beta = ln 2)
        o = k2_ref.softplus_gate(bf(o), bf(x @ wf(sd[a + "gate_proj.weight"]).t()))
    return bf(o) @ wf(sd[a + "o_proj.weight"]).t()


def gdn_delta(cfg: ModelConfig, sd: dict, p: str, x: torch.Tensor, wf) -> torch.Tensor:
    """What the Gated DeltaNet block of layer prefix ``p`` adds to the residual (one sequence from its first token)."""
    bf, eps, T = _bf, cfg.rms_norm_eps, x.shape[0]
    Hk, Hv, Dk, Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    a = p + "linear_attn."
    qkv = bf(x @ wf(sd[a + "in_proj_qkv.weight"]).t())
    z = bf(x @ wf(sd[a + "in_proj_z.weight"]).t()).reshape(T, Hv, Dv)
    ar = x @ bf(sd[a + "in_proj_a.weight"]).t()
    br = x @ bf(sd[a + "in_proj_b.weight"]).t()
    conv, _ = gdn_ref.conv4_silu(qkv, sd[a + "conv1d.weight"].float().reshape(qkv.shape[1], -1), torch.zeros(qkv.shape[1], 3))
    conv = bf(conv)
    qk, kk = Hk * Dk, 2 * Hk * Dk
    q = gdn_ref.l2norm(conv[:, :qk].reshape(T, Hk, Dk))
    k = gdn_ref.l2norm(conv[:, qk:kk].reshape(T, Hk, Dk))
    v = conv[:, kk:].reshape(T, Hv, Dv)
    al, be = gdn_ref.gates(ar, br, sd[a + "A_log"], sd[a + "dt_bias"])
    S = torch.zeros(Hv, Dv, Dk)
    o = gdn_ref.gdn_sequence(S, q, k, v, al, be)
    o = bf(gdn_ref.gated_rmsnorm(o, z, sd[a + "norm.weight"], eps)).reshape(T, Hv * Dv)
    return o @ wf(sd[a + "out_proj.weight"]).t()


def ffn_delta(cfg: ModelConfig, sd: dict, p: str, i: int, x: torch.Tensor, wf) -> torch.Tensor:
    """What the FFN of layer ``i`` (dense, MoE with or without a shared expert, or the K2 router) adds to the residual."""
    bf, T = _bf, x.shape[0]
    m = p + "mlp."
    if not cfg.layer_is_sparse(i):
        act = bf(F.silu(x @ wf(sd[m + "gate_proj.weight"]).t()) * (x @ wf(sd[m + "up_proj.weight"]).t()))
        return act @ wf(sd[m + "down_proj.weight"]).t()
    E, I = cfg.num_experts, cfg.moe_intermediate_size
    if m + "experts.gate_up_proj" in sd:
        gu, dn = sd[m + "experts.gate_up_proj"], sd[m + "experts.down_proj"]
        experts = [(wf(gu[e, :I]), wf(gu[e, I:]), wf(dn[e])) for e in range(E)]
    else:
        experts = [(wf(sd[f"{m}experts.{e}.gate_proj.weight"]), wf(sd[f"{m}experts.{e}.up_proj.weight"]),
                    wf(sd[f"{m}experts.{e}.down_proj.weight"])) for e in range(E)]
    if cfg.is_k2:
        # sigmoid router, bias on the selection only, normalised and scaled weights; ungated shared expert
        ids, w = k2_ref.router_topk(x.bfloat16().float() @ bf(sd[m + "gate.weight"]).t(), sd.get(m + "gate.bias"), cfg.num_experts_per_tok,
                                    cfg.router_sigmoid, cfg.norm_topk_prob, cfg.router_scale)
        y = torch.zeros(T, cfg.hidden_size)
        for t in range(T):
            for j in range(cfg.num_experts_per_tok):
                y[t] += w[t, j] * moe_ref.expert_ffn(x[t: t + 1], *experts[int(ids[t, j])])[0]
        if m + "shared_experts.gate_proj.weight" in sd:
            y += moe_ref.expert_ffn(x, wf(sd[m + "shared_experts.gate_proj.weight"]), wf(sd[m + "shared_experts.up_proj.weight"]),
                                    wf(sd[m + "shared_experts.down_proj.weight"]))
        return y
    shared = sgate = None
    if m + "shared_expert.gate_proj.weight" in sd:
        shared = (wf(sd[m + "shared_expert.gate_proj.weight"]), wf(sd[m + "shared_expert.up_proj.weight"]),
                  wf(sd[m + "shared_expert.down_proj.weight"]))
        sgate = bf(sd[m + "shared_expert_gate.weight"]) if m + "shared_expert_gate.weight" in sd else None
    y, _, _ = moe_ref.moe_forward(x, bf(sd[m + "gate.weight"]), experts, cfg.num_experts_per_tok, shared, sgate, cfg.norm_topk_prob)
    return y


def forward_logits(cfg: ModelConfig, sd: dict, tokens, weight_fn=None) -> torch.Tensor:
    """Logits [T][V] for ``tokens`` from the state dict ``sd`` (names as in models/synthetic.py).  ``weight_fn`` maps every
    projection matrix before use (pass a quantise-dequantise round trip to compare like with like)."""
    wf = weight_fn or (lambda w: w.float())
    pfx = "model.language_model." if any(k.startswith("model.language_model.") for k in sd) else "model."
    eps, off = cfg.rms_norm_eps, cfg.norm_offset
    T = len(tokens)
    pos = torch.arange(T)
    inv_freq = ref.rope_inv_freq(cfg.rot_dim, cfg.rope_theta)
    scale = cfg.softmax_scale or ref.softmax_scale(cfg.head_dim)
    h = sd[pfx + "embed_tokens.weight"].bfloat16().float()[torch.tensor(tokens, dtype=torch.long)]
    bf = _bf
    # K2: the variance of every RMSNorm over the residual is taken per contiguous group of the row
    rms = (lambda t, w: k2_ref.rmsnorm_grouped(t, w.float(), cfg.norm_groups, eps)) if cfg.norm_groups > 1 else \
          (lambda t, w: ref.rmsnorm(t, w.float(), eps, off))
    for i in range(cfg.num_hidden_layers):
        p = f"{pfx}layers.{i}."
        x = bf(rms(h, sd[p + "input_layernorm.weight"]))
        if cfg.is_attention_layer(i):
            h = h + attention_delta(cfg, sd, p, x, pos, inv_freq, scale, wf)
        else:
            h = h + gdn_delta(cfg, sd, p, x, wf)
        x = bf(rms(h, sd[p + "post_attention_layernorm.weight"]))
        h = h + ffn_delta(cfg, sd, p, i, x, wf)
    xf = bf(rms(h, sd[pfx + "norm.weight"]))
    head = sd.get("lm_head.weight", sd[pfx + "embed_tokens.weight"])
    return xf @ wf(head).t()
