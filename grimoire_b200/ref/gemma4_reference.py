"""fp32 whole-model oracle of the sandwich-norm decoders (Gemma-4 text, Muse-Glimmer text), written against the checkpoint's tensor names: one sequence, all
positions at once.  Host-side counterpart of the reference's per-family forward (src/grimoire.cpp:14086-14270) and of its
Python oracle (ref/gemma4.py); ``Gemma4Model`` must agree with it up to its weight / KV quantisation."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from ..models.config import ModelConfig


def _rms(x, w, eps, off=0.0):
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    return y if w is None else y * (off + w.float())


def _rope_full_head(x, pos, inv_freq):
    """x [T][heads][D]; inv_freq [D/2] (zeros leave their pair alone); dimension d pairs with d + D/2."""
    ang = pos.float()[:, None] * inv_freq[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    h = x.shape[-1] // 2
    a, b = x[..., :h], x[..., h:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def forward_logits(cfg: ModelConfig, sd: dict, tokens, weight_fn=None) -> torch.Tensor:
    wf = weight_fn or (lambda w: w.float())
    bf = lambda t: t.bfloat16().float()
    pfx = "model.language_model." if any(k.startswith("model.language_model.") for k in sd) else "model."
    H, D, Hq, Hkv, eps = cfg.hidden_size, cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.rms_norm_eps
    off = cfg.norm_offset
    T = len(tokens)
    pos = torch.arange(T)
    inv_local = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    theta_g = cfg.global_rope_theta or cfg.rope_theta
    n_rot = int(cfg.global_partial_rotary * D // 2)
    inv_global = torch.zeros(D // 2)
    inv_global[:n_rot] = 1.0 / (theta_g ** (torch.arange(0, 2 * n_rot, 2, dtype=torch.float32) / D))
    inv_global = torch.zeros(D // 2) if cfg.global_nope else inv_global / cfg.global_rope_factor
    h = bf(sd[pfx + "embed_tokens.weight"])[torch.tensor(tokens, dtype=torch.long)] * cfg.embed_scale
    if cfg.embed_norm:
        h = _rms(h, None, eps)
    for i in range(cfg.num_hidden_layers):
        p = f"{pfx}layers.{i}."
        a = p + "self_attn."
        sliding = cfg.sliding_layers[i]
        x = bf(_rms(h, sd[p + "input_layernorm.weight"], eps, off))
        q = bf(x @ wf(sd[a + "q_proj.weight"]).t()).reshape(T, Hq, D)
        k_raw = bf(x @ wf(sd[a + "k_proj.weight"]).t()).reshape(T, Hkv, D)
        v_raw = k_raw if a + "v_proj.weight" not in sd else bf(x @ wf(sd[a + "v_proj.weight"]).t()).reshape(T, Hkv, D)
        q = _rms(q, None if cfg.qk_norm_weightless else sd[a + "q_norm.weight"], eps, off)
        k = _rms(k_raw, None if cfg.qk_norm_weightless else sd[a + "k_norm.weight"], eps, off)
        v = bf(_rms(v_raw, None, eps)) if cfg.v_norm else v_raw
        inv = inv_local if sliding else inv_global
        q, k = bf(_rope_full_head(q, pos, inv)), _rope_full_head(k, pos, inv)
        scale = cfg.softmax_scale or 1.0 / math.sqrt(D)
        o = torch.zeros(T, Hq, D)
        for hq in range(Hq):
            g = hq // (Hq // Hkv)
            s = (q[:, hq] @ k[:, g].t()) * scale
            vis = pos[None, :] <= pos[:, None]
            if sliding and cfg.sliding_window > 0:
                vis &= pos[None, :] > pos[:, None] - cfg.sliding_window
            o[:, hq] = torch.softmax(s.masked_fill(~vis, float("-inf")), dim=-1) @ v[:, g]
        o = bf(o.reshape(T, Hq * D))
        if cfg.attn_gate_proj:
            o = bf(o * torch.sigmoid(bf(x @ wf(sd[a + "gate_proj.weight"]).t())))
        y = o @ wf(sd[a + "o_proj.weight"]).t()
        h = h + _rms(y, sd[p + "post_attention_layernorm.weight"], eps, off)
        x = bf(_rms(h, sd[p + "pre_feedforward_layernorm.weight"], eps, off))
        gate, up = bf(x @ wf(sd[p + "mlp.gate_proj.weight"]).t()), bf(x @ wf(sd[p + "mlp.up_proj.weight"]).t())
        y = bf((F.gelu(gate, approximate="tanh") if cfg.geglu else F.silu(gate)) * up) @ wf(sd[p + "mlp.down_proj.weight"]).t()
        h = h + _rms(y, sd[p + "post_feedforward_layernorm.weight"], eps, off)
        if p + "layer_scalar" in sd:
            h = h * float(sd[p + "layer_scalar"].reshape(-1)[0])
    xf = bf(_rms(h, sd[pfx + "norm.weight"], eps, off))
    head = sd.get("lm_head.weight")
    logits = xf @ (bf(sd[pfx + "embed_tokens.weight"]) if head is None or cfg.tie_word_embeddings else wf(head)).t()
    if cfg.logit_softcap > 0:
        logits = torch.tanh(logits / cfg.logit_softcap) * cfg.logit_softcap
    return logits
