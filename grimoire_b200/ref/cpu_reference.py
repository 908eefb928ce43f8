"""Independent fp32 oracle: a full-recompute dense decoder on dequantized weights.

No KV cache, no int8, no bf16 rounding, no fused kernels -- every token recomputes attention over
the whole prefix with plain softmax.  The engine's per-step logits are compared with this
(max abs error, arg-max agreement), the check the reference performs against fp32 dequantized
weights with ``--score-ids/--score-out`` (tools/grimoire_main.cpp:66-167)."""
from __future__ import annotations

import math

import torch

from ..formats.codecs import Fmt
from ..formats.quantize import quantize
from ..models.config import ModelConfig
from ..ops import ref

_QUANTIZED = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def dequantized_state_dict(cfg: ModelConfig, sd: dict[str, torch.Tensor], symmetric: bool = False) -> dict[str, torch.Tensor]:
    """Quantize every projection the engine quantizes (int4, cfg.quant_group) and dequantize it
    back, so the oracle sees exactly the weight values the engine runs with."""
    out = {}
    for name, w in sd.items():
        is_proj = any(name.endswith(f"{p}.weight") for p in _QUANTIZED) or (name == "lm_head.weight")
        if is_proj:
            out[name] = quantize(w, Fmt.INT4, group=cfg.quant_group, symmetric=symmetric).dequant()
        elif name == "model.embed_tokens.weight":
            out[name] = w.bfloat16().float()
        else:
            out[name] = w.float()
    return out


class ReferenceDecoder:
    def __init__(self, cfg: ModelConfig, sd: dict[str, torch.Tensor]):
        self.cfg, self.sd = cfg, sd
        self.inv_freq = ref.rope_inv_freq(cfg.rot_dim, cfg.rope_theta)

    def logits(self, tokens: list[int]) -> torch.Tensor:
        """fp32 logits [T][V] for every position of ``tokens``."""
        cfg, sd = self.cfg, self.sd
        T = len(tokens)
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        off, eps = cfg.norm_offset, cfg.rms_norm_eps
        pos = torch.arange(T)
        h = sd["model.embed_tokens.weight"][torch.tensor(tokens)].float()
        scale = cfg.softmax_scale or 1.0 / math.sqrt(D)
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            x = ref.rmsnorm(h, sd[p + "input_layernorm.weight"], eps, off)
            qg = (x @ sd[p + "self_attn.q_proj.weight"].t())
            if cfg.attn_output_gate:
                qg = qg.reshape(T, Hq, 2 * D)
                q, gate = qg[..., :D], qg[..., D:].reshape(T, Hq * D)
            else:
                q, gate = qg.reshape(T, Hq, D), None
            k = (x @ sd[p + "self_attn.k_proj.weight"].t()).reshape(T, Hkv, D)
            v = (x @ sd[p + "self_attn.v_proj.weight"].t()).reshape(T, Hkv, D)
            if cfg.qk_norm:
                q = ref.head_rmsnorm(q, sd[p + "self_attn.q_norm.weight"], eps, off)
                k = ref.head_rmsnorm(k, sd[p + "self_attn.k_norm.weight"], eps, off)
            q = ref.apply_rope(q, pos, self.inv_freq, cfg.rot_dim)
            k = ref.apply_rope(k, pos, self.inv_freq, cfg.rot_dim)
            a = ref.attention_rows(q, k, v, pos, scale, cfg.sliding_window).reshape(T, Hq * D)
            if gate is not None:
                a = a * torch.sigmoid(gate)
            h = h + a @ sd[p + "self_attn.o_proj.weight"].t()
            x = ref.rmsnorm(h, sd[p + "post_attention_layernorm.weight"], eps, off)
            g = x @ sd[p + "mlp.gate_proj.weight"].t()
            u = x @ sd[p + "mlp.up_proj.weight"].t()
            h = h + ref.swiglu(g, u) @ sd[p + "mlp.down_proj.weight"].t()
        x = ref.rmsnorm(h, sd["model.norm.weight"], eps, off)
        head = sd["model.embed_tokens.weight"] if cfg.tie_word_embeddings else sd["lm_head.weight"]
        return x @ head.t()

    def greedy(self, prompt: list[int], n: int):
        toks = list(prompt)
        out, trace = [], []
        for _ in range(n):
            lg = self.logits(toks)[-1]
            trace.append(lg)
            t = int(ref.argmax_lowest(lg[None])[0])
            out.append(t)
            toks.append(t)
        return out, trace
