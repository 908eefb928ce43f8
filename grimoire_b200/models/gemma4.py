"""Sandwich-norm decoders on the dense engine path: the Gemma-4 text decoder and the Muse-Glimmer text decoder.

What differs from the Qwen3-style dense decoder (reference: ``forward_gemma4``, src/grimoire.cpp:14086-14270, config notes in
include/b70/qwen35.hpp:141-290, oracle ref/gemma4.py):

* the embedding lookup is multiplied by sqrt(hidden);
* two attention layer types: sliding-window layers with plain RoPE over the whole head, and global layers with
  "proportional" RoPE (frequencies base^(-2i / head_dim) for the first partial * head_dim / 2 pairs, the rest of the head
  unrotated, dimension d paired with d + head_dim / 2) -- expressed here as a head-wide inverse-frequency table with a zero
  tail, so the one RoPE / KV-write kernel serves both;
* q and k get a weighted per-head RMSNorm, v a weightless one; the softmax scale is 1.0; with ``attention_k_eq_v`` a global
  layer has no v_proj and takes its v from the k projection BEFORE norm and RoPE;
* sandwich norms: the attention output and the feed-forward output are normalised before they are added to the residual
  stream, and the feed-forward has its own input norm; GeGLU (tanh approximation); the stream is multiplied by a per-layer
  scalar at the end of the layer; the final logits are soft-capped.

The Muse-Glimmer decoder (``forward_muse``, src/grimoire.cpp:13867-14084) is the same sandwich layer with other switches:
the embedding row is RMS-normalised (no weight) before the first layer, q and k get a weightless per-head norm, sliding
layers use RoPE and the full layers no positional embedding at all, the attention output is multiplied by
sigmoid(gate_proj(normed layer input)), the feed-forward is SwiGLU, norms follow the (1 + w) convention and the softmax
scale carries the checkpoint's query prescale.  ``MuseModel`` is this class under that configuration.

Projections, RoPE + KV append, paged decode attention, prompt attention and the head are the engine's kernels; the pieces
only this family has (v norm, sandwich norms, GeGLU product, layer scalar, soft cap) are elementwise torch operations on the
device.  Served on one GPU with one head geometry for both layer types: checkpoints whose global layers have their own
head_dim / KV heads (the 31B model: 512 x 4 against 256 x 16) are refused by name, because the attention kernels stop at
head_dim 256.
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from ..formats.w4_tile_layout import concat_rows
from ..ops import core as K
from ..ops import ref
from ..ops.workspace import Workspace
from .config import ModelConfig
from .dense import DenseModel, RowBatch


@dataclass
class Gemma4Layer:
    in_norm: torch.Tensor
    post_attn_norm: torch.Tensor
    pre_ff_norm: torch.Tensor
    post_ff_norm: torch.Tensor
    qkv: object                 # q | k | v rows, or q | k when the layer takes v from k
    o: object
    gate_up: object             # [gate rows | up rows], plain epilogue (the GeGLU product follows)
    down: object
    q_norm: Optional[torch.Tensor]
    k_norm: Optional[torch.Tensor]
    scalar: float
    is_global: bool
    k_eq_v: bool
    gate: object = None         # attention output gate projection [Hq * D][H] (Muse)


def proportional_inv_freq(head_dim: int, theta: float, partial: float, factor: float = 1.0) -> torch.Tensor:
    """Head-wide inverse frequencies of proportional RoPE: head_dim / 2 entries, zeros past the rotated pairs."""
    n = int(partial * head_dim // 2)
    inv = torch.zeros(head_dim // 2, dtype=torch.float32)
    inv[:n] = 1.0 / (theta ** (torch.arange(0, 2 * n, 2, dtype=torch.float32) / head_dim))
    return inv / factor


def unsupported_gemma4(cfg: ModelConfig) -> Optional[str]:
    if (cfg.global_head_dim and cfg.global_head_dim != cfg.head_dim) or \
            (cfg.num_global_key_value_heads and cfg.num_global_key_value_heads != cfg.num_key_value_heads):
        return (f"this gemma4 checkpoint gives its global layers their own geometry (head_dim {cfg.global_head_dim}, "
                f"{cfg.num_global_key_value_heads} kv heads); the attention kernels serve one geometry up to head_dim 256")
    if not cfg.sliding_layers or len(cfg.sliding_layers) != cfg.num_hidden_layers:
        return "a gemma4 config must say for every layer whether it is sliding or global"
    return None


class Gemma4Model(DenseModel):
    def __init__(self, cfg: ModelConfig, device, workspace: Optional[Workspace] = None):
        why = unsupported_gemma4(cfg)
        if why:
            raise ValueError(why)
        super().__init__(cfg, device, workspace=workspace)
        D = cfg.head_dim
        # sliding layers: window, plain RoPE over the whole head (the base class's geometry); global layers: no window and
        # the proportional table
        self.geom_global = dataclasses.replace(self.geom, window=0, rot=D)
        theta_g = cfg.global_rope_theta or cfg.rope_theta
        # weightless q / k norm: a unit weight under the model's norm convention
        self.unit_norm = (torch.zeros(D) if cfg.norm_zero_centered else torch.ones(D)).to(self.device) if cfg.qk_norm_weightless else None
        if cfg.global_nope:
            self.inv_freq_global = torch.zeros(D // 2, device=self.device)      # angle 0 everywhere: the rotation is the identity
        elif cfg.global_rope_proportional:
            self.inv_freq_global = proportional_inv_freq(D, theta_g, cfg.global_partial_rotary, cfg.global_rope_factor).to(self.device)
        else:
            rot = int(D * cfg.global_partial_rotary) // 2 * 2
            self.geom_global = dataclasses.replace(self.geom_global, rot=rot)
            self.inv_freq_global = ref.rope_inv_freq(rot, theta_g).to(self.device)
        self.layers: list[Gemma4Layer] = []

    # ---- construction ----
    def add_gemma_layer(self, i: int, w: dict) -> None:
        """``w``: q, k, v (None on a k-eq-v layer), o, gate, up, down as fp32 ``[out][in]`` or stored QuantWeights; in_norm,
        post_attn_norm, pre_ff_norm, post_ff_norm, q_norm, k_norm vectors; scalar."""
        cfg, dev = self.cfg, self.device
        is_global = not cfg.sliding_layers[i]
        k_eq_v = w.get("v") is None
        if k_eq_v and not (cfg.k_eq_v and is_global):
            raise KeyError(f"layer {i} has no v_proj but the config does not make it a k-eq-v global layer")
        parts = [self._quant(w["q"]), self._quant(w["k"])] + ([] if k_eq_v else [self._quant(w["v"])])
        f32 = lambda t: None if t is None else t.to(device=dev, dtype=torch.float32).contiguous()
        sc = w.get("scalar")
        self.layers.append(Gemma4Layer(
            f32(w["in_norm"]), f32(w["post_attn_norm"]), f32(w["pre_ff_norm"]), f32(w["post_ff_norm"]),
            self._linear(concat_rows(parts), f"L{i}.qkv"), self._linear(self._quant(w["o"]), f"L{i}.o"),
            self._linear(concat_rows([self._quant(w["gate"]), self._quant(w["up"])]), f"L{i}.gate_up"),
            self._linear(self._quant(w["down"]), f"L{i}.down"),
            self.unit_norm if cfg.qk_norm_weightless else f32(w.get("q_norm")), self.unit_norm if cfg.qk_norm_weightless else f32(w.get("k_norm")),
            1.0 if sc is None else float(torch.as_tensor(sc).float().reshape(-1)[0]), is_global, k_eq_v,
            self._linear(self._quant(w["attn_gate"]), f"L{i}.attn_gate") if w.get("attn_gate") is not None else None))
        if cfg.attn_gate_proj and self.layers[-1].gate is None:
            raise KeyError(f"layer {i} has no attention gate projection (self_attn.gate_proj)")

    @classmethod
    def from_state_dict(cls, cfg: ModelConfig, sd: dict, device, workspace: Optional[Workspace] = None) -> "Gemma4Model":
        m = cls(cfg, device, workspace)
        pfx = "model.language_model." if any(k.startswith("model.language_model.") for k in sd) else "model."
        for i in range(cfg.num_hidden_layers):
            p = f"{pfx}layers.{i}."
            g = lambda k: sd.get(p + k)
            m.add_gemma_layer(i, dict(
                q=g("self_attn.q_proj.weight"), k=g("self_attn.k_proj.weight"), v=g("self_attn.v_proj.weight"),
                o=g("self_attn.o_proj.weight"), gate=g("mlp.gate_proj.weight"), up=g("mlp.up_proj.weight"), down=g("mlp.down_proj.weight"),
                in_norm=g("input_layernorm.weight"), post_attn_norm=g("post_attention_layernorm.weight"),
                pre_ff_norm=g("pre_feedforward_layernorm.weight"), post_ff_norm=g("post_feedforward_layernorm.weight"),
                q_norm=g("self_attn.q_norm.weight"), k_norm=g("self_attn.k_norm.weight"), scalar=g("layer_scalar"),
                attn_gate=g("self_attn.gate_proj.weight")))
        m.set_embeddings(sd[pfx + "embed_tokens.weight"], sd[pfx + "norm.weight"], sd.get("lm_head.weight"))
        return m

    @classmethod
    def from_checkpoint(cls, path, device, workspace: Optional[Workspace] = None) -> "Gemma4Model":
        """HF directory with the family's tensor names (src/qwen35_loader.cpp:1165-1240)."""
        from ..formats.checkpoint import Checkpoint

        ck = Checkpoint(path) if isinstance(path, (str, bytes)) or hasattr(path, "__fspath__") else path
        cfg = ck.cfg
        m = cls(cfg, device, workspace)
        for i in range(cfg.num_hidden_layers):
            p = f"{ck.prefix}layers.{i}."
            lin = lambda k: ck.linear(p + k)
            m.add_gemma_layer(i, dict(
                q=lin("self_attn.q_proj"), k=lin("self_attn.k_proj"), v=lin("self_attn.v_proj"), o=lin("self_attn.o_proj"),
                gate=lin("mlp.gate_proj"), up=lin("mlp.up_proj"), down=lin("mlp.down_proj"),
                in_norm=ck.plain(p + "input_layernorm.weight"), post_attn_norm=ck.plain(p + "post_attention_layernorm.weight"),
                pre_ff_norm=ck.plain(p + "pre_feedforward_layernorm.weight"), post_ff_norm=ck.plain(p + "post_feedforward_layernorm.weight"),
                q_norm=ck.plain(p + "self_attn.q_norm.weight"), k_norm=ck.plain(p + "self_attn.k_norm.weight"),
                scalar=ck.plain(p + "layer_scalar"), attn_gate=lin("self_attn.gate_proj") if cfg.attn_gate_proj else None))
        head = None if cfg.tie_word_embeddings else ck.linear("lm_head")
        m.set_embeddings(ck.embedding(), ck.plain(ck.prefix + "norm.weight"), head)
        return m

    @classmethod
    def random(cls, cfg: ModelConfig, device, seed: int = 0, **_kw) -> "Gemma4Model":
        from .synthetic import random_gemma4_state_dict

        return cls.from_state_dict(cfg, random_gemma4_state_dict(cfg, seed), device)

    def make_buffers(self, max_rows: int, max_logit_rows: int, dense_kv_tokens: int = 0):
        b = super().make_buffers(max_rows, max_logit_rows, dense_kv_tokens)
        b.gu = torch.zeros(max_rows, 2 * self.I, dtype=torch.bfloat16, device=self.device)       # gate | up before the GeGLU product
        return b

    def weight_bytes(self) -> int:
        n = self.lm_head.nbytes()
        for L in self.layers:
            n += L.qkv.nbytes() + L.o.nbytes() + L.gate_up.nbytes() + L.down.nbytes()
        return n

    # ---- forward ----
    def forward(self, rb: RowBatch, buf, kv_layers, block_table) -> torch.Tensor:
        cfg = self.cfg
        M = rb.tokens.shape[0]
        eps, off = cfg.rms_norm_eps, cfg.norm_offset
        h, x, part = buf.h[:M], buf.x[:M], buf.partial[:M]
        qkv, q, attn, act, gu = buf.qkv[:M], buf.q[:M], buf.attn[:M], buf.act[:M], buf.gu[:M]
        Hq, Hkv, D, I = self.Hq, self.Hkv, cfg.head_dim, self.I
        qw, kw = Hq * D, Hkv * D
        K.embed(rb.tokens, self.embed, h, cfg.embed_scale)
        if cfg.embed_norm:
            h.copy_(h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps))
        prefill = rb.mode == "prefill"
        if prefill and rb.segments is not None:
            raise NotImplementedError("several prompts in one pass are not built for this family")
        T = rb.q_pos0 + M
        for li, L in enumerate(self.layers):
            kvl = kv_layers[li]
            geom, inv = (self.geom_global, self.inv_freq_global) if L.is_global else (self.geom, self.inv_freq)
            K.add_rmsnorm(h, L.in_norm, x, eps, off)
            if L.k_eq_v:
                L.qkv(x, qkv[:, : qw + kw], "bf16")
                qkv[:, qw + kw:].copy_(qkv[:, qw: qw + kw])              # v is the k projection before norm and RoPE
            else:
                L.qkv(x, qkv, "bf16")
            if cfg.v_norm:
                v = qkv[:, qw + kw:].float().reshape(M, Hkv, D)
                qkv[:, qw + kw:].copy_((v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).reshape(M, kw).to(qkv.dtype))
            if prefill:
                if rb.q_pos0 > 0:
                    K.gather_kv_dense(kvl, block_table[rb.seq_slot], rb.q_pos0, buf.dense_k, buf.dense_v)
                K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, inv, geom, q, kvl, L.q_norm, L.k_norm, None,
                               buf.dense_k[rb.q_pos0: T], buf.dense_v[rb.q_pos0: T])
                K.flash_prefill(q, buf.dense_k, buf.dense_v, geom, attn, rb.q_pos0, None)
            else:
                K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, inv, geom, q, kvl, L.q_norm, L.k_norm, None)
                if not (rb.verify is not None and K.paged_verify_attn(q, rb.verify[0], rb.verify[1], block_table, kvl, geom, attn,
                                                                      rb.splits, self.ws, None)):
                    K.paged_decode_attn(q, rb.row_seq, rb.row_pos, block_table, kvl, geom, attn, rb.splits, self.ws, None)
            if L.gate is not None:                                        # output gate from the normed layer input (x is still it)
                L.gate(x, q, "bf16")
                attn.copy_((attn.float() * torch.sigmoid(q.float())).to(attn.dtype))
            # sandwich: the normalised attention output joins the stream
            L.o(attn, part, "f32")
            h.add_(ref.rmsnorm(part, L.post_attn_norm, eps, off))
            K.add_rmsnorm(h, L.pre_ff_norm, x, eps, off)
            L.gate_up(x, gu, "bf16")
            gate_act = F.gelu(gu[:, :I].float(), approximate="tanh") if cfg.geglu else F.silu(gu[:, :I].float())
            act.copy_((gate_act * gu[:, I:].float()).to(act.dtype))
            L.down(act, part, "f32")
            h.add_(ref.rmsnorm(part, L.post_ff_norm, eps, off))
            if L.scalar != 1.0:
                h.mul_(L.scalar)
            if self.tap_index:
                j = self.tap_index.get(li)
                if j is not None:
                    buf.taps[:M, j].copy_(h)
        if rb.logits_rows is None:
            hsel, n = h, M
        else:
            n = rb.logits_rows.shape[0]
            hsel = h.index_select(0, rb.logits_rows) if n != M else h
        logits = self._head(hsel, buf, n, rb)
        if cfg.logit_softcap > 0:
            logits.copy_(torch.tanh(logits / cfg.logit_softcap) * cfg.logit_softcap)
        return logits


class MuseModel(Gemma4Model):
    """Muse-Glimmer text decoder: the sandwich layer above under the Muse switches of the configuration."""
