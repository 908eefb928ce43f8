"""Model description: one dataclass for every architecture the engine runs, plus the named
configurations the benchmarks use.

Field names follow the HF ``config.json`` keys the reference parses into ``Qwen35Config``
(include/b70/qwen35.hpp:70-294, src/qwen35_loader.cpp:330-640): dense attention decoders
(Qwen3-style), Gated-DeltaNet hybrids (3 linear-attention layers : 1 gated full-attention layer),
MoE FFNs with an optional shared expert, and an optional MTP draft head.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Optional

FULL_ATTN = "full_attention"
LINEAR_ATTN = "linear_attention"


@dataclass
class ModelConfig:
    model_type: str = "qwen3"
    hidden_size: int = 256
    num_hidden_layers: int = 2
    num_attention_heads: int = 4
    num_key_value_heads: int = 2
    head_dim: int = 64
    vocab_size: int = 4096
    intermediate_size: int = 768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    partial_rotary_factor: float = 1.0
    tie_word_embeddings: bool = False
    attn_output_gate: bool = False          # q_proj emits [q | gate] per head
    qk_norm: bool = False                   # per-head RMSNorm of q and k before RoPE
    norm_zero_centered: bool = False        # (1 + w) convention of the Qwen3.5 family
    sliding_window: int = 0
    attention_bias: bool = False
    softmax_scale: Optional[float] = None
    layer_types: list[str] = field(default_factory=list)
    # Gated DeltaNet
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    gdn_chunk: int = 64
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    norm_topk_prob: bool = True
    # Gemma-4 family (sandwich norms, GeGLU, two attention layer types with their own RoPE)
    embed_scale: float = 1.0                # embeddings are multiplied by this on lookup (sqrt(hidden))
    logit_softcap: float = 0.0              # final logits = cap * tanh(logits / cap) (0: none)
    geglu: bool = False                     # gelu_tanh(gate) * up instead of silu(gate) * up
    sandwich_norms: bool = False            # post-attention / pre- and post-feed-forward norms around the residual adds
    layer_scalar: bool = False              # hidden *= layer_scalar at the end of every layer
    v_norm: bool = False                    # weightless per-head RMSNorm of v
    k_eq_v: bool = False                    # global layers have no v_proj: v is the k projection before its norm and RoPE
    sliding_layers: list[bool] = field(default_factory=list)     # per layer: sliding-window attention (others are global)
    global_rope_theta: float = 0.0          # RoPE of the global layers (0: same as the sliding layers)
    global_partial_rotary: float = 1.0
    global_rope_factor: float = 1.0
    global_rope_proportional: bool = False  # frequencies over the whole head, the tail left unrotated, pairs d <-> d + D/2
    global_head_dim: int = 0                # global layers' own head_dim / kv heads (0: same as the sliding layers)
    num_global_key_value_heads: int = 0
    # Muse-Glimmer family (the sandwich layer of above with these switches)
    embed_norm: bool = False                # weightless RMSNorm of the embedding row before the first layer
    qk_norm_weightless: bool = False        # q / k per-head RMSNorm without a learned weight
    global_nope: bool = False               # global layers apply no rotary embedding at all
    attn_gate_proj: str = ""                # "sigmoid": attention output *= sigmoid(gate_proj(normed layer input))
    # K2-Horizon family (a Qwen3-MoE with grouped norms, a softplus attention gate, a sigmoid router and a routed value projection)
    norm_groups: int = 1                    # RMSNorm variance per contiguous group of the row
    router_sigmoid: bool = False            # sigmoid scores; a router bias steers the selection only
    router_scale: float = 1.0               # routed weights are multiplied by this after normalisation
    num_shared_experts: int = 0             # ungated shared expert of width moe_intermediate_size * this
    mova_experts: int = 0                   # sparse layers replace v_proj by a routed bank of value experts
    mova_top_k: int = 0
    mlp_only_layers: list[int] = field(default_factory=list)     # layers with a dense FFN in an MoE model
    decoder_sparse_step: int = 1            # layer i is sparse when (i + 1) % step == 0 and it is not mlp-only
    parallel_ffn_intermediate_size: int = 0      # Agnes: width of the second SwiGLU of every mlp, folded into the first at load (intermediate_size counts it)
    # Qwen4-Exp family (the hybrid decoder under a multi-stream residual, sparse attention and per-layer n-gram embeddings)
    hc_count: int = 0                       # residual streams (0: a plain residual)
    hc_lowrank: int = 0                     # width of the mix's low-rank gate
    ple_layer_ids: list[int] = field(default_factory=list)       # 1-based layers that add the n-gram embedding before their block
    ple_embed_dim: int = 0
    ple_conv_kernel_size: int = 4
    ngram_size: int = 3
    heads_per_ngram: int = 8
    ngram_vocab_size_base: int = 0
    ngram_seed: int = 1234
    eos_token_id: int = 0
    indexer_n_heads: int = 0                # sparse attention: indexer heads (0: dense attention)
    indexer_head_dim: int = 0
    indexer_budget: int = 0                 # tokens a query attends to (plus the block still being filled)
    indexer_compress_ratio: int = 0         # tokens per pooled key block
    # MTP draft head
    mtp_num_hidden_layers: int = 0
    # quantization of the projections in a synthetic / converted model
    quant: str = "int4"
    quant_group: int = 128

    def __post_init__(self):
        if not self.layer_types:
            self.layer_types = [FULL_ATTN] * self.num_hidden_layers
        if len(self.layer_types) != self.num_hidden_layers:
            raise ValueError("layer_types length must equal num_hidden_layers")

    # ---- derived ----
    @property
    def rot_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def norm_offset(self) -> float:
        return 1.0 if self.norm_zero_centered else 0.0

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim * (2 if self.attn_output_gate else 1)

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def is_gemma4(self) -> bool:
        return self.model_type.startswith("gemma4")

    @property
    def is_agnes(self) -> bool:
        return self.model_type.startswith("agnes")

    @property
    def is_qwen4_exp(self) -> bool:
        return self.hc_count > 1

    @property
    def is_k2(self) -> bool:
        return "k2_horizon" in self.model_type

    def layer_is_sparse(self, i: int) -> bool:
        """MoE FFN (and, for K2, the routed value projection) on layer i; dense FFN otherwise."""
        if not self.is_moe or i in self.mlp_only_layers or self.decoder_sparse_step <= 0:
            return False
        return (i + 1) % self.decoder_sparse_step == 0

    @property
    def is_muse(self) -> bool:
        return "muse_glimmer" in self.model_type

    @property
    def is_sandwich(self) -> bool:
        """Served by the sandwich-norm decoder class (models/gemma4.py)."""
        return self.is_gemma4 or self.is_muse

    def is_attention_layer(self, i: int) -> bool:
        return self.layer_types[i] == FULL_ATTN

    def num_attention_layers(self) -> int:
        return sum(1 for t in self.layer_types if t == FULL_ATTN)

    def param_count(self) -> int:
        H = self.hidden_size
        n = self.vocab_size * H * (1 if self.tie_word_embeddings else 2)
        for i in range(self.num_hidden_layers):
            if self.is_attention_layer(i):
                n += H * (self.q_size + 2 * self.kv_size) + self.num_attention_heads * self.head_dim * H
            else:
                kd = self.linear_num_key_heads * self.linear_key_head_dim
                vd = self.linear_num_value_heads * self.linear_value_head_dim
                n += H * (2 * kd + vd) + H * vd + 2 * H * self.linear_num_value_heads + vd * H
            if self.is_moe:
                n += self.num_experts * 3 * H * self.moe_intermediate_size + H * self.num_experts
                n += 3 * H * self.shared_expert_intermediate_size
            else:
                n += 3 * H * self.intermediate_size
        return n

    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @staticmethod
    def from_hf(cfg: dict) -> "ModelConfig":
        """Build from a HF ``config.json`` dict (nested ``text_config`` handled like
        src/qwen35_loader.cpp:271-316)."""
        if "text_config" in cfg and isinstance(cfg["text_config"], dict):
            inner = dict(cfg["text_config"])
            for k in ("tie_word_embeddings",):
                if k in cfg and k not in inner:
                    inner[k] = cfg[k]
            cfg = inner
        mt = cfg.get("model_type", "qwen3")
        rp = cfg.get("rope_parameters") or cfg.get("rope_scaling") or {}
        n_layers = int(cfg["num_hidden_layers"])
        heads = int(cfg["num_attention_heads"])
        hd = int(cfg.get("head_dim") or cfg["hidden_size"] // heads)
        raw_types = list(cfg.get("layer_types") or [])

        def kind(i: int, t: str) -> str:
            # listed names only: an unknown spelling that fell through to full attention would load, generate fluent text
            # and not be the model (src/qwen35_loader.cpp:800-858)
            if t in ("linear_attention", "linear") or "delta" in t:
                return LINEAR_ATTN
            if t in ("full_attention", "sliding_attention", "attention", "qsa_attention", "qwen_sparse_attention") or "global" in t:
                return FULL_ATTN
            raise ValueError(f"config.json layer_types[{i}] is {t!r}, which is neither a known linear nor a known full attention layer")

        lt = [kind(i, str(t)) for i, t in enumerate(raw_types)] if not (mt.startswith("gemma4") or "muse_glimmer" in mt) else raw_types
        family35 = mt.startswith("qwen3_5") or mt.startswith("qwen3_next") or mt.startswith("qwen3.5")
        if mt.startswith("gemma4"):
            return ModelConfig._gemma4_from_hf(cfg, mt, n_layers, heads, hd)
        if "muse_glimmer" in mt:
            return ModelConfig._muse_from_hf(cfg, mt, n_layers, heads, hd)
        if "k2_horizon" in mt:
            return ModelConfig._k2_from_hf(cfg, mt, n_layers, heads, hd)
        q4 = {}
        if mt.startswith("agnes"):
            # Agnes: the 3.5-style hybrid under other names, with a second narrow SwiGLU inside every mlp that the loader
            # folds into the main one (src/qwen35_loader.cpp:571-600, :749-777); its DeltaNet geometry must be present
            family35 = True
            q4 = dict(parallel_ffn_intermediate_size=int(cfg.get("parallel_ffn_intermediate_size", 0)))
            if int(cfg.get("linear_num_key_heads", 0)) <= 0 or int(cfg.get("linear_num_value_heads", 0)) <= 0:
                raise ValueError("Agnes: no gated-DeltaNet geometry in the config")
        if "qwen4_exp" in mt:
            q4 = ModelConfig._qwen4_exp_fields(cfg)
            lt = [LINEAR_ATTN if t == LINEAR_ATTN else FULL_ATTN for t in lt]     # "qsa_attention" layers are full-attention layers
            family35 = True
        return ModelConfig(
            **q4,
            model_type=mt,
            hidden_size=int(cfg["hidden_size"]), num_hidden_layers=n_layers, num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads", heads)), head_dim=hd,
            vocab_size=int(cfg["vocab_size"]),
            # Agnes: the served FFN is the main SwiGLU with the parallel one folded in, so its width is the sum
            intermediate_size=int(cfg.get("intermediate_size", 0)) + q4.get("parallel_ffn_intermediate_size", 0),
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
            rope_theta=float(rp.get("rope_theta", cfg.get("rope_theta", 1e6))),
            partial_rotary_factor=float(rp.get("partial_rotary_factor", cfg.get("partial_rotary_factor", 1.0))),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            attn_output_gate=bool(cfg.get("attn_output_gate", family35)),
            qk_norm=bool(cfg.get("qk_norm", mt.startswith("qwen3"))),
            norm_zero_centered=bool(cfg.get("norm_zero_centered", family35)),
            sliding_window=int(cfg.get("sliding_window") or 0),
            attention_bias=bool(cfg.get("attention_bias", False)),
            layer_types=lt,
            linear_num_key_heads=int(cfg.get("linear_num_key_heads", 0)),
            linear_num_value_heads=int(cfg.get("linear_num_value_heads", 0)),
            linear_key_head_dim=int(cfg.get("linear_key_head_dim", 0)),
            linear_value_head_dim=int(cfg.get("linear_value_head_dim", 0)),
            linear_conv_kernel_dim=int(cfg.get("linear_conv_kernel_dim", 4)),
            num_experts=int(cfg.get("num_experts", 0)), num_experts_per_tok=int(cfg.get("num_experts_per_tok", 0)),
            moe_intermediate_size=int(cfg.get("moe_intermediate_size", 0)),
            shared_expert_intermediate_size=int(cfg.get("shared_expert_intermediate_size", 0)),
            norm_topk_prob=bool(cfg.get("norm_topk_prob", True)),
            mtp_num_hidden_layers=int(cfg.get("mtp_num_hidden_layers", 0)),
            # Qwen3-MoE: dense FFN on the listed layers and on the layers off the sparse step
            mlp_only_layers=[int(v) for v in (cfg.get("mlp_only_layers") or [])],
            decoder_sparse_step=int(cfg.get("decoder_sparse_step", 1) or 1),
        )

    @staticmethod
    def _qwen4_exp_fields(cfg: dict) -> dict:
        """The family's own keys (src/qwen35_loader.cpp:617-660; defaults of ref/qwen4_exp_config.py:41-49).  The five indexer keys
        come together or not at all; ``ple_layer_ids`` are 1-based; a sigmoid DeltaNet output gate is not served."""
        idx = {k: int(cfg.get(k) or 0) for k in ("indexer_n_heads", "indexer_kv_heads", "indexer_head_dim", "indexer_budget",
                                                  "indexer_compress_ratio")}
        if any(idx.values()):
            if not all(idx.values()):
                raise ValueError("qwen4_exp: the five indexer_* keys must be given together: " + ", ".join(k for k, v in idx.items() if not v))
            if idx["indexer_kv_heads"] != 1 or idx["indexer_budget"] % idx["indexer_compress_ratio"]:
                raise ValueError("qwen4_exp: the indexer needs one key head and a budget that is a multiple of the compression ratio")
        if cfg.get("output_gate_type") == "sigmoid":
            raise ValueError("qwen4_exp: a sigmoid DeltaNet output gate is not served")
        eos = cfg.get("eos_token_id", 0)
        eos = eos[0] if isinstance(eos, (list, tuple)) else eos
        n = int(cfg["num_hidden_layers"])
        ple = sorted({int(v) for v in (cfg.get("ple_layer_ids") or [])})
        if any(v < 1 or v > n for v in ple):
            raise ValueError("qwen4_exp: ple_layer_ids are 1-based and must name existing layers")
        hc = int(cfg.get("hc_count", 4))
        if hc <= 1:
            raise ValueError("qwen4_exp: hc_count must be above 1")
        return dict(hc_count=hc, hc_lowrank=int(cfg.get("hc_lowrank", 320)), ple_layer_ids=ple,
                    ple_embed_dim=int(cfg.get("ple_embed_dim") or cfg["hidden_size"]),
                    ple_conv_kernel_size=int(cfg.get("ple_conv_kernel_size", 4)), ngram_size=int(cfg.get("ngram_size", 3)),
                    heads_per_ngram=int(cfg.get("heads_per_ngram", 8)), ngram_vocab_size_base=int(cfg.get("ngram_vocab_size_base", 20_000_000)),
                    ngram_seed=int(cfg.get("seed", 1234)), eos_token_id=int(eos or 0), indexer_n_heads=idx["indexer_n_heads"],
                    indexer_head_dim=idx["indexer_head_dim"], indexer_budget=idx["indexer_budget"],
                    indexer_compress_ratio=idx["indexer_compress_ratio"])

    @staticmethod
    def _gemma4_from_hf(cfg: dict, mt: str, n_layers: int, heads: int, hd: int) -> "ModelConfig":
        """Gemma-4 text config (src/qwen35_loader.cpp:360-480): ``layer_types`` of sliding_attention / full_attention,
        ``rope_parameters`` keyed BY LAYER TYPE (sliding: plain RoPE; full: proportional RoPE with a partial factor),
        scaling 1.0, sqrt(hidden) embedding scale, GeGLU, sandwich norms, per-layer scalar, final logit soft cap."""
        lt = list(cfg.get("layer_types") or [])
        if len(lt) != n_layers:
            raise ValueError("a gemma4 config must list layer_types for every layer")
        sliding = [t == "sliding_attention" for t in lt]
        rp = cfg.get("rope_parameters") or {}
        rs, rg = rp.get("sliding_attention") or {}, rp.get("full_attention") or {}
        return ModelConfig(
            model_type=mt, hidden_size=int(cfg["hidden_size"]), num_hidden_layers=n_layers, num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads", heads)), head_dim=hd, vocab_size=int(cfg["vocab_size"]),
            intermediate_size=int(cfg.get("intermediate_size", 0)), rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
            rope_theta=float(rs.get("rope_theta", cfg.get("rope_local_base_freq", 1e4))), partial_rotary_factor=1.0,
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", True)), qk_norm=True, norm_zero_centered=False,
            sliding_window=int(cfg.get("sliding_window") or 0), softmax_scale=1.0,
            embed_scale=float(cfg["hidden_size"]) ** 0.5, logit_softcap=float(cfg.get("final_logit_softcapping") or 0.0),
            geglu=True, sandwich_norms=True, layer_scalar=True, v_norm=True, k_eq_v=bool(cfg.get("attention_k_eq_v", False)),
            sliding_layers=sliding, global_rope_theta=float(rg.get("rope_theta", 1e6)),
            global_partial_rotary=float(rg.get("partial_rotary_factor", 1.0)), global_rope_factor=float(rg.get("factor", 1.0)),
            global_rope_proportional=rg.get("rope_type", "proportional") == "proportional",
            global_head_dim=int(cfg.get("global_head_dim") or 0), num_global_key_value_heads=int(cfg.get("num_global_key_value_heads") or 0))

    @staticmethod
    def _k2_from_hf(cfg: dict, mt: str, n_layers: int, heads: int, hd: int) -> "ModelConfig":
        """K2-Horizon config (src/qwen35_loader.cpp:681-735): grouped norms, attention gate function, sigmoid router with
        bias and scaling, shared experts as one MLP of moe_intermediate_size * num_shared_experts, MoVA value experts on the
        sparse layers, dense FFN on ``mlp_only_layers`` / off-step layers; plain-w norms."""
        rp = cfg.get("rope_parameters") or {}
        gate = str(cfg.get("attention_gate_func") or "")
        n_shared, moe_i = int(cfg.get("num_shared_experts", 0)), int(cfg.get("moe_intermediate_size", 0))
        return ModelConfig(
            model_type=mt, hidden_size=int(cfg["hidden_size"]), num_hidden_layers=n_layers, num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads", heads)), head_dim=hd, vocab_size=int(cfg["vocab_size"]),
            intermediate_size=int(cfg.get("intermediate_size", 0)), rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
            rope_theta=float(rp.get("rope_theta", cfg.get("rope_theta", 1e6))), tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            qk_norm=bool(cfg.get("query_key_norm", False)), norm_zero_centered=False,
            attn_gate_proj="softplus" if "softplus" in gate else ("sigmoid" if gate else ""),
            num_experts=int(cfg.get("num_experts", 0)), num_experts_per_tok=int(cfg.get("num_experts_per_tok", 0)),
            moe_intermediate_size=moe_i, shared_expert_intermediate_size=moe_i * n_shared, num_shared_experts=n_shared,
            norm_topk_prob=bool(cfg.get("norm_topk_prob", True)), norm_groups=int(cfg.get("layernorm_num_groups", 1)),
            router_sigmoid="sigmoid" in str(cfg.get("router_score_func") or ""), router_scale=float(cfg.get("router_scaling_factor", 1.0)),
            mova_experts=int(cfg.get("mova_num_experts", 0)), mova_top_k=int(cfg.get("mova_num_experts_per_tok", 0)),
            mlp_only_layers=[int(v) for v in (cfg.get("mlp_only_layers") or [])], decoder_sparse_step=int(cfg.get("decoder_sparse_step", 1)),
            quant="fp8_block")

    @staticmethod
    def _muse_from_hf(cfg: dict, mt: str, n_layers: int, heads: int, hd: int) -> "ModelConfig":
        """Muse-Glimmer text config (src/qwen35_loader.cpp:667-680): sliding RoPE layers and full NoPE layers from
        ``layer_types``, query prescale from ``scale_query_by`` / ``qk_scale_factor``, attention output gate, (1 + w) norms."""
        lt = list(cfg.get("layer_types") or [])
        if len(lt) != n_layers:
            raise ValueError("a muse_glimmer config must list layer_types for every layer")
        rp = cfg.get("rope_parameters") or cfg.get("rope_scaling") or {}
        ex, qk = float(cfg.get("scale_query_by") or 0.0), float(cfg.get("qk_scale_factor") or 0.0)
        prescale = ex if ex > 0 else (qk if qk > 0 else 1.0)
        return ModelConfig(
            model_type=mt, hidden_size=int(cfg["hidden_size"]), num_hidden_layers=n_layers, num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads", heads)), head_dim=hd, vocab_size=int(cfg["vocab_size"]),
            intermediate_size=int(cfg.get("intermediate_size", 0)), rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
            rope_theta=float(rp.get("rope_theta", cfg.get("rope_theta", 1e6))),
            partial_rotary_factor=float(rp.get("partial_rotary_factor", cfg.get("partial_rotary_factor", 1.0))),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)), qk_norm=True, norm_zero_centered=True,
            sliding_window=int(cfg.get("sliding_window") or 0), softmax_scale=prescale / float(hd) ** 0.5,
            sandwich_norms=True, sliding_layers=[t == "sliding_attention" for t in lt], embed_norm=True, qk_norm_weightless=True,
            global_nope=True, attn_gate_proj="sigmoid")

    @staticmethod
    def from_dir(path: str | Path) -> "ModelConfig":
        return ModelConfig.from_hf(json.loads((Path(path) / "config.json").read_text()))


# ---------------------------------------------------------------------------------------------
# named configurations
# ---------------------------------------------------------------------------------------------
def tiny_dense() -> ModelConfig:
    """2 layers, hidden 256, 4q/2kv x 64, FFN 768, vocab 4096, tied embeddings, int4 g128."""
    return ModelConfig(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                       vocab_size=4096, intermediate_size=768, tie_word_embeddings=True, rope_theta=1e6)


def dense_27b(layers: int = 64) -> ModelConfig:
    """27B-class dense decoder: 64 layers, hidden 5120, 40q/8kv x 128, FFN 17408, vocab 151936."""
    return ModelConfig(hidden_size=5120, num_hidden_layers=layers, num_attention_heads=40, num_key_value_heads=8,
                       head_dim=128, vocab_size=151936, intermediate_size=17408, rope_theta=1e6)


def small_dense(layers: int = 4, wide: bool = False) -> ModelConfig:
    """A small GPU test model with 27B-like ratios (hidden 1024, 8q/2kv x 128, FFN 2816).  ``wide`` has 16q/8kv heads and
    FFN 4096, so that it still divides over 4 and 8 tensor-parallel ranks."""
    if wide:
        return ModelConfig(hidden_size=1024, num_hidden_layers=layers, num_attention_heads=16, num_key_value_heads=8,
                           head_dim=128, vocab_size=8192, intermediate_size=4096, rope_theta=1e6)
    return ModelConfig(hidden_size=1024, num_hidden_layers=layers, num_attention_heads=8, num_key_value_heads=2,
                       head_dim=128, vocab_size=8192, intermediate_size=2816, rope_theta=1e6)


def hybrid_moe_80b(layers: int = 48) -> ModelConfig:
    """Hybrid linear-attention MoE, 80B total / 3B active: 3 Gated DeltaNet layers then 1 gated
    full-attention layer; 512 experts x FFN 512, top-10 + 1 shared expert."""
    lt = [FULL_ATTN if (i % 4) == 3 else LINEAR_ATTN for i in range(layers)]
    return ModelConfig(model_type="qwen3_next", hidden_size=2048, num_hidden_layers=layers, num_attention_heads=16,
                       num_key_value_heads=2, head_dim=256, vocab_size=151936, intermediate_size=0,
                       partial_rotary_factor=0.25, attn_output_gate=True, qk_norm=True, norm_zero_centered=True,
                       layer_types=lt, linear_num_key_heads=16, linear_num_value_heads=32, linear_key_head_dim=128,
                       linear_value_head_dim=128, linear_conv_kernel_dim=4, gdn_chunk=64, num_experts=512,
                       num_experts_per_tok=10, moe_intermediate_size=512, shared_expert_intermediate_size=512,
                       quant="fp8_block")


def tiny_hybrid_moe(layers: int = 4) -> ModelConfig:
    lt = [FULL_ATTN if (i % 4) == 3 else LINEAR_ATTN for i in range(layers)]
    return ModelConfig(model_type="qwen3_next", hidden_size=256, num_hidden_layers=layers, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=4096, intermediate_size=0,
                       partial_rotary_factor=1.0, attn_output_gate=True, qk_norm=True, norm_zero_centered=True,
                       layer_types=lt, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=64,
                       linear_value_head_dim=64, num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128,
                       shared_expert_intermediate_size=128, quant="fp8_block")


def hybrid_dense_27b(layers: int = 64) -> ModelConfig:
    """The 27B hybrid with a dense FFN: 3 Gated DeltaNet layers then 1 gated full-attention layer (16 of 64), hidden 5120,
    24q / 4kv x 256, FFN 17408, DeltaNet 16 key / 48 value heads x 128 (the reference's own 27B: src/kernels.hpp:70-72,
    src/gemm_fast.cpp:812-816), int4 g128 projections."""
    lt = [FULL_ATTN if (i % 4) == 3 else LINEAR_ATTN for i in range(layers)]
    return ModelConfig(model_type="qwen3_5", hidden_size=5120, num_hidden_layers=layers, num_attention_heads=24,
                       num_key_value_heads=4, head_dim=256, vocab_size=151936, intermediate_size=17408,
                       partial_rotary_factor=0.25, attn_output_gate=True, qk_norm=True, norm_zero_centered=True,
                       layer_types=lt, linear_num_key_heads=16, linear_num_value_heads=48, linear_key_head_dim=128,
                       linear_value_head_dim=128, linear_conv_kernel_dim=4, gdn_chunk=64, rope_theta=1e7, quant="int4")


def tiny_hybrid_dense(layers: int = 4) -> ModelConfig:
    lt = [FULL_ATTN if (i % 4) == 3 else LINEAR_ATTN for i in range(layers)]
    return ModelConfig(model_type="qwen3_5", hidden_size=256, num_hidden_layers=layers, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=4096, intermediate_size=512,
                       partial_rotary_factor=1.0, attn_output_gate=True, qk_norm=True, norm_zero_centered=True,
                       layer_types=lt, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=64,
                       linear_value_head_dim=64, quant="int4")


def tiny_moe(layers: int = 2) -> ModelConfig:
    """A Qwen3-MoE-style decoder: plain (ungated) attention in every layer, routed experts without a shared expert."""
    return ModelConfig(model_type="qwen3_moe", hidden_size=256, num_hidden_layers=layers, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=4096, intermediate_size=0, qk_norm=True,
                       num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128, shared_expert_intermediate_size=0,
                       quant="fp8_block")


def tiny_qwen4_exp(layers: int = 4) -> ModelConfig:
    """The hybrid MoE decoder under three residual streams, sparse attention (budget 16 tokens in blocks of 4) and an n-gram
    embedding before layers 1 and 3."""
    lt = [FULL_ATTN if (i % 2) == 1 else LINEAR_ATTN for i in range(layers)]
    return ModelConfig(model_type="qwen4_exp_text", hidden_size=128, num_hidden_layers=layers, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=512, intermediate_size=0,
                       partial_rotary_factor=0.5, attn_output_gate=True, qk_norm=True, norm_zero_centered=True,
                       layer_types=lt, linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=64,
                       linear_value_head_dim=64, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                       shared_expert_intermediate_size=128, quant="fp8_block", hc_count=3, hc_lowrank=16, ple_layer_ids=[1, 3],
                       ple_embed_dim=32, ple_conv_kernel_size=3, ngram_size=3, heads_per_ngram=2, ngram_vocab_size_base=50,
                       ngram_seed=7, eos_token_id=2, indexer_n_heads=2, indexer_head_dim=64, indexer_budget=16, indexer_compress_ratio=4)


def tiny_gemma4(layers: int = 4) -> ModelConfig:
    """A small Gemma-4-style decoder: 3 sliding-window layers then 1 global layer (no v_proj, proportional RoPE over a
    quarter of the head), sandwich norms, GeGLU, layer scalars, logit soft cap; one head geometry for both layer types."""
    sliding = [(i % 4) != 3 for i in range(layers)]
    return ModelConfig(model_type="gemma4_text", hidden_size=256, num_hidden_layers=layers, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=4096, intermediate_size=512, tie_word_embeddings=True,
                       rope_theta=1e4, qk_norm=True, sliding_window=16, softmax_scale=1.0, embed_scale=16.0, logit_softcap=30.0,
                       geglu=True, sandwich_norms=True, layer_scalar=True, v_norm=True, k_eq_v=True, sliding_layers=sliding,
                       global_rope_theta=1e6, global_partial_rotary=0.25, global_rope_proportional=True, quant="int4")


def tiny_muse(layers: int = 4) -> ModelConfig:
    """A small Muse-Glimmer-style decoder: 3 sliding RoPE layers then 1 full layer without positional embedding, sandwich
    norms in the (1 + w) convention, weightless q / k norms, a sigmoid output gate projection, SwiGLU, normalised embeddings."""
    return ModelConfig(model_type="muse_glimmer_text", hidden_size=256, num_hidden_layers=layers, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=4096, intermediate_size=512, tie_word_embeddings=False,
                       rope_theta=1e6, qk_norm=True, norm_zero_centered=True, sliding_window=16, softmax_scale=0.5 / 8.0,
                       sandwich_norms=True, sliding_layers=[(i % 4) != 3 for i in range(layers)], embed_norm=True,
                       qk_norm_weightless=True, global_nope=True, attn_gate_proj="sigmoid", quant="int4")


def tiny_k2(layers: int = 3) -> ModelConfig:
    """A small K2-Horizon-style decoder: layer 0 dense, the rest sparse (routed value projection + MoE with an ungated
    shared expert), two-group norms, softplus attention gate, sigmoid router with a selection bias and a scaling factor."""
    return ModelConfig(model_type="k2_horizon", hidden_size=256, num_hidden_layers=layers, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=4096, intermediate_size=512, qk_norm=True,
                       attn_gate_proj="softplus", num_experts=16, num_experts_per_tok=4, moe_intermediate_size=128,
                       shared_expert_intermediate_size=128, num_shared_experts=1, norm_topk_prob=True, norm_groups=2, router_sigmoid=True,
                       router_scale=2.5, mova_experts=8, mova_top_k=2, mlp_only_layers=[0], decoder_sparse_step=1, quant="fp8_block")


PRESETS = {"tiny_qwen4_exp": tiny_qwen4_exp, "tiny_k2": tiny_k2, "tiny_muse": tiny_muse, "tiny_gemma4": tiny_gemma4, "hybrid_dense_27b": hybrid_dense_27b, "tiny_hybrid_dense": tiny_hybrid_dense, "tiny_moe": tiny_moe, "tiny_dense": tiny_dense, "dense_27b": dense_27b, "small_dense": small_dense,
           "hybrid_moe_80b": hybrid_moe_80b, "tiny_hybrid_moe": tiny_hybrid_moe}
