"""DFlash block-drafter configuration.

Only the *configuration resolution* of the reference's DFlash / DFlash2 drafter is provided here:
turning a draft checkpoint's ``config.json`` into the facts the draft forward pass needs, with the
precedence rules the reference pins in include/b70/dflash_config.hpp:60-352 (which follow vLLM's
qwen3_dflash resolution): ``dflash_config`` overrides ``eagle_config`` overrides the top level for
the drafter's own knobs; the attention shape is read from ``layer_types`` / ``dflash_config.use_swa``
/ ``is_causal`` / ``dflash_config.causal`` only; a silent config means full, non-causal attention;
the default RoPE theta is 1e6.  Every one of these is a silent failure when wrong (the verifier just
rejects the drafts), so each default that is not a checkpoint fact is reported in ``notes`` and
impossible combinations in ``error``.  The draft model itself is models/dflash_drafter.py.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field


@dataclass
class DFlashLayerAttn:
    window: int = 0          # 0 = full attention
    causal: bool = False


@dataclass
class DFlashSettings:
    n_layers: int = 0
    hidden: int = 0
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    inter: int = 0
    vocab: int = 0
    draft_vocab: int = 0
    mask_token: int = -1
    selector_top_k: int = 0
    selector_rank: int = 0
    conv_kernel_size: int = 0      # second-generation drafter: taps of the grouped dynamic convolutions (0: none)
    conv_group_size: int = 0
    input_embedding_scale: float = 1.0
    output_multiplier: float = 1.0
    final_logit_softcapping: float = 0.0
    block_size: int = 16
    config_window: int = 0
    rope_theta: float = 1.0e6
    rms_eps: float = 1.0e-6
    attention_bias: bool = False
    use_aux_hidden_state: bool = True
    attn_from_config: bool = False
    tap_key: str = ""
    target_layers: list = field(default_factory=list)
    layers: list = field(default_factory=list)
    notes: list = field(default_factory=list)
    error: str = ""


def _is_num(v) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


def _stated_flag(obj, key):
    """A flag the config states explicitly; numbers count (bool(1)), other kinds do not."""
    if not isinstance(obj, dict) or key not in obj:
        return None
    v = obj[key]
    if isinstance(v, bool):
        return v
    if _is_num(v):
        return v != 0
    return None


def resolve_dflash_config(text: str) -> DFlashSettings:
    s = DFlashSettings()
    try:
        top = json.loads(text)
    except ValueError as e:
        s.error = f"draft config.json is not valid JSON: {e}"
        return s
    if not isinstance(top, dict):
        s.error = "draft config.json is not a JSON object"
        return s
    dflash = top.get("dflash_config") if isinstance(top.get("dflash_config"), dict) else None
    eagle = top.get("eagle_config") if isinstance(top.get("eagle_config"), dict) else None
    scopes = [sc for sc in (dflash, eagle, top) if sc is not None]

    def lookup(key, pred):
        for sc in scopes:
            if key in sc and pred(sc[key]):
                return sc[key]
        return None

    def number_or(key, fallback):
        v = lookup(key, _is_num)
        return int(v) if v is not None else fallback

    def flag_or(key, fallback):
        v = lookup(key, lambda x: isinstance(x, bool))
        return v if v is not None else fallback

    s.n_layers = number_or("num_hidden_layers", 0)
    s.hidden = number_or("hidden_size", 0)
    s.n_heads = number_or("num_attention_heads", 0)
    s.n_kv_heads = number_or("num_key_value_heads", s.n_heads)
    s.inter = number_or("intermediate_size", 0)
    s.vocab = number_or("vocab_size", 0)
    s.draft_vocab = number_or("draft_vocab_size", s.vocab)
    s.attention_bias = flag_or("attention_bias", False)
    s.use_aux_hidden_state = flag_or("use_aux_hidden_state", True)
    s.selector_top_k = number_or("selector_top_k", 0)
    s.selector_rank = number_or("selector_rank", 0)
    s.conv_kernel_size = number_or("conv_kernel_size", 0)
    s.conv_group_size = number_or("conv_group_size", 0)
    for key in ("input_embedding_scale", "output_multiplier", "final_logit_softcapping"):
        v = lookup(key, _is_num)
        if v is not None:
            setattr(s, key, float(v))
    if (s.conv_kernel_size > 0) != (s.conv_group_size > 0) and not s.error:
        s.error = "conv_kernel_size and conv_group_size must be given together"
    s.block_size = number_or("block_size", 16)
    if s.block_size <= 0:
        s.block_size = 16
    if s.n_layers <= 0:
        s.error = "draft config.json has no usable num_hidden_layers"
    s.head_dim = number_or("head_dim", 0)
    if s.head_dim <= 0 and s.n_heads > 0:
        s.head_dim = s.hidden // s.n_heads
    v = lookup("rms_norm_eps", _is_num)
    if v is not None:
        s.rms_eps = float(v)

    rope = None
    rp = top.get("rope_parameters")
    if isinstance(rp, dict) and _is_num(rp.get("rope_theta")):
        rope = float(rp["rope_theta"])
    elif _is_num(top.get("rope_theta")):
        rope = float(top["rope_theta"])
    if rope is None:
        s.notes.append("no rope_theta in the draft config; using the default 1000000")
    else:
        s.rope_theta = rope

    v = lookup("mask_token_id", _is_num)
    if v is not None:
        s.mask_token = int(v)
    else:
        s.notes.append("no mask_token_id in the draft config: mask rows would be embedded from a guessed id")

    for key in ("target_layer_ids", "aux_hidden_state_layer_ids", "eagle_aux_hidden_state_layer_ids"):
        arr = lookup(key, lambda x: isinstance(x, list))
        if arr is None or not arr or not all(_is_num(e) for e in arr):
            continue
        s.target_layers, s.tap_key = [int(e) for e in arr], key
        break
    if not s.target_layers:
        s.notes.append("the draft config names no target layer ids; any taps used are a built-in default")

    layer_types = top.get("layer_types") if isinstance(top.get("layer_types"), list) else None
    swa_flag = _stated_flag(dflash, "use_swa")
    use_swa = bool(swa_flag) if swa_flag is not None else False
    any_sliding = bool(layer_types) and any(e == "sliding_attention" for e in layer_types)
    is_causal = _stated_flag(top, "is_causal")
    causal_override = _stated_flag(dflash, "causal")
    s.attn_from_config = layer_types is not None or swa_flag is not None or is_causal is not None or causal_override is not None
    if layer_types is not None and s.n_layers > 0:
        if len(layer_types) < s.n_layers and not s.error:
            s.error = f"draft config layer_types has only {len(layer_types)} entries for {s.n_layers} layers"
        elif len(layer_types) > s.n_layers:
            s.notes.append(f"layer_types lists {len(layer_types)} layers for a {s.n_layers}-layer drafter; reading the first {s.n_layers}")

    window = 0
    if dflash is not None and _is_num(dflash.get("swa_window_size")):
        window = int(dflash["swa_window_size"])
    if window <= 0 and _is_num(top.get("sliding_window")):
        window = int(top["sliding_window"])
    s.config_window = window
    for i in range(max(0, s.n_layers)):
        typed_sliding = layer_types is not None and i < len(layer_types) and layer_types[i] == "sliding_attention"
        is_sliding = use_swa if (layer_types is None or (use_swa and not any_sliding)) else typed_sliding
        causal = is_causal if is_causal is not None else (causal_override if causal_override is not None
                                                          else (layer_types is not None and typed_sliding))
        s.layers.append(DFlashLayerAttn(window if is_sliding else 0, bool(causal)))
        if is_sliding and window <= 0 and not s.error:
            s.error = f"draft layer {i} uses sliding attention but the config gives no window"
    if not s.attn_from_config:
        s.notes.append("the draft config describes no attention shape: every layer is full attention and non-causal")
    if (dflash is not None and "attention_sink_bias" in dflash) or "add_swa_attention_sink_bias" in top:
        s.notes.append("this drafter declares an attention sink bias; the draft attention here has no sink term")
    if _is_num(top.get("logit_scale")) and top["logit_scale"] != 1.0:
        s.notes.append("logit_scale is not 1: the draft argmax is unaffected but selector scores are unscaled")
    if s.attention_bias:
        s.notes.append("attention_bias is set: this engine's projections carry no bias term")
    return s
