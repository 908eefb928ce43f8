"""GGUF checkpoints: container access, block dequantisation and the architecture adapter that maps
llama.cpp tensor names onto the HF names the model builders use.

Reference: GGUFFile / gguf_dequantize (src/gguf.cpp, src/gguf_decode.cpp) and the arch adapters with
their inverse tensor transforms (src/gguf_qwen35.cpp:80-785).  The tokenizer stored in the file is
exposed as a ``tokenizer.json``-shaped dict for the C++ BPE core.
"""
from __future__ import annotations

import ctypes
import json
from pathlib import Path
from typing import Optional

import torch

from .. import _native

GGML_TYPES = {0: "F32", 1: "F16", 2: "Q4_0", 3: "Q4_1", 6: "Q5_0", 7: "Q5_1", 8: "Q8_0", 9: "Q8_1", 10: "Q2_K", 11: "Q3_K", 12: "Q4_K",
              13: "Q5_K", 14: "Q6_K", 15: "Q8_K", 20: "IQ4_NL", 23: "IQ4_XS", 24: "I8", 25: "I16", 26: "I32", 27: "I64", 28: "F64",
              30: "BF16", 35: "TQ2_0", 39: "MXFP4"}


def dequantize(type_id: int, raw: bytes | torch.Tensor, n_elems: int) -> torch.Tensor:
    """Decode raw ggml blocks to fp32."""
    lib = _native.host()
    buf = raw if isinstance(raw, (bytes, bytearray)) else raw.contiguous().numpy().tobytes()
    out = torch.empty(n_elems, dtype=torch.float32)
    rc = lib.grm_gguf_dequant(ctypes.c_int(type_id), buf, ctypes.c_int64(len(buf)), ctypes.c_void_p(out.data_ptr()), ctypes.c_int64(n_elems))
    if rc == -1:
        raise NotImplementedError(f"ggml type {type_id} is not decoded by this build")
    if rc != 0:
        raise ValueError(f"ggml type {type_id}: {len(buf)} bytes do not hold {n_elems} elements")
    return out


class GGUFFile:
    def __init__(self, path: str | Path):
        lib = _native.host()
        lib.grm_gguf_open.restype = ctypes.c_void_p
        lib.grm_gguf_tensor_data.restype = ctypes.c_void_p
        lib.grm_gguf_meta_len.restype = ctypes.c_int64
        err = ctypes.create_string_buffer(512)
        h = lib.grm_gguf_open(str(path).encode(), err, 512)
        if not h:
            raise ValueError(f"{path}: {err.value.decode(errors='replace')}")
        self._h, self._lib = ctypes.c_void_p(h), lib
        n = lib.grm_gguf_meta_len(self._h)
        buf = ctypes.create_string_buffer(n + 1)
        lib.grm_gguf_meta(self._h, buf)
        self.metadata = json.loads(buf.raw[:n].decode("utf-8", errors="replace"))
        self.version = lib.grm_gguf_version(self._h)
        self.tensors: dict[str, tuple[int, int, tuple[int, ...], int]] = {}
        name = ctypes.create_string_buffer(512)
        typ, nbytes = ctypes.c_int(), ctypes.c_uint64()
        dims = (ctypes.c_uint64 * 8)()
        for i in range(lib.grm_gguf_tensor_count(self._h)):
            nd = lib.grm_gguf_tensor_info(self._h, i, name, 512, ctypes.byref(typ), dims, ctypes.byref(nbytes))
            self.tensors[name.value.decode()] = (i, typ.value, tuple(int(dims[d]) for d in range(nd)), int(nbytes.value))

    def close(self):
        if self._h:
            self._lib.grm_gguf_close(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def raw(self, name: str) -> bytes:
        i, _, _, nb = self.tensors[name]
        return ctypes.string_at(self._lib.grm_gguf_tensor_data(self._h, i), nb)

    def tensor(self, name: str) -> torch.Tensor:
        """fp32 tensor in the HF (row-major, outermost first) shape; ggml stores dims innermost first."""
        i, typ, dims, nb = self.tensors[name]
        n = 1
        for d in dims:
            n *= d
        return dequantize(typ, self.raw(name), n).reshape(tuple(reversed(dims)))

    def raw_rows(self, name: str) -> tuple[torch.Tensor, int]:
        """A 2-D tensor as its stored blocks: (uint8 [rows][bytes per row], ggml type id).  ggml keeps the input dimension
        innermost, so a weight's output rows are contiguous runs of whole blocks."""
        i, typ, dims, nb = self.tensors[name]
        if len(dims) != 2:
            raise ValueError(f"{name}: not a matrix")
        rows = dims[1]
        if nb % rows:
            raise ValueError(f"{name}: {nb} bytes do not split into {rows} rows")
        buf = torch.frombuffer(bytearray(self.raw(name)), dtype=torch.uint8)
        return buf.reshape(rows, nb // rows), typ

    @property
    def arch(self) -> str:
        return self.metadata.get("general.architecture", "")


# llama.cpp tensor names -> HF names (dense attention decoders of the qwen2/qwen3 families)
_LAYER_MAP = {"attn_norm": "input_layernorm", "ffn_norm": "post_attention_layernorm", "attn_q": "self_attn.q_proj",
              "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
              "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm", "ffn_gate": "mlp.gate_proj",
              "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}


# gemma4: the same projections under other norm names, plus the per-layer output scale (src/gguf_qwen35.cpp:700-760)
_GEMMA4_LAYER_MAP = dict(_LAYER_MAP, ffn_norm="pre_feedforward_layernorm", post_attention_norm="post_attention_layernorm",
                         post_ffw_norm="post_feedforward_layernorm")


def hf_name(gguf_name: str, arch: str = "") -> Optional[str]:
    if arch == "gemma4" and gguf_name.startswith("blk."):
        _, layer, rest = gguf_name.split(".", 2)
        stem, _, suffix = rest.rpartition(".")
        if stem == "layer_output_scale":
            return f"model.layers.{layer}.layer_scalar"
        if stem in _GEMMA4_LAYER_MAP:
            return f"model.layers.{layer}.{_GEMMA4_LAYER_MAP[stem]}.{suffix}"
        return None
    if gguf_name == "token_embd.weight":
        return "model.embed_tokens.weight"
    if gguf_name == "output_norm.weight":
        return "model.norm.weight"
    if gguf_name == "output.weight":
        return "lm_head.weight"
    if gguf_name.startswith("blk."):
        _, layer, rest = gguf_name.split(".", 2)
        stem, _, suffix = rest.rpartition(".")
        if stem in _LAYER_MAP:
            return f"model.layers.{layer}.{_LAYER_MAP[stem]}.{suffix}"
    return None


def config_from_gguf(g: GGUFFile):
    """ModelConfig from the GGUF metadata keys (``<arch>.block_count`` ...)."""
    from ..models.config import ModelConfig

    a, m = g.arch, g.metadata
    if a == "gemma4":
        return _gemma4_config_from_gguf(g)
    if a in ("qwen35", "qwen35moe"):
        return _qwen35_config_from_gguf(g)
    if a == "qwen3moe":
        return _qwen3moe_config_from_gguf(g)
    heads = int(m[f"{a}.attention.head_count"])
    hidden = int(m[f"{a}.embedding_length"])
    emb = g.tensors.get("token_embd.weight")
    return ModelConfig(model_type=a, hidden_size=hidden, num_hidden_layers=int(m[f"{a}.block_count"]), num_attention_heads=heads,
                       num_key_value_heads=int(m.get(f"{a}.attention.head_count_kv", heads)),
                       head_dim=int(m.get(f"{a}.attention.key_length", hidden // heads)),
                       vocab_size=int(m.get(f"{a}.vocab_size", emb[2][1] if emb else 0)),
                       intermediate_size=int(m.get(f"{a}.feed_forward_length", 0)),
                       rms_norm_eps=float(m.get(f"{a}.attention.layer_norm_rms_epsilon", 1e-6)),
                       rope_theta=float(m.get(f"{a}.rope.freq_base", 1e6)), tie_word_embeddings="output.weight" not in g.tensors,
                       qk_norm="blk.0.attn_q_norm.weight" in g.tensors)


def _gemma4_config_from_gguf(g: GGUFFile):
    """``gemma4.*`` metadata -> ModelConfig (gguf_gemma4_config, src/gguf_qwen35.cpp:568-690): per-type key / rope keys
    (``*_swa`` for the sliding layers), per-layer ``head_count_kv`` and ``sliding_window_pattern`` arrays, and the
    ``rope_freqs.weight`` tensor whose ones mark the rotated pairs of the global layers' proportional RoPE."""
    from ..models.config import ModelConfig

    m, p = g.metadata, "gemma4."
    L, hidden, heads = int(m[p + "block_count"]), int(m[p + "embedding_length"]), int(m[p + "attention.head_count"])
    hd_full, hd_swa = int(m[p + "attention.key_length"]), int(m[p + "attention.key_length_swa"])
    if int(m.get(p + "attention.shared_kv_layers", 0)) or int(m.get(p + "embedding_length_per_layer_input", 0)) or (p + "expert_count") in m:
        raise ValueError("gemma4 GGUF: shared KV layers, per-layer input embeddings and MoE variants are not served")
    pattern = [int(v) for v in m[p + "attention.sliding_window_pattern"]]
    kv = m[p + "attention.head_count_kv"]
    kv = [int(v) for v in kv] if isinstance(kv, (list, tuple)) else [int(kv)] * L
    if len(pattern) != L or len(kv) != L:
        raise ValueError("gemma4 GGUF: per-layer head_count_kv / sliding_window_pattern must have block_count entries")
    sliding = [bool(v) for v in pattern]
    kv_swa = {kv[i] for i in range(L) if sliding[i]} or {kv[0]}
    kv_full = {kv[i] for i in range(L) if not sliding[i]} or kv_swa
    if len(kv_swa) != 1 or len(kv_full) != 1:
        raise ValueError("gemma4 GGUF: head_count_kv differs within an attention type")
    partial = 1.0
    if "rope_freqs.weight" in g.tensors:
        f = g.tensor("rope_freqs.weight").float()
        partial = float((f == 1.0).sum()) / max(1, f.numel())        # ones on the rotated pairs, a huge factor on the rest
    has_v_full = all(f"blk.{i}.attn_v.weight" in g.tensors for i in range(L) if not sliding[i])
    emb = g.tensors.get("token_embd.weight")
    n_swa, n_full = next(iter(kv_swa)), next(iter(kv_full))
    return ModelConfig(
        model_type="gemma4_text", hidden_size=hidden, num_hidden_layers=L, num_attention_heads=heads, num_key_value_heads=n_swa,
        head_dim=hd_swa, vocab_size=int(m.get(p + "vocab_size", emb[2][1] if emb else 0)),
        intermediate_size=int(m[p + "feed_forward_length"]), rms_norm_eps=float(m[p + "attention.layer_norm_rms_epsilon"]),
        rope_theta=float(m[p + "rope.freq_base_swa"]), tie_word_embeddings="output.weight" not in g.tensors, qk_norm=True,
        sliding_window=int(m[p + "attention.sliding_window"]), softmax_scale=1.0, embed_scale=float(hidden) ** 0.5,
        logit_softcap=float(m.get(p + "final_logit_softcapping", 0.0)), geglu=True, sandwich_norms=True, layer_scalar=True, v_norm=True,
        k_eq_v=not has_v_full, sliding_layers=sliding, global_rope_theta=float(m[p + "rope.freq_base"]), global_partial_rotary=partial,
        global_rope_proportional=True, global_head_dim=hd_full if hd_full != hd_swa else 0,
        num_global_key_value_heads=n_full if n_full != n_swa else 0)


def _qwen35_config_from_gguf(g: GGUFFile):
    """``qwen35.*`` / ``qwen35moe.*`` metadata -> ModelConfig of the hybrid (Gated DeltaNet + gated attention) family
    (gguf_qwen35_config, src/gguf_qwen35.cpp:80-212).  llama.cpp's ssm names carry the DeltaNet geometry: ``ssm.group_count``
    key heads, ``ssm.time_step_rank`` value heads, ``ssm.state_size`` key width, ``ssm.inner_size`` = value heads x value
    width; every ``full_attention_interval``-th layer attends; a trailing ``nextn_predict_layers`` block is the draft head
    and does not count as a decoder layer; a q projection with twice the query rows carries the output gate."""
    from ..models.config import ModelConfig

    a, m = g.arch, g.metadata
    moe, p = a == "qwen35moe", a + "."
    blocks, mtp = int(m[p + "block_count"]), int(m.get(p + "nextn_predict_layers", 0))
    hidden, heads, kv = int(m[p + "embedding_length"]), int(m[p + "attention.head_count"]), int(m[p + "attention.head_count_kv"])
    hd, vd, rope = int(m[p + "attention.key_length"]), int(m[p + "attention.value_length"]), int(m[p + "rope.dimension_count"])
    nk, nv, dk = int(m[p + "ssm.group_count"]), int(m[p + "ssm.time_step_rank"]), int(m[p + "ssm.state_size"])
    inner, conv, interval = int(m[p + "ssm.inner_size"]), int(m[p + "ssm.conv_kernel"]), int(m[p + "full_attention_interval"])
    L = blocks - mtp
    if mtp >= blocks or not hd or hd != vd or not nk or not nv or nv % nk or inner % nv or not interval:
        raise ValueError(f"inconsistent {a} GGUF geometry")
    emb = g.tensors.get("token_embd.weight")
    if emb is None or len(emb[2]) != 2 or emb[2][0] != hidden:
        raise ValueError("GGUF token_embd.weight shape disagrees with embedding_length")
    gate = None
    for i in range(L):
        q = g.tensors.get(f"blk.{i}.attn_q.weight")
        if q is None:
            continue
        if len(q[2]) != 2 or q[2][0] != hidden or q[2][1] not in (heads * hd, 2 * heads * hd):
            raise ValueError("GGUF attn_q.weight has invalid query width")
        this = q[2][1] == 2 * heads * hd
        if gate is not None and gate != this:
            raise ValueError("GGUF attn_q output gate differs across layers")
        gate = this
    if gate is None:
        raise ValueError("GGUF has no full-attention attn_q.weight")
    types = ["linear_attention" if (i + 1) % interval else "full_attention" for i in range(L)]
    rec = m.get(p + "recurrent_layers")
    if rec is not None and [bool(v) for v in rec] != [t == "linear_attention" for t in types]:
        raise ValueError("GGUF recurrent_layers contradicts full_attention_interval")
    tc = {"model_type": "qwen3_5_moe_text" if moe else "qwen3_5_text", "num_hidden_layers": L, "hidden_size": hidden,
          "vocab_size": emb[2][1], "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": hd,
          "rms_norm_eps": float(m[p + "attention.layer_norm_rms_epsilon"]), "linear_num_key_heads": nk, "linear_num_value_heads": nv,
          "linear_key_head_dim": dk, "linear_value_head_dim": inner // nv, "linear_conv_kernel_dim": conv, "mtp_num_hidden_layers": mtp,
          "attn_output_gate": gate, "tie_word_embeddings": "output.weight" not in g.tensors, "layer_types": types,
          "rope_parameters": {"rope_theta": float(m[p + "rope.freq_base"]), "partial_rotary_factor": rope / hd}}
    if moe:
        tc.update(num_experts=int(m[p + "expert_count"]), num_experts_per_tok=int(m[p + "expert_used_count"]),
                  moe_intermediate_size=int(m[p + "expert_feed_forward_length"]),
                  shared_expert_intermediate_size=int(m[p + "expert_shared_feed_forward_length"]))
    else:
        tc["intermediate_size"] = int(m[p + "feed_forward_length"])
    return ModelConfig.from_hf({"model_type": "qwen3_5_moe" if moe else "qwen3_5", "text_config": tc})


def _qwen3moe_config_from_gguf(g: GGUFFile):
    """``qwen3moe.*`` metadata -> ModelConfig of a Qwen3-MoE decoder (gguf_qwen3_config, src/gguf_qwen35.cpp:214-326): plain
    attention, no shared expert; a layer without a router tensor carries a dense FFN and is listed as ``mlp_only``."""
    from ..models.config import ModelConfig

    m, p = g.metadata, "qwen3moe."
    L, hidden, heads = int(m[p + "block_count"]), int(m[p + "embedding_length"]), int(m[p + "attention.head_count"])
    kv, hd = int(m[p + "attention.head_count_kv"]), int(m[p + "attention.key_length"])
    ne, top = int(m[p + "expert_count"]), int(m[p + "expert_used_count"])
    if int(m.get(p + "expert_shared_feed_forward_length", 0)):
        raise ValueError("qwen3moe expert_shared_feed_forward_length is nonzero; Qwen3-MoE has no shared expert")
    if not ne or not top or top > ne or heads % kv or hd != int(m.get(p + "attention.value_length", hd)):
        raise ValueError("inconsistent qwen3moe GGUF geometry")
    emb = g.tensors.get("token_embd.weight")
    if emb is None or len(emb[2]) != 2 or emb[2][0] != hidden:
        raise ValueError("qwen3moe token_embd.weight shape disagrees with embedding_length")
    dense_layers = []
    for i in range(L):
        if f"blk.{i}.ffn_gate_inp.weight" not in g.tensors:
            for role in ("ffn_gate", "ffn_up", "ffn_down"):
                if f"blk.{i}.{role}.weight" not in g.tensors:
                    raise ValueError(f"qwen3moe layer {i} has neither a router nor {role}.weight")
            dense_layers.append(i)
    return ModelConfig.from_hf({
        "model_type": "qwen3_moe", "num_hidden_layers": L, "hidden_size": hidden, "intermediate_size": int(m[p + "feed_forward_length"]),
        "vocab_size": emb[2][1], "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": hd,
        "rope_theta": float(m[p + "rope.freq_base"]), "rms_norm_eps": float(m[p + "attention.layer_norm_rms_epsilon"]),
        "attn_output_gate": False, "tie_word_embeddings": "output.weight" not in g.tensors, "num_experts": ne,
        "num_experts_per_tok": top, "moe_intermediate_size": int(m[p + "expert_feed_forward_length"]),
        "shared_expert_intermediate_size": 0, "decoder_sparse_step": 1, "norm_topk_prob": True, "mlp_only_layers": dense_layers})


_HYBRID_LAYER_MAP = dict(_LAYER_MAP, post_attention_norm="post_attention_layernorm", attn_qkv="linear_attn.in_proj_qkv",
                         attn_gate="linear_attn.in_proj_z", ssm_alpha="linear_attn.in_proj_a", ssm_beta="linear_attn.in_proj_b",
                         ssm_conv1d="linear_attn.conv1d", ssm_norm="linear_attn.norm", ssm_out="linear_attn.out_proj",
                         ffn_gate_inp="mlp.gate", ffn_gate_inp_shexp="mlp.shared_expert_gate", ffn_gate_shexp="mlp.shared_expert.gate_proj",
                         ffn_up_shexp="mlp.shared_expert.up_proj", ffn_down_shexp="mlp.shared_expert.down_proj")
_NEXTN_MAP = {"nextn.eh_proj.weight": "mtp.fc.weight", "nextn.enorm.weight": "mtp.pre_fc_norm_embedding.weight",
              "nextn.hnorm.weight": "mtp.pre_fc_norm_hidden.weight", "nextn.shared_head_norm.weight": "mtp.norm.weight"}
_ZERO_CENTRED = ("attn_norm", "post_attention_norm", "attn_q_norm", "attn_k_norm")


def v_head_order(nk: int, nv: int, width: int = 1) -> torch.Tensor:
    """Source index of every element of a value-head axis: HF groups the ``nv`` value heads by key head (head = key * r + j,
    r = nv / nk), llama.cpp's converter stores them tiled (j * nk + key) so that a head repeat broadcasts
    (gguf_v_tiled_index, src/gguf_qwen35.cpp:51).  ``width`` elements per head move together."""
    r = nv // nk
    h = torch.arange(nv)
    tiled = (h % r) * nk + h // r
    return (tiled[:, None] * width + torch.arange(width)[None, :]).reshape(-1)


def _hybrid_state_dict(g: GGUFFile, cfg) -> dict[str, torch.Tensor]:
    """HF-named fp32 tensors of a ``qwen35`` / ``qwen35moe`` / ``qwen3moe`` file with the converter's transforms undone
    (gguf_qwen35_index + read_gguf_f32, src/gguf_qwen35.cpp:328-563): value heads back into key-grouped order on the rows
    of in_proj_qkv's v part / in_proj_z / in_proj_a / in_proj_b / conv1d, the columns of out_proj and the entries of
    dt_bias / A; ``ssm_a`` = -exp(A_log) back to A_log; the stored ``1 + w`` of every zero-centred norm back to w (both
    rounded to bf16, the checkpoint's precision); the stacked expert tensors split into gate_up / down."""
    a = g.arch
    q35 = a != "qwen3moe"
    pre = "model.language_model." if q35 else "model."
    L, mtp = cfg.num_hidden_layers, cfg.mtp_num_hidden_layers
    nk, nv, dk, dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
    qk = 2 * nk * dk
    bf = lambda t: t.bfloat16().float()
    unnorm = (lambda t: bf(t - 1.0)) if q35 else (lambda t: t)
    out: dict[str, torch.Tensor] = {}
    experts: dict[str, dict[str, torch.Tensor]] = {}
    for name in g.tensors:
        if name == "token_embd.weight":
            out[pre + "embed_tokens.weight"] = g.tensor(name)
            continue
        if name == "output.weight":
            out["lm_head.weight"] = g.tensor(name)
            continue
        if name == "output_norm.weight":
            out[pre + "norm.weight"] = unnorm(g.tensor(name))
            continue
        if name.startswith("nextn.") or name == "rope_freqs.weight":
            continue
        if not name.startswith("blk."):
            raise ValueError(f"unmapped GGUF tensor: {name}")
        _, layer, role = name.split(".", 2)
        l = int(layer)
        if l == L and mtp < 1:
            continue                                     # a draft block the metadata does not declare stays unused
        if l > L or l < 0:
            raise ValueError(f"unmapped GGUF layer tensor: {name}")
        if l == L:
            if role in _NEXTN_MAP:
                t = g.tensor(name)
                out[_NEXTN_MAP[role]] = t if role == "nextn.eh_proj.weight" else unnorm(t)
                continue
            if role in ("nextn.embed_tokens.weight", "nextn.shared_head_head.weight"):
                continue                                 # the draft head shares the main embedding and output head
            if role.startswith("nextn."):
                raise ValueError(f"unmapped GGUF MTP tensor: {name}")
        b = "mtp.layers.0." if l == L else f"{pre}layers.{l}."
        stem, _, suffix = role.rpartition(".")
        if role == "ssm_a":
            out[b + "linear_attn.A_log"] = bf(torch.log(-g.tensor(name).reshape(-1)[v_head_order(nk, nv)].double()).float())
            continue
        if role == "ssm_dt.bias":
            out[b + "linear_attn.dt_bias"] = g.tensor(name).reshape(-1)[v_head_order(nk, nv)]
            continue
        if stem in ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"):
            t = g.tensor(name)                           # [E][rows][cols]
            if t.dim() != 3 or t.shape[0] != cfg.num_experts:
                raise ValueError(f"GGUF expert shape mismatch: {name}")
            experts.setdefault(b, {})[stem] = t
            continue
        hf = _HYBRID_LAYER_MAP.get(stem) if not (stem == "ffn_norm" and q35) else None
        if hf is None:
            raise ValueError(f"unmapped GGUF tensor: {name}")
        t = g.tensor(name)
        if stem in _ZERO_CENTRED:
            t = unnorm(t)
        elif stem in ("attn_qkv", "ssm_conv1d"):
            t = torch.cat([t[:qk], t[qk:][v_head_order(nk, nv, dv)]])
            if stem == "ssm_conv1d":
                t = t.reshape(t.shape[0], 1, -1)         # HF keeps the depthwise filter as [C][1][K]
        elif stem == "attn_gate":
            t = t[v_head_order(nk, nv, dv)]
        elif stem in ("ssm_alpha", "ssm_beta"):
            t = t[v_head_order(nk, nv)]
        elif stem == "ssm_out":
            t = t[:, v_head_order(nk, nv, dv)]
        elif stem == "ffn_gate_inp_shexp" and t.dim() == 1:
            t = t.reshape(1, -1)
        out[f"{b}{hf}.{suffix}"] = t
    for b, e in experts.items():
        if set(e) != {"ffn_gate_exps", "ffn_up_exps", "ffn_down_exps"}:
            raise ValueError(f"GGUF layer {b} lacks one of the stacked expert tensors")
        out[b + "mlp.experts.gate_up_proj"] = torch.cat([e["ffn_gate_exps"], e["ffn_up_exps"]], dim=1)
        out[b + "mlp.experts.down_proj"] = e["ffn_down_exps"]
    return out


def state_dict_from_gguf(g: GGUFFile, cfg=None) -> dict[str, torch.Tensor]:
    """Every tensor with a known HF name, dequantized to fp32 (the hybrid and MoE families need their config for the
    converter's inverse transforms)."""
    if g.arch in ("qwen35", "qwen35moe", "qwen3moe"):
        return _hybrid_state_dict(g, cfg if cfg is not None else config_from_gguf(g))
    out = {}
    for name in g.tensors:
        hn = hf_name(name, g.arch)
        if hn is not None:
            out[hn] = g.tensor(name)
    return out


def tokenizer_json_from_gguf(g: GGUFFile) -> Optional[dict]:
    """The BPE tokenizer stored in the file as a tokenizer.json-shaped dict."""
    m = g.metadata
    toks, merges = m.get("tokenizer.ggml.tokens"), m.get("tokenizer.ggml.merges")
    kind = m.get("tokenizer.ggml.model")
    types = m.get("tokenizer.ggml.token_type") or [1] * len(toks or [])
    if toks and kind in ("llama", "gemma4"):
        # SentencePiece-style pieces: spaces as U+2581 (one prepended unless the file says otherwise), byte fallback pieces
        # <0xNN>; "llama" files carry scores and no merge list, "gemma4" files carry merges and add no space prefix
        prefix = bool(m.get("tokenizer.ggml.add_space_prefix", kind == "llama"))
        if kind == "gemma4" and prefix:
            raise ValueError("gemma4 tokenizer.ggml.add_space_prefix=true is unsupported")
        norm = [{"type": "Prepend", "prepend": "\u2581"}] if prefix else []
        norm.append({"type": "Replace", "pattern": {"String": " "}, "content": "\u2581"})
        unk = m.get("tokenizer.ggml.unknown_token_id")
        model = {"type": "BPE", "vocab": {t: i for i, t in enumerate(toks)}, "merges": list(merges or []), "byte_fallback": True,
                 "unk_token": toks[int(unk)] if unk is not None and 0 <= int(unk) < len(toks) else "<unk>"}
        if not merges:
            model["scores"] = [float(v) for v in (m.get("tokenizer.ggml.scores") or [])]
        added = [{"id": i, "content": t, "special": True} for i, (t, ty) in enumerate(zip(toks, types)) if ty in (3, 4)]
        return {"added_tokens": added, "normalizer": {"type": "Sequence", "normalizers": norm}, "model": model}
    if not toks or merges is None or kind not in ("gpt2", "bpe"):
        return None
    added = [{"id": i, "content": t, "special": True} for i, (t, ty) in enumerate(zip(toks, types)) if ty in (3, 4)]
    return {"added_tokens": added, "normalizer": {"type": "NFC"},
            "model": {"type": "BPE", "vocab": {t: i for i, t in enumerate(toks)}, "merges": merges}}


NATIVE_TYPES = (2, 8, 12, 13, 14, 20, 23)       # block types the raw-block kernels serve (csrc/kernels/gemv_gguf.cu)


def native_ok(g: GGUFFile, cfg) -> bool:
    """Every projection of every layer is stored in a block type the raw-block kernels serve."""
    for i in range(cfg.num_hidden_layers):
        for stem in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down"):
            t = g.tensors.get(f"blk.{i}.{stem}.weight")
            if t is None or t[1] not in NATIVE_TYPES:
                return False
    return True


def tokenizer_config_from_gguf(g: GGUFFile) -> dict:
    """The ``tokenizer_config.json`` keys the front end reads: bos / eos token texts and whether prompts start with BOS."""
    m = g.metadata
    toks = m.get("tokenizer.ggml.tokens") or []
    out = {}
    for key, name in (("tokenizer.ggml.bos_token_id", "bos_token"), ("tokenizer.ggml.eos_token_id", "eos_token")):
        i = m.get(key)
        if i is not None and 0 <= int(i) < len(toks):
            out[name] = toks[int(i)]
    if "tokenizer.ggml.add_bos_token" in m:
        out["add_bos_token"] = bool(m["tokenizer.ggml.add_bos_token"])
    if isinstance(m.get("tokenizer.chat_template"), str):
        out["chat_template"] = m["tokenizer.chat_template"]
    return out
