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


def state_dict_from_gguf(g: GGUFFile) -> dict[str, torch.Tensor]:
    """Every tensor with a known HF name, dequantized to fp32."""
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
    if not toks or merges is None or m.get("tokenizer.ggml.model") not in ("gpt2", "bpe"):
        return None
    types = m.get("tokenizer.ggml.token_type") or [1] * len(toks)
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
