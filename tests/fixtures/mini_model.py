"""Synthetic HF checkpoints for tests: a real ``config.json`` + ``model.safetensors`` (+ optional
GPTQ triples, + a trained byte-level BPE ``tokenizer.json``) with random, never-zero weights -- the
role of the reference's tools/mini_model.hpp:18-110."""
from __future__ import annotations

import json
from pathlib import Path

import torch

from grimoire_b200.formats import gptq
from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.formats.safetensors_io import save_file
from grimoire_b200.models.config import ModelConfig
from grimoire_b200.models.synthetic import random_hybrid_state_dict, random_mtp_state_dict, random_state_dict

_PROJ = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def write_checkpoint(path: Path, cfg: ModelConfig, seed: int = 0, quant: str = "bf16", tokenizer: bool = False, shards: int = 1,
                     mtp: bool = False):
    path.mkdir(parents=True, exist_ok=True)
    sd = random_state_dict(cfg, seed)
    if mtp:
        sd.update(random_mtp_state_dict(cfg, seed))
    out = {}
    for name, w in sd.items():
        is_proj = any(name.endswith(p + ".weight") for p in _PROJ)
        if quant == "gptq" and is_proj:
            qw = quantize(w, Fmt.INT4, group=cfg.quant_group)
            a, b, c = gptq.gptq_pack(qw)
            base = name[: -len(".weight")]
            out[base + ".qweight"], out[base + ".qzeros"], out[base + ".scales"] = a, b, c
            out[base + ".g_idx"] = (torch.arange(qw.K) // cfg.quant_group).to(torch.int32)
        else:
            out[name] = w.bfloat16()
    hf = {"model_type": "qwen3", "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_hidden_layers,
          "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads,
          "head_dim": cfg.head_dim, "vocab_size": cfg.vocab_size, "intermediate_size": cfg.intermediate_size,
          "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta, "tie_word_embeddings": cfg.tie_word_embeddings,
          "qk_norm": cfg.qk_norm, "mtp_num_hidden_layers": 1 if mtp else 0}
    if quant == "gptq":
        hf["quantization_config"] = {"quant_method": "gptq", "bits": 4, "group_size": cfg.quant_group, "sym": False}
    (path / "config.json").write_text(json.dumps(hf))
    if shards == 1:
        save_file(out, path / "model.safetensors", {"format": "pt"})
    else:
        names = list(out)
        wm = {}
        for s in range(shards):
            part = {n: out[n] for n in names[s::shards]}
            fn = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
            save_file(part, path / fn)
            wm.update({n: fn for n in part})
        (path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))
    if tokenizer:
        write_tokenizer(path, cfg.vocab_size)
    return sd


def write_hybrid_checkpoint(path: Path, cfg: ModelConfig, seed: int = 0, fused_experts: bool = False, mtp: bool = False):
    """A checkpoint of the hybrid family (Gated DeltaNet / gated or plain attention; MoE with or without a shared expert, or a
    dense FFN) under the HF names of that family."""
    path.mkdir(parents=True, exist_ok=True)
    sd = random_hybrid_state_dict(cfg, seed, fused_experts=fused_experts, mtp=mtp)
    hf = {"mtp_num_hidden_layers": 1 if mtp else 0, "model_type": cfg.model_type, "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_hidden_layers,
          "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
          "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_norm_eps, "rope_theta": cfg.rope_theta,
          "partial_rotary_factor": cfg.partial_rotary_factor, "tie_word_embeddings": cfg.tie_word_embeddings,
          "layer_types": ["linear_attention" if t != "full_attention" else "full_attention" for t in cfg.layer_types],
          "linear_num_key_heads": cfg.linear_num_key_heads, "linear_num_value_heads": cfg.linear_num_value_heads,
          "linear_key_head_dim": cfg.linear_key_head_dim, "linear_value_head_dim": cfg.linear_value_head_dim,
          "linear_conv_kernel_dim": cfg.linear_conv_kernel_dim, "num_experts": cfg.num_experts,
          "num_experts_per_tok": cfg.num_experts_per_tok, "moe_intermediate_size": cfg.moe_intermediate_size,
          "shared_expert_intermediate_size": cfg.shared_expert_intermediate_size, "norm_topk_prob": cfg.norm_topk_prob,
          "intermediate_size": cfg.intermediate_size, "attn_output_gate": cfg.attn_output_gate, "qk_norm": cfg.qk_norm,
          "norm_zero_centered": cfg.norm_zero_centered}
    if cfg.mlp_only_layers or cfg.decoder_sparse_step != 1:
        hf.update({"mlp_only_layers": cfg.mlp_only_layers, "decoder_sparse_step": cfg.decoder_sparse_step})
    if cfg.is_k2:
        hf.update({"layernorm_num_groups": cfg.norm_groups, "attention_gate_func": "softplus" if cfg.attn_gate_proj == "softplus" else "",
                   "router_score_func": "sigmoid" if cfg.router_sigmoid else "softmax", "router_scaling_factor": cfg.router_scale,
                   "num_shared_experts": cfg.num_shared_experts, "mova_num_experts": cfg.mova_experts,
                   "mova_num_experts_per_tok": cfg.mova_top_k, "mlp_only_layers": cfg.mlp_only_layers,
                   "decoder_sparse_step": cfg.decoder_sparse_step, "query_key_norm": cfg.qk_norm, "moe_gate_bias": True})
        hf.pop("layer_types")
    (path / "config.json").write_text(json.dumps(hf))
    save_file({k: v.bfloat16() for k, v in sd.items()}, path / "model.safetensors", {"format": "pt"})
    return sd


def write_tokenizer(path: Path, vocab_size: int):
    from tokenizers import Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, trainers

    pat = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
    tok = Tokenizer(models.BPE())
    tok.normalizer = normalizers.NFC()
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated", invert=False),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    tr = trainers.BpeTrainer(vocab_size=min(vocab_size, 600), show_progress=False, initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                             special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>", "<think>", "</think>", "<tool_call>", "</tool_call>"])
    corpus = ["the quick brown fox jumps over the lazy dog", "hello world, how are you today?", "def f(x):\n    return x + 1\n",
              "user assistant system tool weather in Paris is sunny"] * 8
    tok.train_from_iterator(corpus, tr)
    tok.save(str(path / "tokenizer.json"))
    (path / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>"}))


def write_qwen4_exp_checkpoint(path: Path, cfg: ModelConfig, seed: int = 0):
    """A Qwen4-Exp checkpoint under the family's names: nested ``text_config`` with the hyper-connection, n-gram and indexer
    keys (1-based ``ple_layer_ids``, ``eos_token_id`` as a list the way Qwen configs write it)."""
    from grimoire_b200.models.synthetic import random_qwen4_exp_state_dict

    path.mkdir(parents=True, exist_ok=True)
    sd = random_qwen4_exp_state_dict(cfg, seed)
    tc = {"model_type": "qwen4_exp_text", "hidden_size": cfg.hidden_size, "num_hidden_layers": cfg.num_hidden_layers,
          "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
          "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.rms_norm_eps,
          "rope_parameters": {"rope_theta": cfg.rope_theta, "partial_rotary_factor": cfg.partial_rotary_factor},
          "layer_types": ["linear_attention" if t != "full_attention" else "qsa_attention" for t in cfg.layer_types],
          "linear_num_key_heads": cfg.linear_num_key_heads, "linear_num_value_heads": cfg.linear_num_value_heads,
          "linear_key_head_dim": cfg.linear_key_head_dim, "linear_value_head_dim": cfg.linear_value_head_dim,
          "linear_conv_kernel_dim": cfg.linear_conv_kernel_dim, "num_experts": cfg.num_experts,
          "num_experts_per_tok": cfg.num_experts_per_tok, "moe_intermediate_size": cfg.moe_intermediate_size,
          "shared_expert_intermediate_size": cfg.shared_expert_intermediate_size, "norm_topk_prob": cfg.norm_topk_prob,
          "intermediate_size": cfg.intermediate_size, "hc_count": cfg.hc_count, "hc_lowrank": cfg.hc_lowrank,
          "ple_layer_ids": cfg.ple_layer_ids, "ple_embed_dim": cfg.ple_embed_dim, "ple_conv_kernel_size": cfg.ple_conv_kernel_size,
          "ngram_size": cfg.ngram_size, "heads_per_ngram": cfg.heads_per_ngram, "ngram_vocab_size_base": cfg.ngram_vocab_size_base,
          "seed": cfg.ngram_seed, "eos_token_id": [cfg.eos_token_id, cfg.eos_token_id + 1], "indexer_n_heads": cfg.indexer_n_heads,
          "indexer_kv_heads": 1, "indexer_head_dim": cfg.indexer_head_dim, "indexer_budget": cfg.indexer_budget,
          "indexer_compress_ratio": cfg.indexer_compress_ratio}
    (path / "config.json").write_text(json.dumps({"model_type": "qwen4_exp", "tie_word_embeddings": cfg.tie_word_embeddings, "text_config": tc}))
    save_file({k: v.bfloat16() for k, v in sd.items()}, path / "model.safetensors", {"format": "pt"})
    return sd
