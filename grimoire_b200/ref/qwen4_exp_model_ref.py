"""fp32 whole-model oracle of the Qwen4-Exp family: one sequence, every position at once, no caches.  It strings the
operator oracles of ``qwen4_exp_ref`` around the hybrid family's block oracles (``hybrid_reference``) the way the family's
model does (ref/qwen4_exp_nvidia_model.py:276-332, :489-590; forward_qwen4_exp, src/grimoire.cpp:14269 on): embedding
repeated into every stream, [n-gram embedding] -> mix -> block -> combine twice per layer, the tail mixer as final norm.
Sparse attention always goes through the selection (while a sequence is shorter than the budget the list is every earlier
token).  ``Qwen4ExpModel`` must agree with it up to its weight / KV quantisation."""
from __future__ import annotations

import torch

from ..models.config import ModelConfig
from ..ops import ref
from . import hybrid_reference as HR
from . import qwen4_exp_ref as R


def forward_logits(cfg: ModelConfig, sd: dict, tokens, weight_fn=None, trace: dict | None = None) -> torch.Tensor:
    """Logits [T][V].  ``weight_fn`` maps the blocks' projection matrices (a quantise-dequantise round trip); the family's
    own small projections are bf16.  ``trace`` collects the token lists the sparse attention used, per layer."""
    wf = weight_fn or (lambda w: w.float())
    bf = lambda t: t.bfloat16().float()
    pfx = "model.language_model." if any(k.startswith("model.language_model.") for k in sd) else "model."
    H, hc, eps = cfg.hidden_size, cfg.hc_count, cfg.rms_norm_eps
    T = len(tokens)
    pos = torch.arange(T)
    inv_freq = ref.rope_inv_freq(cfg.rot_dim, cfg.rope_theta)
    scale = cfg.softmax_scale or ref.softmax_scale(cfg.head_dim)
    hyper = bf(sd[pfx + "embed_tokens.weight"])[torch.tensor(tokens, dtype=torch.long)].repeat(1, hc)
    ple_ids = sorted(set(cfg.ple_layer_ids))
    nh, d, r, budget = cfg.indexer_n_heads, cfg.indexer_head_dim, cfg.indexer_compress_ratio, cfg.indexer_budget

    def wrapped(p: str, hyper: torch.Tensor, block) -> torch.Tensor:
        normed = bf(R.hc_norm(hyper, sd[p + "hc_norm.weight"], hc, eps))
        x = bf(R.hc_mix(normed, bf(sd[p + "input_mix_weight_down.weight"]), bf(sd[p + "input_mix_weight_up.weight"]), hc))
        return R.hc_combine(hyper, normed, block(x), bf(sd[p + "block_inject_weight.weight"]), hc)

    def ple(p: str, layer_id: int, hyper: torch.Tensor) -> torch.Tensor:
        heads = (cfg.ngram_size - 1) * cfg.heads_per_ngram
        mult = R.ngram_multipliers(cfg.ngram_size, cfg.vocab_size, cfg.ngram_seed, layer_id)
        sizes, offsets, _ = R.ngram_vocab_layout(cfg.ngram_vocab_size_base, heads, layer_id)
        ids = torch.tensor([R.ple_ngram_ids(int(tokens[t]), list(tokens[:t]), mult, sizes, offsets, cfg.ngram_size - 1, cfg.heads_per_ngram,
                                            cfg.eos_token_id) for t in range(T)], dtype=torch.long)
        emb = bf(sd[p + "ple_embedding.ngram_embedding.weight"])[ids.reshape(-1)].reshape(T, -1)
        key, value = bf(emb @ bf(sd[p + "key_proj.weight"]).t()), bf(emb @ bf(sd[p + "value_proj.weight"]).t())
        gated, conv_in = R.ple_gate(key, value, hyper, sd[p + "norm_key.weight"], sd[p + "norm_query.weight"], sd[p + "norm_conv.weight"], hc, eps)
        w = sd[p + "conv1d.weight"].float()
        return R.ple_conv(conv_in, gated, hyper, w.reshape(w.shape[0], -1), cfg.ngram_size)

    def sparse_attend(p: str, x: torch.Tensor, li: int):
        ix = p + "self_attn.indexer."
        pq = bf(x @ bf(sd[ix + "index_qk_proj.weight"]).t())
        norm_rope = lambda v, w, at: ref.apply_rope(ref.head_rmsnorm(v, w.float(), eps, 1.0), at, inv_freq, cfg.rot_dim)
        qi = bf(norm_rope(pq[:, : nh * d].reshape(T, nh, d), sd[ix + "q_layernorm.weight"], pos))
        nb = T // r
        mean = pq[: nb * r, nh * d:].reshape(nb, r, d).mean(1)
        pooled = bf(norm_rope(mean[:, None, :], sd[ix + "k_layernorm.weight"], torch.arange(nb) * r)[:, 0]) if nb else torch.zeros(0, d)

        def attend(q, k, v):
            k3, v3 = bf(k).transpose(0, 1), v.transpose(0, 1)
            out = torch.zeros(T, cfg.num_attention_heads, cfg.head_dim)
            for t in range(T):
                visible = (t + 1) // r
                lg = R.qsa_index_logits(qi[t], pooled, visible)
                idx = R.qsa_expand_blocks(R.qsa_topk_blocks(lg, visible, budget // r), r, budget, t + 1, t)
                if trace is not None:
                    trace.setdefault(li, []).append(idx)
                out[t] = R.qsa_attention(bf(q[t]), k3, v3, idx, scale)
            return out
        return attend

    for i in range(cfg.num_hidden_layers):
        p = f"{pfx}layers.{i}."
        if (i + 1) in ple_ids:
            hyper = ple(p + "ple.", ple_ids.index(i + 1), hyper)
        if cfg.is_attention_layer(i):
            block = lambda x, p=p, i=i: HR.attention_delta(cfg, sd, p, x, pos, inv_freq, scale, wf, attend=sparse_attend(p, x, i) if nh else None)
        else:
            block = lambda x, p=p: HR.gdn_delta(cfg, sd, p, x, wf)
        hyper = wrapped(p + "attn_hyper_connection.", hyper, block)
        hyper = wrapped(p + "mlp_hyper_connection.", hyper, lambda x, p=p, i=i: HR.ffn_delta(cfg, sd, p, i, x, wf))
    m = pfx + "hyper_connection_mixer."
    normed = bf(R.hc_norm(hyper, sd[m + "hc_norm.weight"], hc, eps))
    xf = bf(R.hc_mix(normed, bf(sd[m + "input_mix_weight_down.weight"]), bf(sd[m + "input_mix_weight_up.weight"]), hc))
    head = sd.get("lm_head.weight", sd[pfx + "embed_tokens.weight"])
    return xf @ wf(head).t()
