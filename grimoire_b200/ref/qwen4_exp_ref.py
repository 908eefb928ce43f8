"""Host oracles of the three mechanisms the Qwen4-Exp family layers on the hybrid decoder (include/b70/qwen4_exp.hpp;
ref/qwen4_exp_*.py): HyperConnections, Qwen sparse attention and the per-layer n-gram embedding.

**HyperConnections.**  The residual is ``hc`` streams wide ([hc * H]).  A block sees one H-wide input from ``hc_mix`` and
its output is put back into every stream by ``hc_combine``::

    normed = per-stream RMSNorm(hyper) * (1 + w)                    (each stream on its own variance; w spans hc * H)
    mix:     g = silu(W_down normed / hc);  u = sigmoid(W_up g);  out[h] = mean_c(u[c][h] * normed[c][h])
    combine: inj[c] = 2 sigmoid((W_inj normed)[c] / hc);  out[c][h] = hyper[c][h] + block[h] * inj[c]

The division by hc sits INSIDE the nonlinearities; combine adds to the UNNORMALISED streams.

**QSA.**  An MQA indexer scores mean-pooled key blocks -- relu per head, THEN summed over heads, THEN scaled by
1 / sqrt(d) --, the top budget / ratio visible blocks are kept (fewer visible blocks leave -1 holes), each block expands to
its ``ratio`` tokens (truncated to the budget, masked to the sequence), and the tokens of the block still being filled,
the query's own included, are appended unconditionally; attention runs over that gathered list.

**PLE.**  n-gram ids per head: ``offset[h] + (xor_i token[t - i] * multiplier[i]) mod size[h]`` where head h has order
h // heads_per_ngram + 2 (a predecessor takes part only while shift < order), positions before the sequence and everything
older than an EOS read as EOS, sizes are consecutive primes above the base, multipliers are odd splitmix64 values; a
per-stream gate ``sigmoid(sign(d) sqrt(max(|d|, 1e-6)))`` with d = <norm_k(key), norm_q(query)> / sqrt(H) scales the value
row into every stream, and a dilated depthwise convolution of the normed gated rows is added through SiLU on top of
``hidden + gated``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

_M64 = (1 << 64) - 1


# ------------------------------------------------------------------ HyperConnections
def hc_norm(x: torch.Tensor, w: torch.Tensor, hc: int, eps: float) -> torch.Tensor:
    rows, wide = x.shape
    xs = x.float().reshape(rows, hc, wide // hc)
    y = xs * torch.rsqrt(xs.pow(2).mean(-1, keepdim=True) + eps)
    return y.reshape(rows, wide) * (1.0 + w.float())


def hc_mix(normed: torch.Tensor, down: torch.Tensor, up: torch.Tensor, hc: int) -> torch.Tensor:
    """normed [rows][hc * H]; down [lowrank][hc * H]; up [hc * H][lowrank] -> block input [rows][H]."""
    g = F.silu(normed.float() @ down.float().t() / hc)
    u = torch.sigmoid(g @ up.float().t())
    rows, wide = normed.shape
    return (u * normed.float()).reshape(rows, hc, wide // hc).mean(1)


def hc_combine(hyper: torch.Tensor, normed: torch.Tensor, block: torch.Tensor, inj: torch.Tensor, hc: int) -> torch.Tensor:
    """hyper, normed [rows][hc * H]; block [rows][H]; inj [hc][hc * H] -> new streams [rows][hc * H]."""
    w = 2.0 * torch.sigmoid(normed.float() @ inj.float().t() / hc)                 # [rows][hc]
    rows, wide = hyper.shape
    return (hyper.float().reshape(rows, hc, wide // hc) + block.float()[:, None, :] * w[:, :, None]).reshape(rows, wide)


# ------------------------------------------------------------------ QSA
def qsa_index_logits(q: torch.Tensor, keys: torch.Tensor, visible: int) -> torch.Tensor:
    """q [heads][d] (one query row), keys [blocks][d] -> logits [blocks], -inf from ``visible`` on."""
    s = torch.relu(q.float() @ keys.float().t()).sum(0) / math.sqrt(q.shape[-1])
    s[max(0, visible):] = float("-inf")
    return s


def qsa_topk_blocks(logits: torch.Tensor, visible: int, topk: int) -> list[int]:
    vis = max(0, min(visible, logits.shape[0]))
    order = sorted(range(vis), key=lambda n: -float(logits[n]))           # stable: ties keep the lower block first
    out = order[:topk]
    return out + [-1] * (topk - len(out))


def qsa_expand_blocks(blocks, ratio: int, token_topk: int, seq_len: int, query_pos: int) -> list[int]:
    out = []
    for b in blocks:
        for r in range(ratio):
            if len(out) >= token_topk:
                break
            t = b * ratio + r if b >= 0 else -1
            out.append(t if 0 <= t < seq_len else -1)
    out += [-1] * (token_topk - len(out))
    visible = query_pos + 1
    tail_start = visible // ratio * ratio
    for i in range(ratio - 1):
        t = tail_start + i
        out.append(t if (i < visible - tail_start and t < seq_len) else -1)
    return out


def qsa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, idx, scale: float) -> torch.Tensor:
    """q [heads][d]; k, v [kv_heads][cap][d]; idx: gathered token list with -1 holes -> out [heads][d]."""
    heads, d = q.shape
    rep = heads // k.shape[0]
    take = torch.tensor([i for i in idx if i >= 0], dtype=torch.long)
    out = torch.zeros(heads, d)
    if take.numel() == 0:
        return out
    for h in range(heads):
        kk, vv = k[h // rep].float()[take], v[h // rep].float()[take]
        p = torch.softmax((kk @ q[h].float()) * scale, dim=0)
        out[h] = p @ vv
    return out


# ------------------------------------------------------------------ PLE
def splitmix64(v: int) -> int:
    v = (v + 0x9E3779B97F4A7C15) & _M64
    v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & _M64
    return v ^ (v >> 31)


def is_prime(v: int) -> bool:
    if v < 2:
        return False
    for p in (2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37):
        if v % p == 0:
            return v == p
    d, s = v - 1, 0
    while d % 2 == 0:
        d //= 2
        s += 1
    for a in (2, 325, 9375, 28178, 450775, 9780504, 1795265022):
        if a % v == 0:
            continue
        x = pow(a, d, v)
        if x in (1, v - 1):
            continue
        for _ in range(s - 1):
            x = x * x % v
            if x == v - 1:
                break
        else:
            return False
    return True


def nth_prime_after(start: int, count: int) -> int:
    prime = start
    for _ in range(count):
        c = prime + 1
        if c <= 2:
            prime = 2
            continue
        if c % 2 == 0:
            c += 1
        while not is_prime(c):
            c += 2
        prime = c
    return prime


def ngram_multipliers(ngram_size: int, vocab_size: int, seed: int, layer_id: int) -> list[int]:
    half = max(1, (((1 << 63) - 1) // vocab_size) // 2)
    base = (seed + 10007 * layer_id) & _M64
    return [2 * (splitmix64((base + 0x9E3779B97F4A7C15 * (i + 1)) & _M64) % half) + 1 for i in range(ngram_size)]


def ngram_vocab_layout(vocab_base: int, ngram_heads: int, layer_id: int):
    sizes, offsets, off = [], [], 0
    for h in range(ngram_heads):
        sizes.append(nth_prime_after(vocab_base - 1, layer_id * ngram_heads + h + 1))
        offsets.append(off)
        off += sizes[-1]
    return sizes, offsets, off


def _wrap64(v: int) -> int:
    """Two's-complement int64 (the reference multiplies and xors in int64)."""
    v &= _M64
    return v - (1 << 64) if v >= (1 << 63) else v


def ple_ngram_ids(token: int, hist, multipliers, sizes, offsets, context_len: int, heads_per_ngram: int, eos: int) -> list[int]:
    """``hist``: the preceding tokens, newest last.  One id per n-gram head."""
    out = []
    for h in range(len(sizes)):
        order = h // heads_per_ngram + 2
        mixed = _wrap64(token * multipliers[0])
        crossed = False
        for shift in range(1, context_len + 1):
            at = len(hist) - shift
            cand = hist[at] if at >= 0 else eos
            if crossed:
                cand = eos
            if cand == eos:
                crossed = True
            if order > shift:
                mixed = _wrap64(mixed ^ _wrap64(cand * multipliers[shift]))
        r = mixed % sizes[h] if sizes[h] else 0            # Python's % is already the non-negative remainder
        out.append(r + offsets[h])
    return out


def ple_gate(key: torch.Tensor, value: torch.Tensor, query: torch.Tensor, nk: torch.Tensor, nq: torch.Tensor, ncw: torch.Tensor,
             hc: int, eps: float):
    """key, query [rows][hc * H]; value [rows][H]; norm weights [hc * H] -> (gated, conv_in) [rows][hc * H]."""
    rows, wide = key.shape
    H = wide // hc
    norm = lambda t, w: (t.float().reshape(rows, hc, H) * torch.rsqrt(t.float().reshape(rows, hc, H).pow(2).mean(-1, keepdim=True) + eps)
                         * (1.0 + w.float().reshape(1, hc, H)))
    d = (norm(key, nk) * norm(query, nq)).sum(-1) / math.sqrt(H)                     # [rows][hc]
    g = torch.sigmoid(torch.sign(torch.where(d < 0, -torch.ones_like(d), torch.ones_like(d))) * torch.sqrt(torch.clamp(d.abs(), min=1e-6)))
    gated = g[:, :, None] * value.float()[:, None, :]
    conv_in = gated * torch.rsqrt(gated.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + ncw.float().reshape(1, hc, H))
    return gated.reshape(rows, wide), conv_in.reshape(rows, wide)


def ple_conv(conv_in: torch.Tensor, gated: torch.Tensor, hidden: torch.Tensor, w: torch.Tensor, dilation: int) -> torch.Tensor:
    """Rows are consecutive positions of one sequence from position 0.  w [channels][kernel].
    out[t] = hidden[t] + gated[t] + silu(sum_k w[k] * conv_in[t - (K - 1 - k) * dilation])."""
    T, C = conv_in.shape
    Kn = w.shape[1]
    acc = torch.zeros(T, C)
    for k in range(Kn):
        sh = (Kn - 1 - k) * dilation
        if sh < T:
            acc[sh:] += w.float()[:, k][None, :] * conv_in.float()[: T - sh]
    return hidden.float() + gated.float() + F.silu(acc)
