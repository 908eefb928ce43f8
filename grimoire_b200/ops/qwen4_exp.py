"""The Qwen4-Exp mechanisms as device operators (csrc/kernels/qwen4_exp_ops.cu; CPU path = ref/qwen4_exp_ref.py):

* ``HyperConnection``: the multi-stream residual's mix (streams -> one block input) and combine (block output -> every
  stream), with the low-rank down / up and the injection projections as bf16 linears;
* ``QsaSelector`` + ``qsa_gather_attention``: indexer logits over pooled key blocks, top blocks, token list with the
  unconditional tail, attention over the gathered list;
* ``PleNgram``: the n-gram id computation (exact 64-bit integer arithmetic on the host: prime table layout, splitmix
  multipliers, sticky EOS), the row gather from a pinned host table, the per-stream gate and the dilated convolution.

Reference: include/b70/qwen4_exp.hpp (host reference of the same operators), launch_hc_* / launch_qsa_* / launch_ple_*
(src/ops.cpp:2352-3630), flash_decode_qsa_list (src/attention.cpp:511)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native
from ..ref import qwen4_exp_ref as R
from .linear import BF16Linear

_c, _f = ctypes.c_int, ctypes.c_float


class HyperConnection:
    def __init__(self, norm_w: torch.Tensor, down: torch.Tensor, up: torch.Tensor, inj: Optional[torch.Tensor], hc: int, eps: float, device,
                 max_rows: int = 64, scratch: Optional["HyperConnection"] = None):
        """``inj`` None: a mixer that only reads the streams (the model's tail).  ``scratch``: another connection of the same
        geometry whose row buffers this one borrows -- a model runs mix -> block -> combine of one connection before the
        next one's mix, so one set of buffers serves them all."""
        self.device = torch.device(device)
        self.hc, self.eps = hc, eps
        self.wide = norm_w.shape[0]
        self.H, self.low = self.wide // hc, down.shape[0]
        self.norm_w = norm_w.to(device=self.device, dtype=torch.float32).contiguous()
        self.down, self.up = BF16Linear(down, self.device, "hc.down"), BF16Linear(up, self.device, "hc.up")
        self.inj = BF16Linear(inj, self.device, "hc.inj") if inj is not None else None
        if scratch is not None:
            if (scratch.wide, scratch.low, scratch.hc) != (self.wide, self.low, self.hc) or scratch.max_rows < max_rows:
                raise ValueError("borrowed hyper-connection buffers do not fit")
            for name in ("normed_f", "normed_b", "g_f", "g_b", "u", "injl"):
                setattr(self, name, getattr(scratch, name))
            self.max_rows = scratch.max_rows
            return
        mk = lambda *s, dt: torch.zeros(*s, dtype=dt, device=self.device)
        self.normed_f, self.normed_b = mk(max_rows, self.wide, dt=torch.float32), mk(max_rows, self.wide, dt=torch.bfloat16)
        self.g_f, self.g_b = mk(max_rows, (self.low + 7) // 8 * 8, dt=torch.float32), mk(max_rows, (self.low + 7) // 8 * 8, dt=torch.bfloat16)
        self.u = mk(max_rows, self.wide, dt=torch.float32)
        self.injl = mk(max_rows, 8, dt=torch.float32)
        self.max_rows = max_rows

    def mix(self, hyper: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """hyper fp32 [M][hc * H] -> out (bf16 or fp32) [M][H]; keeps the normalised streams for ``combine``."""
        M, hc = hyper.shape[0], self.hc
        nf, nb = self.normed_f[:M], self.normed_b[:M]
        if not hyper.is_cuda:
            nf.copy_(R.hc_norm(hyper, self.norm_w, hc, self.eps))
            nb.copy_(nf.to(nb.dtype))
            out.copy_(R.hc_mix(nb.float(), self.down.w.float(), self.up.w.float(), hc).to(out.dtype))
            return out
        lib = _native.cuda()
        _native.check(lib.grm_hc_norm(_native.ptr(hyper), _native.ptr(self.norm_w), _native.ptr(nf), _native.ptr(nb), _c(M), _c(self.H), _c(hc),
                                      _f(self.eps), _native.stream_ptr()), "hc_norm")
        gf, gb = self.g_f[:M, : self.low], self.g_b[:M, : self.low]
        self.down(nb, gf, "f32")
        _native.check(lib.grm_hc_lowrank_gate(_native.ptr(self.g_f[:M]), _native.ptr(self.g_b[:M]), ctypes.c_long(M * self.g_f.shape[1]), _c(hc),
                                              _native.stream_ptr()), "hc_lowrank_gate")
        u = self.u[:M]
        self.up(gb, u, "f32")
        bf = out.dtype == torch.bfloat16
        _native.check(lib.grm_hc_mix_finish(_native.ptr(u), _native.ptr(nf), _native.ptr(out) if bf else None, None if bf else _native.ptr(out),
                                            _c(M), _c(self.H), _c(hc), _native.stream_ptr()), "hc_mix_finish")
        return out

    def combine(self, hyper: torch.Tensor, block: torch.Tensor) -> torch.Tensor:
        """hyper (fp32, in place) += block (fp32 [M][H]) gated per stream by the injection of the normalised streams ``mix`` left."""
        M, hc = hyper.shape[0], self.hc
        if not hyper.is_cuda:
            hyper.copy_(R.hc_combine(hyper, self.normed_b[:M].float(), block, self.inj.w.float(), hc))
            return hyper
        injl = self.injl[:M, :hc]
        self.inj(self.normed_b[:M], injl, "f32")
        _native.check(_native.cuda().grm_hc_combine(_native.ptr(hyper), _native.ptr(block), _native.ptr(injl), _c(injl.stride(0)), _c(M), _c(self.H),
                                                    _c(hc), _native.stream_ptr()), "hc_combine")
        return hyper


class QsaSelector:
    """Token selection of Qwen sparse attention for decode rows of one sequence."""

    def __init__(self, heads: int, head_dim: int, budget: int, ratio: int, device):
        if budget % ratio:
            raise ValueError("the indexer budget must be a multiple of the compression ratio")
        self.heads, self.d, self.budget, self.ratio = heads, head_dim, budget, ratio
        self.block_topk = budget // ratio
        self.width = budget + ratio - 1
        self.device = torch.device(device)

    def select(self, q_idx: torch.Tensor, pooled_keys: torch.Tensor, query_pos: torch.Tensor, seq_len: torch.Tensor) -> torch.Tensor:
        """q_idx bf16 [rows][heads][d]; pooled_keys bf16 [blocks][d] (mean-pooled key blocks of the sequence); query_pos, seq_len
        int32 [rows] -> token list int32 [rows][budget + ratio - 1] with -1 holes."""
        rows, blocks = q_idx.shape[0], pooled_keys.shape[0]
        visible = torch.minimum((query_pos + 1) // self.ratio, seq_len // self.ratio).to(torch.int32)     # complete blocks only
        if not q_idx.is_cuda:
            out = []
            for r in range(rows):
                lg = R.qsa_index_logits(q_idx[r].float(), pooled_keys.float(), int(visible[r]))
                blk = R.qsa_topk_blocks(lg, int(visible[r]), self.block_topk)
                out.append(R.qsa_expand_blocks(blk, self.ratio, self.budget, int(seq_len[r]), int(query_pos[r])))
            return torch.tensor(out, dtype=torch.int32)
        lib = _native.cuda()
        logits = torch.empty(rows, blocks, dtype=torch.float32, device=self.device)
        _native.check(lib.grm_qsa_index_logits(_native.ptr(q_idx), _native.ptr(pooled_keys), _native.ptr(visible), _native.ptr(logits), _c(rows),
                                               _c(self.heads), _c(self.d), _c(blocks), _native.stream_ptr()), "qsa_index_logits")
        k = min(self.block_topk, blocks)
        # ties must go to the lower block (stable order): a tiny index-proportional penalty below the logits' resolution
        # would change values, so sort stably instead
        order = torch.sort(logits, dim=-1, descending=True, stable=True)
        blk = torch.full((rows, self.block_topk), -1, dtype=torch.int32, device=self.device)
        top = order.indices[:, :k].to(torch.int32)
        top = torch.where(torch.isinf(order.values[:, :k]), torch.full_like(top, -1), top)
        blk[:, :k] = top
        out = torch.empty(rows, self.width, dtype=torch.int32, device=self.device)
        _native.check(lib.grm_qsa_expand(_native.ptr(blk), _c(self.block_topk), _c(self.ratio), _c(self.budget), _native.ptr(seq_len),
                                         _native.ptr(query_pos), _native.ptr(out), _c(rows), _native.stream_ptr()), "qsa_expand")
        return out


def qsa_gather_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, idx: torch.Tensor, out: torch.Tensor, scale: float) -> torch.Tensor:
    """q bf16 [rows][heads][d]; k, v bf16 [kv_heads][cap][d]; idx int32 [rows][n] (-1 = hole) -> out bf16 [rows][heads][d]."""
    rows, heads, d = q.shape
    if not q.is_cuda:
        for r in range(rows):
            out[r].copy_(R.qsa_attention(q[r], k, v, idx[r].tolist(), scale).to(out.dtype))
        return out
    code = _native.cuda().grm_qsa_gather_attn(_native.ptr(q), _native.ptr(k), _native.ptr(v), _native.ptr(idx), _native.ptr(out), _c(rows), _c(heads),
                                              _c(k.shape[0]), _c(d), _c(k.shape[1]), _c(idx.shape[1]), _f(scale), _native.stream_ptr())
    _native.check(code, "qsa_gather_attn")
    return out


class PleNgram:
    """Per-layer n-gram embedding: ids on the host, rows from a host-resident table, gate and convolution on the device."""

    def __init__(self, table: torch.Tensor, vocab_base: int, vocab_size: int, ngram_size: int, heads_per_ngram: int, seed: int, layer_id: int,
                 eos: int, device):
        self.ngram_heads = (ngram_size - 1) * heads_per_ngram
        self.heads_per_ngram, self.context = heads_per_ngram, ngram_size - 1
        self.eos, self.device = eos, torch.device(device)
        self.mult = R.ngram_multipliers(ngram_size, vocab_size, seed, layer_id)
        self.sizes, self.offsets, self.total = R.ngram_vocab_layout(vocab_base, self.ngram_heads, layer_id)
        if table.shape[0] < self.total:
            raise ValueError(f"the n-gram table has {table.shape[0]} rows, the layout needs {self.total}")
        # the table stays in host memory (pinned when a GPU is present): only the rows of the current tokens are read
        self.table = table.pin_memory() if self.device.type == "cuda" and not table.is_pinned() else table

    def ids(self, tokens, history) -> torch.Tensor:
        """ids [len(tokens)][ngram_heads] for consecutive ``tokens`` that follow ``history`` (older tokens, newest last)."""
        hist = list(history)
        out = []
        for t in tokens:
            out.append(R.ple_ngram_ids(int(t), hist, self.mult, self.sizes, self.offsets, self.context, self.heads_per_ngram, self.eos))
            hist.append(int(t))
        return torch.tensor(out, dtype=torch.long)

    def gather(self, ids: torch.Tensor) -> torch.Tensor:
        """Rows of the table for ``ids`` -> [rows][heads * dim] on the device."""
        rows = self.table[ids.reshape(-1)].reshape(ids.shape[0], -1)
        return rows.to(self.device, non_blocking=True)


def ple_gate(key, value, query, nk, nq, ncw, hc: int, eps: float):
    """fp32 key, query [rows][hc * H], value [rows][H] -> (gated, conv_in) fp32 [rows][hc * H]."""
    if not key.is_cuda:
        return R.ple_gate(key, value, query, nk, nq, ncw, hc, eps)
    rows, wide = key.shape
    gated, conv_in = torch.empty_like(key), torch.empty_like(key)
    code = _native.cuda().grm_ple_gate(_native.ptr(key), _native.ptr(value), _native.ptr(query), _native.ptr(nk), _native.ptr(nq), _native.ptr(ncw),
                                       _native.ptr(gated), _native.ptr(conv_in), _c(rows), _c(wide // hc), _c(hc), _f(eps), _native.stream_ptr())
    _native.check(code, "ple_gate")
    return gated, conv_in


def ple_conv(conv_in: torch.Tensor, gated: torch.Tensor, hidden: torch.Tensor, w: torch.Tensor, dilation: int, t0: int = 0) -> torch.Tensor:
    """conv_in fp32 [t0 + T][C] (t0 rows of history first); gated, hidden fp32 [T][C]; w fp32 [C][K] -> out fp32 [T][C]."""
    T, C = gated.shape
    if not gated.is_cuda:
        full_g, full_h = torch.zeros(t0 + T, C), torch.zeros(t0 + T, C)
        full_g[t0:], full_h[t0:] = gated, hidden
        return R.ple_conv(conv_in, full_g, full_h, w, dilation)[t0:]
    out = torch.empty_like(gated)
    code = _native.cuda().grm_ple_conv(_native.ptr(conv_in), _native.ptr(gated), _native.ptr(hidden), _native.ptr(w), _native.ptr(out), _c(T), _c(t0),
                                       _c(C), _c(w.shape[1]), _c(dilation), _native.stream_ptr())
    _native.check(code, "ple_conv")
    return out
