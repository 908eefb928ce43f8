"""Qwen4-Exp: the hybrid decoder (Gated DeltaNet + gated attention, MoE or dense FFN) under a multi-stream residual.

What differs from ``HybridModel`` is the structure AROUND the blocks (reference: forward_qwen4_exp,
src/grimoire.cpp:14269-14340 and its body; ref/qwen4_exp_nvidia_model.py:276-332, :489-590):

* the residual is ``hc_count`` streams wide; the embedding row is repeated into every stream;
* no input / post-attention layernorm: each block is wrapped by a hyper-connection whose grouped norm + gated mean makes
  the block's input (``mix``) and whose injection puts the block's output back into every stream (``combine``).  The
  reference defers a combine into the next connection's mix; combining at once is the same arithmetic;
* layers named by ``ple_layer_ids`` first add an n-gram embedding to the streams (ids from the last ``ngram_size - 1``
  tokens, rows from a host-resident table, per-stream gate, dilated depthwise convolution over the sequence);
* full-attention layers carry an indexer (``self_attn.indexer.*``): normed + roped index queries score mean-pooled,
  normed, roped key blocks; a query attends to the tokens of its top blocks plus the block still being filled.  While a
  sequence is shorter than the budget that list is every earlier token, and the layer runs the dense attention kernels;
* no final norm: the tail mixer's norm + gated mean is what the head reads.

The blocks themselves (projections, DeltaNet recurrence, paged int8 KV attention, expert GEMMs) are ``HybridModel``'s,
writing into a zeroed block-output buffer instead of the residual.  The family's own pieces run through
``ops/qwen4_exp.py`` (device kernels; host oracles on the CPU path); the indexer's norm / RoPE / pooling are elementwise
torch operations.  One GPU, no speculative verify blocks, no prefix-cache snapshots (the n-gram history and the
convolution tail are per conversation and only move forward).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..ops import core as K
from ..ops import hybrid as Hb
from ..ops import ref
from ..ops.linear import BF16Linear
from ..ops.qwen4_exp import HyperConnection, PleNgram, QsaSelector, ple_conv, ple_gate, qsa_gather_attention
from .config import ModelConfig
from .dense import RowBatch
from .hybrid import HybridBuffers, HybridModel, _DictSource


class _Q4Source:
    """A tensor source seen through the names ``HybridModel.from_checkpoint`` asks for: the family has no layernorms and no
    final norm, so those resolve to identity scales (never applied: this model's forward does not call them)."""

    def __init__(self, src, cfg: ModelConfig):
        self.src, self.cfg, self.prefix = src, cfg, src.prefix

    def plain(self, name: str):
        if name.endswith(("input_layernorm.weight", "post_attention_layernorm.weight")) or name == self.prefix + "norm.weight":
            return torch.zeros(self.cfg.hidden_size)
        return self.src.plain(name)

    def linear(self, name: str):
        return self.src.linear(name)

    def tensor(self, name: str):
        return self.src.tensor(name)

    def embedding(self):
        return self.src.embedding()


@dataclasses.dataclass
class _Ple:
    ngram: PleNgram
    key_proj: BF16Linear
    value_proj: BF16Linear
    nk: torch.Tensor
    nq: torch.Tensor
    ncw: torch.Tensor
    conv_w: torch.Tensor            # fp32 [hc * H][kernel]
    dilation: int
    tail_rows: int                  # (kernel - 1) * dilation rows of convolution input kept per conversation
    tails: dict                     # slot -> (next position, fp32 [tail_rows][hc * H])


@dataclasses.dataclass
class _Indexer:
    proj: BF16Linear                # [(heads + 1) * d][H]: index queries | one raw index key
    qn: torch.Tensor
    kn: torch.Tensor
    raw: dict                       # slot -> bf16 [cap][d] raw keys by position
    pooled: dict                    # slot -> bf16 [cap / ratio][d] normed, roped means of complete blocks


@dataclasses.dataclass
class _Extra:
    attn_hc: HyperConnection
    mlp_hc: HyperConnection
    indexer: Optional[_Indexer] = None
    ple: Optional[_Ple] = None


def _dense(t):
    return t.dequant() if hasattr(t, "dequant") else t.float()


class Qwen4ExpBuffers(HybridBuffers):
    def __init__(self, m: "Qwen4ExpModel", max_rows: int, max_logit_rows: int, dense_kv_tokens: int = 0):
        super().__init__(m, max_rows, max_logit_rows, dense_kv_tokens)
        cfg = m.cfg
        self.hyper = torch.zeros(max_rows, cfg.hc_count * cfg.hidden_size, dtype=torch.float32, device=m.device)
        self.hyper_sel = torch.zeros(max_logit_rows, cfg.hc_count * cfg.hidden_size, dtype=torch.float32, device=m.device)


class Qwen4ExpModel(HybridModel):
    graph_safe = False              # n-gram ids are made on the host from the step's tokens: no captured decode graph

    def __init__(self, cfg: ModelConfig, device, workspace=None, max_slots: int = 8, proj: Optional[str] = None):
        super().__init__(cfg, device, workspace, max_slots, proj)
        self.supports_verify_rows = False
        self.extra: list[_Extra] = []
        self.final_mixer: Optional[HyperConnection] = None
        self._scratch: Optional[HyperConnection] = None
        self._hist: dict[int, list[int]] = {}          # slot -> the conversation's tokens so far
        self.selector = None
        if cfg.indexer_n_heads:
            self.selector = QsaSelector(cfg.indexer_n_heads, cfg.indexer_head_dim, cfg.indexer_budget, cfg.indexer_compress_ratio, self.device)
            if cfg.rot_dim > cfg.indexer_head_dim:
                raise ValueError("the indexer's head is narrower than the rotary part of the attention head")
        self._qk = self._qv = None                     # dense bf16 K / V of one conversation for the gathered attention

    # ------------------------------------------------------------------------------------------ loading
    @staticmethod
    def from_checkpoint(path, device, max_slots: int = 8, proj: Optional[str] = None, **_) -> "Qwen4ExpModel":
        """Load by the family's tensor names (src/qwen35_loader.cpp:1060-1145): the hybrid decoder's blocks, plus per layer
        ``{attn,mlp}_hyper_connection.{hc_norm, input_mix_weight_down, input_mix_weight_up, block_inject_weight}``, on
        attention layers ``self_attn.indexer.{index_qk_proj, q_layernorm, k_layernorm}``, on n-gram layers
        ``ple.{key_proj, value_proj, conv1d, norm_key, norm_query, norm_conv, ple_embedding.ngram_embedding}``, and the tail
        ``hyper_connection_mixer.{hc_norm, input_mix_weight_down, input_mix_weight_up}``."""
        from ..formats.checkpoint import Checkpoint

        ck = Checkpoint(path) if isinstance(path, (str, bytes)) or hasattr(path, "__fspath__") else path
        cfg = ck.cfg
        m = HybridModel.from_checkpoint(_Q4Source(ck, cfg), device, max_slots=max_slots, proj=proj, model_cls=Qwen4ExpModel)
        hc, eps, dev = cfg.hc_count, cfg.rms_norm_eps, m.device

        def need(v, name):
            if v is None:
                raise KeyError(f"checkpoint has no tensor for {name}")
            return v

        def connection(prefix: str, inject: bool) -> HyperConnection:
            w = lambda k: _dense(need(ck.linear(prefix + k), prefix + k))
            c = HyperConnection(need(ck.plain(prefix + "hc_norm.weight"), prefix + "hc_norm").float(), w("input_mix_weight_down"),
                                w("input_mix_weight_up"), w("block_inject_weight") if inject else None, hc, eps, dev, max_rows=1,
                                scratch=m._scratch)
            if m._scratch is None:
                m._scratch = c
            return c

        ple_ids = sorted(set(cfg.ple_layer_ids))
        for i in range(cfg.num_hidden_layers):
            p = f"{ck.prefix}layers.{i}."
            x = _Extra(connection(p + "attn_hyper_connection.", True), connection(p + "mlp_hyper_connection.", True))
            if cfg.is_attention_layer(i) and cfg.indexer_n_heads:
                ix = p + "self_attn.indexer."
                x.indexer = _Indexer(BF16Linear(_dense(need(ck.linear(ix + "index_qk_proj"), ix + "index_qk_proj")), dev, f"L{i}.index_qk"),
                                     need(ck.plain(ix + "q_layernorm.weight"), ix + "q_layernorm").float().to(dev),
                                     need(ck.plain(ix + "k_layernorm.weight"), ix + "k_layernorm").float().to(dev), {}, {})
            if (i + 1) in ple_ids:
                pl = p + "ple."
                table = need(ck.plain(pl + "ple_embedding.ngram_embedding.weight"), pl + "ple_embedding.ngram_embedding")
                conv = need(ck.plain(pl + "conv1d.weight"), pl + "conv1d").float()
                conv = conv.reshape(conv.shape[0], -1).to(dev).contiguous()
                f32 = lambda k: need(ck.plain(pl + k + ".weight"), pl + k).float().to(dev).contiguous()
                x.ple = _Ple(PleNgram(table.bfloat16(), cfg.ngram_vocab_size_base, cfg.vocab_size, cfg.ngram_size, cfg.heads_per_ngram,
                                      cfg.ngram_seed, ple_ids.index(i + 1), cfg.eos_token_id, dev),
                             BF16Linear(_dense(need(ck.linear(pl + "key_proj"), pl + "key_proj")), dev, f"L{i}.ple.key"),
                             BF16Linear(_dense(need(ck.linear(pl + "value_proj"), pl + "value_proj")), dev, f"L{i}.ple.value"),
                             f32("norm_key"), f32("norm_query"), f32("norm_conv"), conv, cfg.ngram_size,
                             (conv.shape[1] - 1) * cfg.ngram_size, {})
            m.extra.append(x)
        m.final_mixer = connection(ck.prefix + "hyper_connection_mixer.", False)
        return m

    @staticmethod
    def random(cfg: ModelConfig, device, seed: int = 0, max_slots: int = 8, **_) -> "Qwen4ExpModel":
        from .synthetic import random_qwen4_exp_state_dict

        return Qwen4ExpModel.from_checkpoint(_DictSource(cfg, random_qwen4_exp_state_dict(cfg, seed)), device, max_slots=max_slots)

    def make_buffers(self, max_rows: int, max_logit_rows: int, dense_kv_tokens: int = 0) -> Qwen4ExpBuffers:
        return Qwen4ExpBuffers(self, max_rows, max_logit_rows, dense_kv_tokens)

    def weight_bytes(self) -> int:
        n = super().weight_bytes()
        for x in self.extra + [_Extra(self.final_mixer, self.final_mixer)]:
            for c in {id(x.attn_hc): x.attn_hc, id(x.mlp_hc): x.mlp_hc}.values():
                n += c.down.nbytes() + c.up.nbytes() + (c.inj.nbytes() if c.inj is not None else 0)
            if x.indexer is not None:
                n += x.indexer.proj.nbytes()
            if x.ple is not None:
                n += x.ple.key_proj.nbytes() + x.ple.value_proj.nbytes()         # the n-gram table stays in host memory
        return n

    # ------------------------------------------------------------------------------------------ per-conversation state
    def reset_slot(self, slot: int) -> None:
        super().reset_slot(slot)
        self._hist.pop(slot, None)
        for x in self.extra:
            if x.ple is not None:
                x.ple.tails.pop(slot, None)
            if x.indexer is not None:
                x.indexer.raw.pop(slot, None)
                x.indexer.pooled.pop(slot, None)

    def snapshot_slot(self, slot: int):
        raise NotImplementedError("prefix-cache snapshots of this family are not built (n-gram history and convolution tails)")

    def begin_verify(self, *a, **k):
        raise NotImplementedError("this model scores one row of a conversation per step")

    def _ensure_scratch(self, rows: int) -> None:
        s = self._scratch
        if s.max_rows >= rows:
            return
        mk = lambda *sh, dt: torch.zeros(*sh, dtype=dt, device=self.device)
        low8 = (s.low + 7) // 8 * 8
        s.normed_f, s.normed_b = mk(rows, s.wide, dt=torch.float32), mk(rows, s.wide, dt=torch.bfloat16)
        s.g_f, s.g_b, s.u = mk(rows, low8, dt=torch.float32), mk(rows, low8, dt=torch.bfloat16), mk(rows, s.wide, dt=torch.float32)
        s.injl, s.max_rows = mk(rows, 8, dt=torch.float32), rows
        for c in [self.final_mixer] + [c for x in self.extra for c in (x.attn_hc, x.mlp_hc)]:
            for name in ("normed_f", "normed_b", "g_f", "g_b", "u", "injl", "max_rows"):
                setattr(c, name, getattr(s, name))

    @staticmethod
    def _grown(store: dict, slot: int, rows: int, width: int, dtype, device) -> torch.Tensor:
        t = store.get(slot)
        if t is None or t.shape[0] < rows:
            n = max(64, 1 << (max(rows, 1) - 1).bit_length())
            new = torch.zeros(n, width, dtype=dtype, device=device)
            if t is not None:
                new[: t.shape[0]].copy_(t)
            store[slot] = t = new
        return t

    # ------------------------------------------------------------------------------------------ family pieces
    def _ple_add(self, P: _Ple, hyper: torch.Tensor, runs, tokens) -> None:
        """hyper rows += the gated n-gram embedding and its dilated convolution, run by run (one conversation each)."""
        cfg = self.cfg
        ctx = cfg.ngram_size - 1
        for slot, row0, n, pos0 in runs:
            hist = self._hist[slot]
            ids = P.ngram.ids(tokens[row0: row0 + n], hist[max(0, pos0 - ctx): pos0])
            emb = P.ngram.gather(ids).to(torch.bfloat16)
            key = torch.empty(n, P.key_proj.N, dtype=torch.float32, device=self.device)
            val = torch.empty(n, P.value_proj.N, dtype=torch.float32, device=self.device)
            P.key_proj(emb, key, "f32")
            P.value_proj(emb, val, "f32")
            rows = hyper[row0: row0 + n]
            gated, conv_in = ple_gate(key.bfloat16().float(), val.bfloat16().float(), rows.contiguous(), P.nk, P.nq, P.ncw, cfg.hc_count, cfg.rms_norm_eps)
            at, tail = P.tails.get(slot, (0, None))
            if pos0 == 0 or tail is None:
                tail = torch.zeros(P.tail_rows, rows.shape[1], dtype=torch.float32, device=self.device)
            elif at != pos0:
                raise RuntimeError("the n-gram layer's convolution tail only moves forward: rows must follow the conversation's last row")
            full = torch.cat([tail, conv_in], dim=0)
            rows.copy_(ple_conv(full, gated, rows.contiguous(), P.conv_w, P.dilation, t0=P.tail_rows))
            P.tails[slot] = (pos0 + n, full[full.shape[0] - P.tail_rows:].clone())

    def _gemma_norm_rope(self, v: torch.Tensor, w: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """v fp32 [rows][heads][d]: per-head RMSNorm with a (1 + w) scale, then the attention's RoPE at ``pos``."""
        cfg = self.cfg
        return ref.apply_rope(ref.head_rmsnorm(v, w, cfg.rms_norm_eps, 1.0), pos, self.inv_freq, cfg.rot_dim)

    def _index(self, X: _Indexer, x: torch.Tensor, runs, row_pos: torch.Tensor) -> torch.Tensor:
        """Index queries bf16 [M][heads][d] of the rows; the conversations' raw keys and the pooled keys of the blocks these
        rows complete are stored on the way."""
        cfg = self.cfg
        nh, d, r, M = cfg.indexer_n_heads, cfg.indexer_head_dim, cfg.indexer_compress_ratio, x.shape[0]
        pq = torch.empty(M, (nh + 1) * d, dtype=torch.float32, device=self.device)
        X.proj(x, pq, "f32")
        pq = pq.bfloat16()
        qi = self._gemma_norm_rope(pq[:, : nh * d].float().reshape(M, nh, d), X.qn, row_pos).bfloat16()
        for slot, row0, n, pos0 in runs:
            raw = self._grown(X.raw, slot, pos0 + n, d, torch.bfloat16, self.device)
            raw[pos0: pos0 + n].copy_(pq[row0: row0 + n, nh * d:])
            b0, b1 = pos0 // r, (pos0 + n) // r
            if b1 > b0:
                pooled = self._grown(X.pooled, slot, b1, d, torch.bfloat16, self.device)
                mean = raw[b0 * r: b1 * r].float().reshape(b1 - b0, r, d).mean(1)
                first = torch.arange(b0, b1, device=self.device) * r
                pooled[b0:b1].copy_(self._gemma_norm_rope(mean[:, None, :], X.kn, first)[:, 0].bfloat16())
        return qi

    def _sparse_attention(self, X: _Indexer, qi, q, gate, attn, kvl, block_table, runs) -> None:
        cfg, g = self.cfg, self.geom
        r = cfg.indexer_compress_ratio
        for slot, row0, n, pos0 in runs:
            T = pos0 + n
            if self._qk is None or self._qk.shape[0] < T:
                cap = max(256, 1 << (T - 1).bit_length())
                self._qk = torch.zeros(cap, g.Hkv * g.D, dtype=torch.bfloat16, device=self.device)
                self._qv = torch.zeros_like(self._qk)
            K.gather_kv_dense(kvl, block_table[slot], T, self._qk, self._qv)
            k3 = self._qk[:T].view(T, g.Hkv, g.D).transpose(0, 1).contiguous()
            v3 = self._qv[:T].view(T, g.Hkv, g.D).transpose(0, 1).contiguous()
            qpos = torch.arange(pos0, T, dtype=torch.int32, device=self.device)
            pooled = X.pooled.get(slot)
            pooled = pooled[: T // r] if pooled is not None else torch.zeros(0, cfg.indexer_head_dim, dtype=torch.bfloat16, device=self.device)
            idx = self.selector.select(qi[row0: row0 + n].contiguous(), pooled.contiguous(), qpos, qpos + 1)
            out = torch.empty(n, g.Hq, g.D, dtype=torch.bfloat16, device=self.device)
            qsa_gather_attention(q[row0: row0 + n].view(n, g.Hq, g.D).contiguous(), k3, v3, idx.to(self.device), out, g.scale)
            o = out.view(n, g.Hq * g.D).float()
            if gate is not None:
                o = o * torch.sigmoid(gate[row0: row0 + n].float())
            attn[row0: row0 + n].copy_(o.to(attn.dtype))

    # ------------------------------------------------------------------------------------------ forward
    def forward(self, rb: RowBatch, buf: Qwen4ExpBuffers, kv_layers, block_table) -> torch.Tensor:
        cfg, geom = self.cfg, self.geom
        M, H, hc, eps = rb.tokens.shape[0], cfg.hidden_size, cfg.hc_count, cfg.rms_norm_eps
        self._ensure_scratch(buf.max_rows)
        blk, x, hyper = buf.h[:M], buf.x[:M], buf.hyper[:M]
        K.embed(rb.tokens, self.embed, blk)
        hyper.view(M, hc, H).copy_(blk[:, None, :].expand(M, hc, H))            # the embedding row repeated into every stream
        prefill = rb.mode == "prefill"
        T = rb.q_pos0 + M
        tokens = [int(t) for t in rb.tokens.tolist()]
        if prefill:
            runs = [(int(rb.seq_slot), 0, M, int(rb.q_pos0))]
            run_slot = torch.tensor([rb.seq_slot], dtype=torch.int32, device=self.device)
            run_start = torch.zeros(1, dtype=torch.int32, device=self.device)
            run_len = torch.tensor([M], dtype=torch.int32, device=self.device)
            touched = torch.tensor([rb.seq_slot], dtype=torch.long, device=self.device)
        else:
            if rb.runs is not None:
                raise NotImplementedError("this model scores one row of a conversation per step")
            slots, pos = rb.row_seq.tolist(), rb.row_pos.tolist()
            runs = [(int(s), i, 1, int(p)) for i, (s, p) in enumerate(zip(slots, pos))]
            run_slot, run_start, run_len = rb.row_seq, buf.run_start[:M], buf.run_len[:M]
            touched = rb.row_seq.long()
        for slot, row0, n, pos0 in runs:
            hist = self._hist.setdefault(slot, [])
            if len(hist) < pos0:
                raise RuntimeError("rows of a conversation must arrive in order (the n-gram layers read its earlier tokens)")
            del hist[pos0:]
        sparse = self.selector is not None and max(p0 + n for _, _, n, p0 in runs) > cfg.indexer_budget
        for li, (L, X) in enumerate(zip(self.layers, self.extra)):
            if X.ple is not None:
                self._ple_add(X.ple, hyper, runs, tokens)
            X.attn_hc.mix(hyper, x)
            blk.zero_()
            if L.kind == "gdn":
                si = L.state_index
                L.in_qkv(x, buf.gdn_qkv[:M], "bf16")
                L.in_z(x, buf.gdn_z[:M], "bf16")
                L.in_ab(x, buf.gdn_ab[:M], "f32")
                Hb.conv4_silu(buf.gdn_qkv[:M], L.conv_w, self.ring[si], self.ring_tmp, rb.row_seq, rb.row_pos, buf.gdn_conv[:M], touched)
                Hb.gdn_runs(buf.gdn_conv[:M], buf.gdn_ab[:M], buf.gdn_z[:M], L.A_log, L.dt_bias, L.gdn_norm, eps, self.state[si],
                            run_slot, run_start, run_len, buf.gdn_o[:M], self.Hk, self.Hv, self.Dk, self.Dv, chunked=prefill and M >= 32)
                L.out_proj(buf.gdn_o[:M], blk, "add_f32")
            else:
                kvl = kv_layers[L.kv_index]
                qkv, q, attn = buf.qkv[:M], buf.q[:M], buf.attn[:M]
                gate = buf.gate[:M] if geom.q_gated else None
                L.qkv(x, qkv, "bf16")
                qi = self._index(X.indexer, x, runs, rb.row_pos) if X.indexer is not None else None
                if sparse and X.indexer is not None:
                    K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, gate)
                    self._sparse_attention(X.indexer, qi, q, gate, attn, kvl, block_table, runs)
                elif prefill:
                    if rb.q_pos0 > 0:
                        K.gather_kv_dense(kvl, block_table[rb.seq_slot], rb.q_pos0, buf.dense_k, buf.dense_v)
                    K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, gate,
                                   buf.dense_k[rb.q_pos0: T], buf.dense_v[rb.q_pos0: T])
                    K.flash_prefill(q, buf.dense_k, buf.dense_v, geom, attn, rb.q_pos0, gate)
                else:
                    K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, gate)
                    K.paged_decode_attn(q, rb.row_seq, rb.row_pos, block_table, kvl, geom, attn, rb.splits, self.ws, gate)
                L.o(attn, blk, "add_f32")
            X.attn_hc.combine(hyper, blk)
            X.mlp_hc.mix(hyper, x)
            blk.zero_()
            if L.moe is None:
                act = buf.act_d[:M]
                L.ffn_gu(x, act, "swiglu")
                L.ffn_down(act, blk, "add_f32")
            else:
                self._cur_layer = li
                self._moe(L, x, blk, buf, M, decode=not prefill)
            X.mlp_hc.combine(hyper, blk)
        for slot, row0, n, pos0 in runs:
            self._hist[slot].extend(tokens[row0: row0 + n])
        if rb.logits_rows is None:
            hsel, n = hyper, M
        else:
            n = rb.logits_rows.shape[0]
            hsel = buf.hyper_sel[:n]
            hsel.copy_(hyper.index_select(0, rb.logits_rows) if n != M else hyper)
        xf, logits = buf.xf[:n], buf.logits[:n]
        self.final_mixer.mix(hsel, xf)                  # the tail mixer's norm + gated mean stands where a final norm would
        self.lm_head(xf, logits, "f32")
        return logits
