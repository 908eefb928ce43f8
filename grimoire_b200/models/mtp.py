"""Multi-token-prediction (MTP) draft head and its drafter.

The head is the checkpoint's own one-layer predictor (reference: ``MtpHead`` grimoire.cpp:3507-3517,
``mtp_draft`` :15753-15963, ``mtp_warm`` / ``mtp_warm_rows`` :15672-15752): for a position i it takes
the target's last hidden state h_i and the token that followed, t_{i+1}, and predicts t_{i+2}:

    z   = fc([ rmsnorm_e(embed(t_{i+1})) ; rmsnorm_h(h_i) ])          (2H -> H)
    z   = one decoder layer (own KV cache layer, same paged pool, same block table)
    out = lm_head(rmsnorm(z))            (optionally only the first ``draft_vocab`` rows, :15920-15960)

Drafting K tokens chains the head on its own output hidden state.  The head's KV entry of a position
must come from the *target's* hidden state, so it is (re)filled from the target's rows during prefill
("warm") and after every accepted block ("catch-up"); entries written while drafting are provisional
and get overwritten.  All scratch comes from the target's activation buffers; the head only owns its
residual stream and the concatenated fc input.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from ..ops import core as K
from ..ops.linear import BF16Linear
from .dense import DenseModel, RowBatch


class MtpHead:
    def __init__(self, target, draft_vocab: int = 0):
        """``target``: a ``DenseModel``, or a ``HybridModel`` with a dense FFN (the 27B-style hybrid, whose draft layer is one
        gated full-attention layer with a dense FFN: the head reads only the target's residual rows, embedding and output
        head, and borrows the attention-side scratch the two buffer classes name alike)."""
        cfg = target.cfg
        if cfg.is_moe:
            raise ValueError("the draft head's layer carries a dense FFN: targets with an MoE FFN are not served")
        self.target, self.cfg, self.device = target, cfg, target.device
        self.inner = DenseModel(dataclasses.replace(cfg, num_hidden_layers=1, layer_types=[], mtp_num_hidden_layers=0), target.device,
                                workspace=target.ws)
        self.enorm = self.hnorm = self.final_norm = None
        self.fc = None
        self.head = None
        self.draft_vocab = draft_vocab or cfg.vocab_size
        self._extra: dict[int, tuple] = {}

    # ------------------------------------------------------------------------------------------
    def load(self, fc_w, enorm, hnorm, final_norm, layer_weights: dict, head_w=None) -> "MtpHead":
        """fc_w fp32 [H][2H]; layer_weights: the add_layer_from_dense arguments of the one layer;
        head_w: fp32 [draft_vocab][H] (None: share the target's lm_head)."""
        dev, H = self.device, self.cfg.hidden_size
        f32 = lambda t: t.to(device=dev, dtype=torch.float32).contiguous()
        self.enorm, self.hnorm, self.final_norm = f32(enorm), f32(hnorm), f32(final_norm)
        self.fc = self.inner._linear(self.inner._quant(fc_w), "mtp.fc")
        self.inner.add_layer_from_dense(**layer_weights)
        if head_w is not None:
            self.head = self.inner._linear(self.inner._quant(head_w), "mtp.lm_head")
            self.draft_vocab = head_w.shape[0]
        else:
            if getattr(self.target, "head_split", None) is not None:
                raise ValueError("the draft head shares the target's lm_head, which is split over the tensor-parallel ranks; "
                                 "attach the draft head before TensorParallel.split_head or set GRIMOIRE_TP_HEAD_SPLIT=0")
            self.head = self.target.lm_head
            self.draft_vocab = self.cfg.vocab_size
        return self

    @staticmethod
    def from_checkpoint(target: DenseModel, ck, draft_vocab: int = 0) -> "MtpHead":
        """The checkpoint's own draft head: ``mtp.fc.weight`` [H][2H], ``mtp.pre_fc_norm_embedding`` / ``_hidden`` /
        ``mtp.norm`` and the decoder layer ``mtp.layers.0.*`` (src/grimoire.cpp:8603-8618).  ``ck`` resolves tensors
        (formats.checkpoint.Checkpoint or the artifact adapter).  ``draft_vocab`` > 0 drafts over the first rows of the
        target's lm_head only (GRIMOIRE_MTP_DRAFT_VOCAB, :15920-15960)."""
        head = MtpHead(target, draft_vocab)
        p = "mtp.layers.0."

        def need(v, name):
            if v is None:
                raise KeyError(f"checkpoint has no {name}")
            return v

        lin = lambda k: need(ck.linear(p + k), p + k)
        lw = dict(wq=lin("self_attn.q_proj"), wk=lin("self_attn.k_proj"), wv=lin("self_attn.v_proj"), wo=lin("self_attn.o_proj"),
                  wg=lin("mlp.gate_proj"), wu=lin("mlp.up_proj"), wd=lin("mlp.down_proj"),
                  in_norm=need(ck.plain(p + "input_layernorm.weight"), p + "input_layernorm"),
                  post_norm=need(ck.plain(p + "post_attention_layernorm.weight"), p + "post_attention_layernorm"),
                  q_norm=ck.plain(p + "self_attn.q_norm.weight"), k_norm=ck.plain(p + "self_attn.k_norm.weight"))
        fc = need(ck.linear("mtp.fc"), "mtp.fc.weight")
        fc = fc.dequant() if hasattr(fc, "dequant") else fc
        head_w = None
        cfg = target.cfg
        if draft_vocab and 0 < draft_vocab < cfg.vocab_size:
            hw = ck.linear("lm_head") if not cfg.tie_word_embeddings else None
            hw = ck.embedding() if hw is None else (hw.dequant() if hasattr(hw, "dequant") else hw)
            head_w = hw[:draft_vocab].contiguous()
        return head.load(fc, need(ck.plain("mtp.pre_fc_norm_embedding.weight"), "mtp.pre_fc_norm_embedding"),
                         need(ck.plain("mtp.pre_fc_norm_hidden.weight"), "mtp.pre_fc_norm_hidden"),
                         need(ck.plain("mtp.norm.weight"), "mtp.norm"), lw, head_w)

    @staticmethod
    def random_from_target(target: DenseModel, seed: int = 0, noise: float = 0.01, draft_vocab: int = 0, std: float = 0.02,
                           gen_device=None) -> "MtpHead":
        """Synthetic head: the layer is the target's final layer (re-drawn from the same seeds as
        ``DenseModel.random``) plus Gaussian noise of standard deviation ``noise`` (relative to the weight
        scale ``std``), fc averages its two inputs, norms are the identity scale, and the output head is
        the first ``draft_vocab`` rows of the target's (re-drawn) lm_head."""
        cfg = target.cfg
        head = MtpHead(target, draft_vocab)
        gdev = torch.device(gen_device or target.device)
        g = torch.Generator(device=gdev)
        H, D = cfg.hidden_size, cfg.head_dim
        qrows = cfg.num_attention_heads * D * (2 if cfg.attn_output_gate else 1)

        def rnd(n, k, tag, extra=0.0):
            g.manual_seed(seed * 1000003 + tag)
            w = torch.randn(n, k, generator=g, device=gdev, dtype=torch.float32) * std
            if extra:
                g.manual_seed(seed * 1000003 + tag + 7777777)
                w = w + torch.randn(n, k, generator=g, device=gdev, dtype=torch.float32) * (extra * std)
            return w

        t = (cfg.num_hidden_layers - 1) * 16
        ones = torch.ones(H) if not cfg.norm_zero_centered else torch.zeros(H)
        lw = dict(wq=rnd(qrows, H, t + 1, noise), wk=rnd(cfg.kv_size, H, t + 2, noise), wv=rnd(cfg.kv_size, H, t + 3, noise),
                  wo=rnd(H, cfg.num_attention_heads * D, t + 4, noise), wg=rnd(cfg.intermediate_size, H, t + 5, noise),
                  wu=rnd(cfg.intermediate_size, H, t + 6, noise), wd=rnd(H, cfg.intermediate_size, t + 7, noise),
                  in_norm=ones, post_norm=ones, q_norm=torch.ones(D) if cfg.qk_norm else None,
                  k_norm=torch.ones(D) if cfg.qk_norm else None)
        eye = torch.eye(H, device=gdev) * 0.5
        fc_w = torch.cat([eye, eye], dim=1)
        head_w = None
        if draft_vocab and draft_vocab < cfg.vocab_size and not cfg.tie_word_embeddings:
            g.manual_seed(seed * 1000003 + 900002)
            # the same stream as the target's lm_head: its first rows are the first numbers drawn
            head_w = (torch.randn(cfg.vocab_size, H, generator=g, device=gdev, dtype=torch.float32) * std)[:draft_vocab].contiguous()
        return head.load(fc_w, ones, ones, ones, lw, head_w)

    def nbytes(self) -> int:
        L = self.inner.layers[0]
        n = self.fc.nbytes() + sum(l.nbytes() for l in (L.qkv, L.o, L.gate_up, L.down))
        return n + (self.head.nbytes() if self.head is not self.target.lm_head else 0)

    # ------------------------------------------------------------------------------------------
    def _bufs(self, buf):
        key = id(buf)
        if key not in self._extra:
            H, R = self.cfg.hidden_size, buf.max_rows
            mk = lambda *s, dt: torch.zeros(*s, dtype=dt, device=self.device)
            self._extra[key] = (mk(R, H, dt=torch.float32), mk(R, H, dt=torch.float32), mk(R, 2 * H, dt=torch.bfloat16))
        return self._extra[key]

    def forward(self, rb: RowBatch, hidden: torch.Tensor, buf, kvl, block_table, logits_rows: int = 0, flip: int = 0):
        """One head pass over the rows of ``rb`` with the matching target hidden states ``hidden`` fp32
        [M][H].  Returns (logits of the first ``logits_rows`` rows or None, the head's hidden states
        [M][H]).  ``flip`` picks which of the two residual buffers receives the result, so a chained
        draft can read the previous step's output while writing the next."""
        cfg, geom, L = self.cfg, self.inner.geom, self.inner.layers[0]
        M, H = rb.tokens.shape[0], cfg.hidden_size
        eps, off = cfg.rms_norm_eps, cfg.norm_offset
        hA, hB, catb = self._bufs(buf)
        h2, cat = (hB if flip else hA)[:M], catb[:M]
        x, qkv, q, attn = buf.x[:M], buf.qkv[:M], buf.q[:M], buf.attn[:M]
        act = (buf.act_d if hasattr(buf, "act_d") else buf.act)[:M]        # a hybrid target keeps its dense-FFN rows under act_d
        gate = buf.gate[:M] if buf.gate is not None else None
        K.embed(rb.tokens, self.target.embed, h2)
        K.add_rmsnorm(h2, self.enorm, cat[:, :H], eps, off)
        K.add_rmsnorm(hidden, self.hnorm, cat[:, H:], eps, off)
        self.fc(cat, h2, "f32")
        K.add_rmsnorm(h2, L.in_norm, x, eps, off)
        L.qkv(x, qkv, "bf16")
        if rb.mode == "prefill":
            T = rb.q_pos0 + M
            if rb.q_pos0 > 0:
                K.gather_kv_dense(kvl, block_table[rb.seq_slot], rb.q_pos0, buf.dense_k, buf.dense_v)
            K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inner.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, gate,
                           buf.dense_k[rb.q_pos0: T], buf.dense_v[rb.q_pos0: T])
            K.flash_prefill(q, buf.dense_k, buf.dense_v, geom, attn, rb.q_pos0, gate)
        else:
            K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inner.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, gate)
            K.paged_decode_attn(q, rb.row_seq, rb.row_pos, block_table, kvl, geom, attn, rb.splits, self.inner.ws, gate)
        L.o(attn, h2, "add_f32")
        K.add_rmsnorm(h2, L.post_norm, x, eps, off)
        L.gate_up(x, act, "swiglu")
        L.down(act, h2, "add_f32")
        logits = None
        if logits_rows:
            n = logits_rows
            xf, logits = buf.xf[:n], buf.logits[:n, : self.draft_vocab]
            K.add_rmsnorm(h2[:n], self.final_norm, xf, eps, off)
            self.head(xf, logits, "f32")
        return logits, h2


class MtpDrafter:
    """Drafter protocol (engine/generation.py) on top of an ``MtpHead`` attached to an ``Engine``."""

    def __init__(self, engine, head: MtpHead):
        self.engine, self.head = engine, head
        self.kvl = engine.kv.layers[-1]                 # the extra KV layer the engine allocated for the head
        self.pending: dict[int, tuple[int, torch.Tensor]] = {}      # slot -> (position, target hidden of that position)
        self.stats = {"draft_steps": 0, "warm_rows": 0, "catchup_rows": 0}
        dev = engine.device
        self._ids = torch.zeros(16, dtype=torch.int32, device=dev)
        self._drafts = torch.zeros(16, dtype=torch.int32, device=dev)
        engine.mtp = self
        engine.enable_speculation()

    # ---- prefill: fill the head's KV from the target's hidden states of the chunk ----
    def warm_chunk(self, seq, tokens_dev: torch.Tensor, done: int, m: int, pos0: int, buf, last: bool) -> None:
        eng = self.engine
        prev = self.pending.get(seq.slot)
        if done == 0 and prev is not None and prev[0] == pos0 - 1:
            # the prompt arrives in several prefill calls: the position the previous call left pending gets its
            # entry now that its next token (the first of this call) is known
            one = torch.full((1,), seq.slot, dtype=torch.int32, device=eng.device)
            rb1 = RowBatch(tokens_dev[:1], one, torch.full((1,), pos0 - 1, dtype=torch.int32, device=eng.device), mode="decode",
                           splits=K.decode_splits(pos0, 1, self.head.inner.geom.Hkv))
            self.head.forward(rb1, prev[1].unsqueeze(0), eng.decode_buf, self.kvl, eng.kv.table)
            self.stats["warm_rows"] += 1
        rows = m - 1 if last else m                      # the last prompt position has no next token yet
        hid = buf.h[:m]
        if last:
            self.pending[seq.slot] = (pos0 + m - 1, hid[m - 1].clone())
        if rows <= 0:
            return
        nxt = tokens_dev[done + 1: done + 1 + rows]
        pos = torch.arange(pos0, pos0 + rows, dtype=torch.int32, device=eng.device)
        rb = RowBatch(nxt, torch.full((rows,), seq.slot, dtype=torch.int32, device=eng.device), pos, mode="prefill", q_pos0=pos0,
                      seq_slot=seq.slot)
        self.head.forward(rb, hid[:rows], buf, self.kvl, eng.kv.table)
        self.stats["warm_rows"] += rows

    # ---- drafting ----
    def propose(self, engine, seq, last_token: int, depth: int) -> list[int]:
        p = self.pending.get(seq.slot)
        pos = seq.length - 1
        if p is None or p[0] != pos or depth <= 0:
            return []
        eng, dev = self.engine, self.engine.device
        depth = min(depth, 8)
        eng.kv.ensure(seq, seq.length + depth)
        hidden = p[1].unsqueeze(0)
        self._ids[:1].fill_(int(last_token))
        slot_t = torch.full((1,), seq.slot, dtype=torch.int32, device=dev)
        for j in range(depth):
            rp = torch.full((1,), pos + j, dtype=torch.int32, device=dev)
            rb = RowBatch(self._ids[:1], slot_t, rp, mode="decode", splits=K.decode_splits(pos + j + 1, 1, self.head.inner.geom.Hkv))
            logits, h2 = self.head.forward(rb, hidden, eng.decode_buf, self.kvl, eng.kv.table, logits_rows=1, flip=j & 1)
            K.argmax_rows(logits, self._ids[:1])
            self._drafts[j: j + 1].copy_(self._ids[:1])
            hidden = h2
            self.stats["draft_steps"] += 1
        return [int(v) for v in self._drafts[:depth].tolist()]

    # ---- after a committed block: provisional entries are replaced by ones made from target hiddens ----
    def observe(self, engine, seq, accepted_tokens, row0: int = 0) -> None:
        """``row0``: first row of this conversation's block inside the step that was just verified."""
        eng, dev = self.engine, self.engine.device
        keep = list(accepted_tokens)
        a = len(keep) - 1
        pos0 = seq.length - len(keep)
        hid = eng.decode_buf.h[row0:]
        if a > 0:
            toks = torch.tensor(keep[1:], dtype=torch.int32, device=dev)
            pos = torch.arange(pos0, pos0 + a, dtype=torch.int32, device=dev)
            rb = RowBatch(toks, torch.full((a,), seq.slot, dtype=torch.int32, device=dev), pos, mode="decode",
                          splits=K.decode_splits(pos0 + a, a, self.head.inner.geom.Hkv))
            self.head.forward(rb, hid[:a], eng.decode_buf, self.kvl, eng.kv.table)
            self.stats["catchup_rows"] += a
        self.pending[seq.slot] = (pos0 + a, hid[a].clone())

    def forget(self, slot: int) -> None:
        self.pending.pop(slot, None)
