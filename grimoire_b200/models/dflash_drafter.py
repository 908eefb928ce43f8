"""DFlash block drafter: a small decoder that drafts a block of tokens in ONE pass from the target's residual taps.

What it computes (reference: ``dflash_draft``, src/grimoire.cpp:16516-17289; the drafter's layer math is the Qwen3 decoder
layer of tools/ref_qwen3_dflash.py):

* **Context.**  For every committed position the target keeps the residual stream after a few of its layers (the taps,
  ``DenseModel.set_taps``).  The row [taps x H_target] goes through ``fc`` to the drafter's width, then ``hidden_norm``;
  every drafter layer projects that row with its own k / v weights (k gets the per-head norm and RoPE at the row's
  position) and keeps the result in its context cache.  Rows are ingested once, as they are committed.
* **Block.**  The query block is [bonus token, mask x (M - 1)] at positions L .. L + M - 1, embedded with the drafter's (or
  the target's) embedding table.  Each layer: RMSNorm, q / k / v with per-head q / k norm and RoPE, attention over the
  context rows plus the block's own rows -- NOT causal inside the block unless the layer's config says so, optionally
  windowed -- then o, residual, RMSNorm, SwiGLU MLP, residual.  After the final norm the head gives M - 1 draft tokens at
  once (rows 1 .. M - 1; row 0 is the bonus token's own row); a reduced draft vocabulary maps back through ``d2t``.

The drafter is small (6 layers) and runs once per speculative round, so its projections are plain bf16 matrix products;
the block is verified by the target through the engine's batched verify path like any other draft.  Block width: 8 rows
by default including the bonus row (the reference's measured optimum, grimoire.cpp:16500; ``GRIMOIRE_DFLASH_M`` = 2..16).

Second generation (``conv_kernel_size`` / ``selector_rank`` in the draft config; ref/qwen3_dflash2.py, selector kernels
src/ops.cpp:1885-1940): every layer wraps its attention and its MLP in a grouped dynamic convolution over the block's rows
(coefficients = a per-(tap, group) base plus a projection of the sublayer's input; row r mixes rows r - tap .. r of the SAME
block, never across the block start), the block embeddings are scaled, and the head proposes ``selector_top_k`` candidates
per position whose pair scores unary[c] + <pred[prev] * proj(hidden), succ[c]> are walked greedily from the bonus token, so a
draft token is chosen given the token drafted before it.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch
import torch.nn.functional as F

from ..ops import ref
from .dflash import DFlashSettings, resolve_dflash_config


@dataclass
class DFlashLayer:
    in_norm: torch.Tensor
    post_norm: torch.Tensor
    wq: torch.Tensor          # [Hq * D][H]
    wk: torch.Tensor          # [Hkv * D][H]
    wv: torch.Tensor
    wo: torch.Tensor          # [H][Hq * D]
    q_norm: Optional[torch.Tensor]
    k_norm: Optional[torch.Tensor]
    w_gate: torch.Tensor      # [I][H]
    w_up: torch.Tensor
    w_down: torch.Tensor      # [H][I]
    window: int = 0
    causal: bool = False
    attn_conv: Optional["GroupedConv"] = None      # second generation: dynamic convolutions around attention and MLP
    mlp_conv: Optional["GroupedConv"] = None


@dataclass
class GroupedConv:
    base: torch.Tensor        # fp32 [2][taps][H]: side 0 before the sublayer, side 1 after it
    proj: torch.Tensor        # [2 * taps * groups][H]
    taps: int
    group: int

    def _conv(self, x: torch.Tensor, delta: torch.Tensor, side: int) -> torch.Tensor:
        """x [rows][H] (one block), delta [rows][taps][groups]: out[r] = sum_tap coef[r][tap] * x[r - tap] for r >= tap."""
        rows, H = x.shape
        G = H // self.group
        xb = x.reshape(rows, G, self.group)
        coef = self.base[side].reshape(1, self.taps, G, self.group) + delta.unsqueeze(-1)
        out = coef[:, 0] * xb
        for tap in range(1, min(self.taps, rows)):
            out[tap:] += coef[tap:, tap] * xb[:-tap]
        return out.reshape(rows, H)

    def prepare(self, x: torch.Tensor, lin):
        rows = x.shape[0]
        co = lin(x, self.proj).reshape(rows, 2, self.taps, x.shape[1] // self.group)
        return self._conv(x, co[:, 0], 0), co[:, 1]

    def finish(self, y: torch.Tensor, co: torch.Tensor) -> torch.Tensor:
        return self._conv(y, co, 1)


class DFlashModel:
    """Weights + math of the drafter (no engine state): ``context_kv`` for committed rows, ``block`` for a query block."""

    def __init__(self, st: DFlashSettings, sd: dict, device, target_hidden: int, dtype=torch.bfloat16):
        if st.error:
            raise ValueError(f"draft config: {st.error}")
        self.st, self.device, self.dtype = st, torch.device(device), dtype
        pfx = "model." if any(k.startswith("model.layers.") for k in sd) else ""
        renames = {"encoder.fc.": "fc.", "encoder.output_norm_enc.": "hidden_norm.", "midlayer.": "layers.0."}   # other checkpoints' names

        def get(name, required=True):
            for cand in (pfx + name, name):
                if cand in sd:
                    return sd[cand]
            for old, new in renames.items():
                if name.startswith(new):
                    alt = old + name[len(new):]
                    for cand in (pfx + alt, alt):
                        if cand in sd:
                            return sd[cand]
            if required:
                raise KeyError(f"draft checkpoint has no tensor {name}")
            return None

        mat = lambda t: None if t is None else t.to(device=self.device, dtype=dtype).contiguous()
        vec = lambda t: None if t is None else t.to(device=self.device, dtype=torch.float32).contiguous()
        self.H, self.Hq, self.Hkv, self.D = st.hidden, st.n_heads, st.n_kv_heads, st.head_dim
        self.n_taps = len(st.target_layers)
        self.fc = mat(get("fc.weight", required=st.use_aux_hidden_state))
        if self.fc is not None and self.fc.shape != (self.H, self.n_taps * target_hidden):
            raise ValueError(f"fc is {tuple(self.fc.shape)} but the tap set gives {self.n_taps} x {target_hidden} inputs: the tap set "
                             "does not belong to this drafter")
        self.hidden_norm, self.norm = vec(get("hidden_norm.weight")), vec(get("norm.weight"))
        self.embed = mat(get("embed_tokens.weight", required=False))           # None: the target's table is used
        self.head = mat(sd.get("lm_head.weight"))                               # None: tied to the embedding / the target's head
        self.mask_embedding = mat(get("mask_embedding", required=False))
        d2t = sd.get("d2t")
        self.d2t = None if d2t is None else d2t.to(device=self.device, dtype=torch.long)
        self.selector = None
        if st.selector_rank > 0 and st.selector_top_k > 0:
            self.selector = (mat(get("candidate_selector.predecessor_codebook")), mat(get("candidate_selector.successor_codebook")),
                             mat(get("candidate_selector.hidden_projection.weight")))
        self.layers: list[DFlashLayer] = []

        def conv(p):
            if st.conv_kernel_size <= 0:
                return None
            return GroupedConv(vec(get(p + "base_kernel")), mat(get(p + "kernel_projection.weight")), st.conv_kernel_size, st.conv_group_size)

        for i in range(st.n_layers):
            p = f"layers.{i}."
            at = st.layers[i] if i < len(st.layers) else None
            self.layers.append(DFlashLayer(
                vec(get(p + "input_layernorm.weight")), vec(get(p + "post_attention_layernorm.weight")),
                mat(get(p + "self_attn.q_proj.weight")), mat(get(p + "self_attn.k_proj.weight")), mat(get(p + "self_attn.v_proj.weight")),
                mat(get(p + "self_attn.o_proj.weight")), vec(get(p + "self_attn.q_norm.weight", False)),
                vec(get(p + "self_attn.k_norm.weight", False)), mat(get(p + "mlp.gate_proj.weight")), mat(get(p + "mlp.up_proj.weight")),
                mat(get(p + "mlp.down_proj.weight")), window=at.window if at else 0, causal=at.causal if at else False,
                attn_conv=conv(p + "attention_conv."), mlp_conv=conv(p + "mlp_conv.")))
        self.inv_freq = ref.rope_inv_freq(self.D, st.rope_theta).to(self.device)
        self.scale = self.D ** -0.5

    # ---- pieces ----
    def _lin(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return (x.to(self.dtype) @ w.t()).float()

    def _heads(self, x: torch.Tensor, n: int, norm_w, pos: torch.Tensor, rope: bool = True) -> torch.Tensor:
        x = x.reshape(x.shape[0], n, self.D)
        x = ref.head_rmsnorm(x, norm_w, self.st.rms_eps, 0.0)
        return ref.apply_rope(x, pos, self.inv_freq, self.D) if rope else x

    def combine(self, taps: torch.Tensor) -> torch.Tensor:
        """Target taps [rows][n_taps][H_target] (or already [rows][H] without aux states) -> context rows [rows][H]."""
        x = taps.reshape(taps.shape[0], -1).float()
        return self._lin(x, self.fc) if self.fc is not None else x

    def context_kv(self, ctx: torch.Tensor, pos: torch.Tensor):
        """Context rows [rows][H] at positions ``pos`` -> per layer (k [rows][Hkv][D] with norm + RoPE, v [rows][Hkv][D])."""
        xn = ref.rmsnorm(ctx, self.hidden_norm, self.st.rms_eps, 0.0)
        out = []
        for L in self.layers:
            k = self._heads(self._lin(xn, L.wk), self.Hkv, L.k_norm, pos)
            v = self._lin(xn, L.wv).reshape(-1, self.Hkv, self.D)
            out.append((k, v))
        return out

    def embed_block(self, ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
        e = table[ids.long()].float()
        if self.mask_embedding is not None and self.st.mask_token >= 0:
            e = torch.where((ids == self.st.mask_token)[:, None], self.mask_embedding.float()[None, :], e)
        return e * self.st.input_embedding_scale

    def block(self, h: torch.Tensor, pos: torch.Tensor, ctx_kv, ctx_len: int) -> torch.Tensor:
        """Run the block rows ``h`` [M][H] (embedded) at positions ``pos`` over per-layer context (k, v) of which the first
        ``ctx_len`` rows (positions 0 .. ctx_len - 1) are valid.  Returns the final-normed hidden rows [M][H]."""
        M = h.shape[0]
        G = self.Hq // self.Hkv
        eps = self.st.rms_eps
        kpos = torch.cat([torch.arange(ctx_len, device=h.device), pos.long()])
        for L, (ck, cv) in zip(self.layers, ctx_kv):
            x = ref.rmsnorm(h, L.in_norm, eps, 0.0)
            co = None
            if L.attn_conv is not None:
                x, co = L.attn_conv.prepare(x, self._lin)
            q = self._heads(self._lin(x, L.wq), self.Hq, L.q_norm, pos)
            k = self._heads(self._lin(x, L.wk), self.Hkv, L.k_norm, pos)
            v = self._lin(x, L.wv).reshape(M, self.Hkv, self.D)
            kk = torch.cat([ck[:ctx_len].float(), k]).repeat_interleave(G, dim=1)        # [T][Hq][D]
            vv = torch.cat([cv[:ctx_len].float(), v]).repeat_interleave(G, dim=1)
            s = torch.einsum("mhd,thd->mht", q, kk) * self.scale
            qp = pos.long()[:, None]
            ok = torch.ones(M, kk.shape[0], dtype=torch.bool, device=h.device)
            if L.causal:
                ok &= kpos[None, :] <= qp
            if L.window > 0:
                ok &= kpos[None, :] > qp - L.window
            s = s.masked_fill(~ok[:, None, :], float("-inf"))
            o = torch.einsum("mht,thd->mhd", torch.softmax(s, dim=-1), vv).reshape(M, self.Hq * self.D)
            a = self._lin(o, L.wo)
            h = h + (L.attn_conv.finish(a, co) if co is not None else a)
            x = ref.rmsnorm(h, L.post_norm, eps, 0.0)
            co = None
            if L.mlp_conv is not None:
                x, co = L.mlp_conv.prepare(x, self._lin)
            act = F.silu(self._lin(x, L.w_gate)) * self._lin(x, L.w_up)
            y = self._lin(act, L.w_down)
            h = h + (L.mlp_conv.finish(y, co) if co is not None else y)
        return ref.rmsnorm(h, self.norm, eps, 0.0)

    def logits(self, hidden: torch.Tensor, head: torch.Tensor) -> torch.Tensor:
        lg = self._lin(hidden, head) * self.st.output_multiplier
        cap = self.st.final_logit_softcapping
        return torch.tanh(lg / cap) * cap if cap > 0 else lg

    def select(self, hidden: torch.Tensor, head: torch.Tensor, anchor: int) -> torch.Tensor:
        """Second-generation choice of the draft tokens for the rows ``hidden`` [steps][H] (the mask rows, final-normed):
        top-k candidates per step, pair scores against the previous step's candidates (the bonus token before step 0), and a
        greedy walk that picks each step's best candidate given the candidate picked before it.  Draft-vocabulary ids."""
        pred, succ, proj = self.selector
        k = self.st.selector_top_k
        unary, cand = torch.topk(self.logits(hidden, head), k, dim=-1)                 # [steps][k]
        hp = self._lin(hidden, proj)                                                    # [steps][rank]
        steps = hidden.shape[0]
        prev_ids = torch.cat([torch.full((1, k), int(anchor), dtype=torch.long, device=hidden.device), cand[:-1]], dim=0)
        gated = (pred[prev_ids].float() * hp[:, None, :]).to(self.dtype).float()        # [steps][k prev][rank]
        pair = torch.einsum("lpr,lcr->lpc", gated, succ[cand].float()).to(self.dtype).float()
        scores = unary[:, None, :] + pair                                               # [steps][prev][cand]
        out, previous = [], 0
        sc = scores.cpu()
        for step in range(steps):
            previous = int(sc[step, previous].argmax())
            out.append(cand[step, previous])
        return torch.stack(out)

    def to_target_ids(self, ids: torch.Tensor) -> torch.Tensor:
        return ids if self.d2t is None else ids + self.d2t[ids]


class DFlashDrafter:
    """Drafter protocol (engine/generation.py: propose / observe / forget, plus the engine's prefill hook) over a
    ``DFlashModel``: keeps per-slot context caches in step with what the target has committed."""

    def __init__(self, engine, model: DFlashModel, block_rows: Optional[int] = None):
        from .dense import DenseModel

        tgt = engine.model
        if not isinstance(tgt, DenseModel):
            raise ValueError("the block drafter taps the residual stream of the dense decoder family")
        self.engine, self.m = engine, model
        st = model.st
        if not st.target_layers:
            raise ValueError("the draft config names no target layers to tap")
        if st.mask_token < 0:
            raise ValueError("the draft config has no mask_token_id")
        tgt.set_taps(st.target_layers)
        tgt.add_tap_rows(engine.decode_buf)
        if engine.prefill_buf is not None:
            tgt.add_tap_rows(engine.prefill_buf)
        dev = engine.device
        if model.embed is None:
            if tgt.cfg.hidden_size != model.H:
                raise ValueError("the drafter has no embedding table of its own and the target's has another width")
            model.embed = tgt.embed
        self.table = model.embed
        if model.head is not None:
            self.head = model.head
        else:
            self.head = model.embed                   # tied head (a drafter sharing the target's table shares its head too)
        env = int(os.environ.get("GRIMOIRE_DFLASH_M", "0") or 0)
        self.block_rows = max(2, min(16, block_rows or env or 8, st.block_size))
        lim = engine.limits
        n, T = lim.max_slots, lim.max_ctx
        self.ck = [torch.zeros(n, T, model.Hkv, model.D, dtype=model.dtype, device=dev) for _ in model.layers]
        self.cv = [torch.zeros(n, T, model.Hkv, model.D, dtype=model.dtype, device=dev) for _ in model.layers]
        self.have: dict[int, int] = {}                # slot -> context rows ingested (positions 0 .. have - 1)
        self.stats = {"blocks": 0, "ctx_rows": 0}
        engine.mtp = self                             # the engine's prefill hook (warm_chunk) and speculation switch
        engine.enable_speculation()

    # ---- context ingestion ----
    def _ingest(self, slot: int, taps: torch.Tensor, pos0: int) -> None:
        rows = taps.shape[0]
        if rows <= 0:
            return
        pos = torch.arange(pos0, pos0 + rows, device=taps.device)
        ctx = self.m.combine(taps)
        for li, (k, v) in enumerate(self.m.context_kv(ctx, pos)):
            self.ck[li][slot, pos0: pos0 + rows] = k.to(self.m.dtype)
            self.cv[li][slot, pos0: pos0 + rows] = v.to(self.m.dtype)
        self.have[slot] = pos0 + rows
        self.stats["ctx_rows"] += rows

    def warm_chunk(self, seq, tokens_dev, done: int, m: int, pos0: int, buf, last: bool) -> None:
        """Prefill hook: the chunk's rows were just run by the target; their taps are in ``buf.taps[:m]``."""
        if self.have.get(seq.slot, 0) != pos0:
            self.have[seq.slot] = min(self.have.get(seq.slot, 0), pos0)      # a restored prefix: rows before pos0 may be stale
            if self.have[seq.slot] != pos0:
                self.have[seq.slot] = -1                                      # context incomplete: no drafts for this conversation
                return
        self._ingest(seq.slot, buf.taps[:m], pos0)

    def observe(self, engine, seq, accepted_tokens, row0: int = 0) -> None:
        """After a committed step: rows row0 .. row0 + len(accepted) - 1 of the decode buffers are the accepted rows."""
        n = len(accepted_tokens)
        pos0 = seq.length - n
        if self.have.get(seq.slot, 0) != pos0:
            self.have[seq.slot] = -1
            return
        self._ingest(seq.slot, engine.decode_buf.taps[row0: row0 + n], pos0)

    def forget(self, slot: int) -> None:
        self.have.pop(slot, None)

    # ---- drafting ----
    def propose(self, engine, seq, last_token: int, depth: int) -> list[int]:
        L = seq.length
        if depth <= 0 or self.have.get(seq.slot, 0) != L or L <= 0:
            return []
        M = min(self.block_rows, depth + 1)
        if L + M > self.ck[0].shape[1]:
            return []
        dev = engine.device
        ids = torch.full((M,), self.m.st.mask_token, dtype=torch.long, device=dev)
        ids[0] = int(last_token)
        pos = torch.arange(L, L + M, device=dev)
        h = self.m.embed_block(ids, self.table)
        ctx = [(self.ck[li][seq.slot], self.cv[li][seq.slot]) for li in range(len(self.m.layers))]
        hid = self.m.block(h, pos, ctx, L)
        if self.m.selector is not None:
            out = self.m.to_target_ids(self.m.select(hid[1:], self.head, int(last_token)))
        else:
            out = self.m.to_target_ids(self.m.logits(hid[1:], self.head).argmax(dim=-1))
        self.stats["blocks"] += 1
        return [int(t) for t in out.tolist()]


def load_dflash(path, engine, block_rows: Optional[int] = None) -> DFlashDrafter:
    """Drafter from a checkpoint directory (``config.json`` + safetensors) attached to ``engine``."""
    from ..formats.safetensors_io import SafeTensorsFile

    path = Path(path)
    st = resolve_dflash_config((path / "config.json").read_text())
    sd = {}
    for f in sorted(path.glob("*.safetensors")):
        sf = SafeTensorsFile(f)
        for name in sf.keys():
            sd[name] = sf.get(name).clone()
        sf.close()
    if not sd:
        raise FileNotFoundError(f"no .safetensors file in {path}")
    model = DFlashModel(st, sd, engine.device, engine.model.cfg.hidden_size)
    return DFlashDrafter(engine, model, block_rows)


def random_dflash_state_dict(st: DFlashSettings, target_hidden: int, seed: int = 0, std: float = 0.05, own_embedding: bool = True) -> dict:
    """Random drafter weights under the checkpoint names (tests, benchmarks)."""
    g = torch.Generator().manual_seed(seed)
    rnd = lambda *s: torch.randn(*s, generator=g) * std
    H, D = st.hidden, st.head_dim
    sd = {"fc.weight": rnd(H, len(st.target_layers) * target_hidden), "hidden_norm.weight": 1 + rnd(H), "norm.weight": 1 + rnd(H)}
    if own_embedding:
        sd["embed_tokens.weight"] = rnd(st.vocab, H)
        sd["lm_head.weight"] = rnd(st.draft_vocab, H)
    for i in range(st.n_layers):
        p = f"layers.{i}."
        sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"] = 1 + rnd(H), 1 + rnd(H)
        sd[p + "self_attn.q_proj.weight"] = rnd(st.n_heads * D, H)
        sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"] = rnd(st.n_kv_heads * D, H), rnd(st.n_kv_heads * D, H)
        sd[p + "self_attn.o_proj.weight"] = rnd(H, st.n_heads * D)
        sd[p + "self_attn.q_norm.weight"], sd[p + "self_attn.k_norm.weight"] = 1 + rnd(D), 1 + rnd(D)
        sd[p + "mlp.gate_proj.weight"], sd[p + "mlp.up_proj.weight"] = rnd(st.inter, H), rnd(st.inter, H)
        sd[p + "mlp.down_proj.weight"] = rnd(H, st.inter)
        if st.conv_kernel_size > 0:
            G = H // st.conv_group_size
            for c in ("attention_conv.", "mlp_conv."):
                base = rnd(2, st.conv_kernel_size, H)
                base[:, 0] += 1.0                      # near the identity: tap 0 carries the row itself
                sd[p + c + "base_kernel"] = base
                sd[p + c + "kernel_projection.weight"] = rnd(2 * st.conv_kernel_size * G, H)
    if st.selector_rank > 0:
        sd["candidate_selector.predecessor_codebook"] = rnd(st.vocab, st.selector_rank) * 10
        sd["candidate_selector.successor_codebook"] = rnd(st.draft_vocab, st.selector_rank) * 10
        sd["candidate_selector.hidden_projection.weight"] = rnd(st.selector_rank, H) * 10
    return sd


def dflash_config_json(**kw) -> str:
    """A draft ``config.json`` text from keyword facts (tests, synthetic drafters)."""
    return json.dumps(kw)
