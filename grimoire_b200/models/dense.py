"""Dense attention decoder (Qwen3-style): weights + the universal M-row forward pass.

One function serves prompt prefill, batched decode and speculative verify, exactly as the
reference's ``prefill(tokens, next_tokens, seqb)`` does (grimoire.cpp:20263-23631: "a batched
decode is a prefill whose M rows belong to M different conversations"); the rows' (sequence,
position) pairs and the attention mode are the only difference.

Per layer (compare forward(), grimoire.cpp:14986-15616, ~29 launches per layer there; 8 here):
  rmsnorm -> fused q|k|v projection -> norm/RoPE/int8 page write -> attention -> o_proj (+= h)
  rmsnorm -> fused gate|up projection with SwiGLU epilogue -> down_proj (+= h)
Under tensor parallelism the two row-parallel projections hand their partial sums to the fused
all-reduce (parallel/tp.py) instead of accumulating into ``h`` directly.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..formats.codecs import Fmt
from ..formats.quantize import QuantWeight, quantize, slice_cols, slice_rows
from ..formats.w4_tile_layout import concat_rows, interleave_gate_up_q
from ..ops import core as K
from ..ops import ref
from ..ops.linear import BF16Linear, MXLinear, ROWQ_KIND, RowQLinear, W4Linear
from ..ops.workspace import Workspace
from ..utils import trace
from .config import ModelConfig

# --proj names served by the byte-per-weight kernel (per-row scale, or e8m0 per 32 for mxfp8)
_ROWQ_PROJ = {"int8": Fmt.INT8, "bf16": Fmt.BF16, "mxfp8": Fmt.MXFP8, "fp8_e4m3": Fmt.FP8_E4M3, "fp8_e5m2": Fmt.FP8_E5M2}


@dataclass
class DenseLayer:
    in_norm: torch.Tensor
    post_norm: torch.Tensor
    qkv: W4Linear
    o: W4Linear
    gate_up: W4Linear
    down: W4Linear
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None


@dataclass
class RowBatch:
    """What one forward pass works on.  ``mode`` is 'decode' (every row is its own (seq, pos)
    over the paged cache: decode / batched decode / verify) or 'prefill' (all rows are
    consecutive positions q_pos0.. of ONE sequence ``seq_slot``)."""

    tokens: torch.Tensor                 # int32 [M]
    row_seq: torch.Tensor                # int32 [M]
    row_pos: torch.Tensor                # int32 [M]
    mode: str = "decode"
    q_pos0: int = 0
    seq_slot: int = 0
    splits: int = 1
    logits_rows: Optional[torch.Tensor] = None   # int64 indices of rows that need logits (None = all)
    distinct: bool = False               # decode: every row is a different sequence (no verify block in the step)
    # prefill of several fresh prompts in one pass: (first row, rows) per prompt, rows of a prompt contiguous and at
    # positions 0..rows-1 of its own sequence (admit_batch, grimoire.cpp:12071-12146); None = one sequence
    segments: Optional[list] = None
    # decode with verify blocks on a model with recurrent layers: (run_slot, run_start, run_len) int32 device tensors,
    # one run per maximal group of rows that are consecutive positions of one sequence; None = every row is its own run
    runs: Optional[tuple] = None
    # vocabulary-split lm_head (tensor parallel): True = the returned logits rows are gathered over the ranks; False = only
    # this rank's column slice is valid and the caller picks the token with the (value, index) exchange
    full_logits: bool = True
    # decode step with verify blocks: (int32 device tensor [4][n] of groups -- slot, first row, rows, first position --, n);
    # the attention then reads the cache once per group of rows (attn_verify.cu) instead of once per row
    verify: Optional[tuple] = None


class Buffers:
    """Activation buffers for up to ``max_rows`` rows (allocated once; graph-capture safe)."""

    def __init__(self, cfg: ModelConfig, geom: K.AttnGeom, I_local: int, max_rows: int, max_logit_rows: int, device,
                 dense_kv_tokens: int = 0):
        H = cfg.hidden_size
        bf, f32 = torch.bfloat16, torch.float32
        mk = lambda *s, dt: torch.zeros(*s, dtype=dt, device=device)
        qsz = geom.Hq * geom.D * (2 if geom.q_gated else 1)
        self.h = mk(max_rows, H, dt=f32)
        self.x = mk(max_rows, H, dt=bf)
        self.qkv = mk(max_rows, qsz + 2 * geom.Hkv * geom.D, dt=bf)
        self.q = mk(max_rows, geom.Hq * geom.D, dt=bf)
        self.gate = mk(max_rows, geom.Hq * geom.D, dt=bf) if geom.q_gated else None
        self.attn = mk(max_rows, geom.Hq * geom.D, dt=bf)
        self.act = mk(max_rows, I_local, dt=bf)
        self.partial = mk(max_rows, H, dt=f32)
        self.xf = mk(max_logit_rows, H, dt=bf)
        self.logits = mk(max_logit_rows, cfg.vocab_size, dt=f32)
        self.next_ids = mk(max_logit_rows, dt=torch.int32)
        self.dense_k = mk(dense_kv_tokens, geom.Hkv * geom.D, dt=bf) if dense_kv_tokens else None
        self.dense_v = mk(dense_kv_tokens, geom.Hkv * geom.D, dt=bf) if dense_kv_tokens else None
        self.max_rows = max_rows
        self.max_logit_rows = max_logit_rows
        self.taps = None            # [max_rows][taps][H] fp32 when the model keeps residual taps (DenseModel.set_taps)


class DenseModel:
    def __init__(self, cfg: ModelConfig, device, tp_rank: int = 0, tp_world: int = 1,
                 workspace: Optional[Workspace] = None, pp_rank: int = 0, pp_world: int = 1):
        self.cfg = cfg
        self.device = torch.device(device)
        self.tp_rank, self.tp_world = tp_rank, tp_world
        # pipeline stage r owns layers [layer_begin, layer_end) (grimoire.cpp:2485-2499)
        self.pp_rank, self.pp_world = pp_rank, pp_world
        per, extra = divmod(cfg.num_hidden_layers, pp_world)
        self.layer_begin = pp_rank * per + min(pp_rank, extra)
        self.layer_end = self.layer_begin + per + (1 if pp_rank < extra else 0)
        self.pp = None          # parallel.pp.PipelineParallel when pp_world > 1
        self.cp = None          # parallel.cp.ContextParallel: prefill chunks split by rows over whole-model replicas
        self.up = None          # parallel.ulysses.UlyssesParallel: head-parallel attention, KV heads sharded over replicas
        self.head_split = None  # (first vocabulary row, rows) of this rank's lm_head shard (TensorParallel.split_head)
        self.tap_index: dict[int, int] = {}   # layer id -> slot of buf.taps (set_taps): residual after that layer is kept per row
        self.ws = workspace or Workspace(device)
        if cfg.num_attention_heads % tp_world or cfg.num_key_value_heads % tp_world or cfg.intermediate_size % tp_world:
            raise ValueError("tensor parallel degree must divide heads, kv heads and the FFN width")
        self.Hq = cfg.num_attention_heads // tp_world
        self.Hkv = cfg.num_key_value_heads // tp_world
        self.I = cfg.intermediate_size // tp_world
        self.geom = K.AttnGeom(self.Hq, self.Hkv, cfg.head_dim, cfg.rot_dim,
                               cfg.softmax_scale or ref.softmax_scale(cfg.head_dim), cfg.attn_output_gate,
                               cfg.sliding_window, cfg.rms_norm_eps, cfg.norm_offset)
        self.inv_freq = ref.rope_inv_freq(cfg.rot_dim, cfg.rope_theta).to(self.device)
        self.layers: list[DenseLayer] = []
        self.embed: Optional[torch.Tensor] = None
        self.final_norm: Optional[torch.Tensor] = None
        self.lm_head = None
        self.tp = None          # parallel.tp.TensorParallel when tp_world > 1

    # ------------------------------------------------------------------------------------------
    # construction
    # ------------------------------------------------------------------------------------------
    def _quant(self, w) -> QuantWeight:
        """fp32 tensor or stored QuantWeight -> runtime int4 (stored int4 is used as is)."""
        cfg = self.cfg
        if cfg.quant == "fp8":
            if isinstance(w, QuantWeight):
                return w if w.fmt == Fmt.FP8_BLOCK else quantize(w.dequant(), Fmt.FP8_BLOCK)
            return quantize(w, Fmt.FP8_BLOCK)
        if cfg.quant == "mxfp4":
            if isinstance(w, QuantWeight):
                return w if w.fmt == Fmt.MXFP4 else quantize(w.dequant(), Fmt.MXFP4)
            return quantize(w, Fmt.MXFP4)
        if cfg.quant in _ROWQ_PROJ:
            fmt = _ROWQ_PROJ[cfg.quant]
            if isinstance(w, QuantWeight):
                return w if w.fmt == fmt else quantize(w.dequant(), fmt)
            return quantize(w, fmt)
        if isinstance(w, QuantWeight):
            return w if w.fmt == Fmt.INT4 else quantize(w.dequant(), Fmt.INT4, group=cfg.quant_group)
        return quantize(w, Fmt.INT4, group=cfg.quant_group, symmetric=getattr(cfg, "quant_symmetric", False))

    def set_taps(self, layer_ids) -> None:
        """Keep the residual stream after each of ``layer_ids`` for every row of every pass (``buf.taps`` [rows][taps][H]
        fp32): the inputs of a block drafter (models/dflash_drafter.py).  A tap is the stream at ENTRY of layer id + 1
        (grimoire.cpp:9325), so the last layer cannot be tapped.  Buffers made before this call get their tap rows here."""
        ids = [int(i) for i in layer_ids]
        if any(i < 0 or i >= self.cfg.num_hidden_layers - 1 for i in ids):
            raise ValueError("a tap names a layer outside [0, layers - 2]")
        if self.tp_world > 1 or self.pp_world > 1 or self.cp is not None:
            raise ValueError("residual taps are kept on single-GPU models only")
        self.tap_index = {lid: j for j, lid in enumerate(ids)}

    def _linear(self, qw: QuantWeight, name: str, swiglu: bool = False):
        """Runtime projection for a quantized weight: int4 -> W4Linear, MXFP4 -> MXLinear, block-scaled fp8 ->
        FP8BlockLinear (its SwiGLU form takes [gate rows | up rows], not the per-16 interleave)."""
        if qw.fmt == Fmt.FP8_BLOCK:
            from ..ops.hybrid import FP8BlockLinear

            return FP8BlockLinear(qw, self.device, name)
        if qw.fmt in ROWQ_KIND:
            return RowQLinear(qw, self.device, name, swiglu=swiglu, workspace=self.ws)
        cls = MXLinear if qw.fmt == Fmt.MXFP4 else W4Linear
        return cls(qw, self.device, name, swiglu=swiglu, workspace=self.ws)

    @staticmethod
    def _norm_linear(lin, h, norm_w, x, out, epi: str, eps: float, off: float) -> None:
        """out = epi(lin(RMSNorm(h))): one launch when the projection can take the norm into its prologue (single-row
        int4 GEMV), otherwise the norm kernel writes x and the projection reads it."""
        fused = getattr(lin, "fused_norm", None)
        if fused is not None and h.shape[0] == 1 and fused(h, norm_w, out, epi, eps, off):
            return
        K.add_rmsnorm(h, norm_w, x, eps, off)
        lin(x, out, epi)

    def _head(self, hsel: torch.Tensor, buf: "Buffers", n: int, rb: RowBatch) -> torch.Tensor:
        """Final norm + lm_head over ``n`` rows.  With a vocabulary-split head this rank writes its column slice of the
        logits rows; they are gathered unless the caller asked for the slice only (``rb.full_logits`` False)."""
        cfg = self.cfg
        xf, logits = buf.xf[:n], buf.logits[:n]
        if self.head_split is None:
            self._norm_linear(self.lm_head, hsel, self.final_norm, xf, logits, "f32", cfg.rms_norm_eps, cfg.norm_offset)
            return logits
        v0, vn = self.head_split
        self._norm_linear(self.lm_head, hsel, self.final_norm, xf, logits[:, v0:v0 + vn], "f32", cfg.rms_norm_eps, cfg.norm_offset)
        if rb.mode == "prefill" or rb.full_logits:
            self.tp.gather_head(logits)
        return logits

    @staticmethod
    def _rows(w, a: int, b: int):
        return slice_rows(w, a, b) if isinstance(w, QuantWeight) else w[a:b]

    @staticmethod
    def _cols(w, a: int, b: int):
        return slice_cols(w, a, b) if isinstance(w, QuantWeight) else w[:, a:b]

    def _shard_rows(self, w, heads: int, per: int):
        """rows of a column-parallel weight owned by this rank (whole heads)."""
        n = heads // self.tp_world * per
        return self._rows(w, self.tp_rank * n, (self.tp_rank + 1) * n)

    def add_layer_from_dense(self, wq, wk, wv, wo, wg, wu, wd, in_norm, post_norm, q_norm=None, k_norm=None):
        """Quantize + shard + tile one layer from full-precision logical weights (``[out][in]``)."""
        cfg, dev, W, r = self.cfg, self.device, self.tp_world, self.tp_rank
        D = cfg.head_dim
        qper = D * (2 if cfg.attn_output_gate else 1)
        wq_s = self._shard_rows(wq, cfg.num_attention_heads, qper)
        wk_s = self._shard_rows(wk, cfg.num_key_value_heads, D)
        wv_s = self._shard_rows(wv, cfg.num_key_value_heads, D)
        kq = cfg.num_attention_heads * D // W
        wo_s = self._cols(wo, r * kq, (r + 1) * kq)
        I = cfg.intermediate_size // W
        wg_s, wu_s = self._rows(wg, r * I, (r + 1) * I), self._rows(wu, r * I, (r + 1) * I)
        wd_s = self._cols(wd, r * I, (r + 1) * I)
        qkv = concat_rows([self._quant(wq_s), self._quant(wk_s), self._quant(wv_s)])
        qg, qu = self._quant(wg_s), self._quant(wu_s)
        gu = concat_rows([qg, qu]) if qg.fmt == Fmt.FP8_BLOCK else interleave_gate_up_q(qg, qu)
        f32 = lambda t: None if t is None else t.to(device=dev, dtype=torch.float32).contiguous()
        i = len(self.layers)
        self.layers.append(DenseLayer(
            f32(in_norm), f32(post_norm),
            self._linear(qkv, f"L{i}.qkv"),
            self._linear(self._quant(wo_s), f"L{i}.o"),
            self._linear(gu, f"L{i}.gate_up", swiglu=True),
            self._linear(self._quant(wd_s), f"L{i}.down"),
            f32(q_norm), f32(k_norm)))

    @staticmethod
    def from_gguf_native(cfg: ModelConfig, gf, device, workspace: Optional[Workspace] = None) -> "DenseModel":
        """A dense decoder whose projections stay the raw ggml blocks of its GGUF file (``--proj native``): q|k|v, o, gate|up
        and down become ``GgufLinear``s over the stored bytes (formats/gguf.py: raw_rows), norms and the embedding table are
        decoded, the lm_head stays raw when its block type is served.  Single rank.  Reference: the native GGUF path of the
        loader (src/native_model.cpp) + gemv_native_qk (src/gemv_decode.cpp:1216)."""
        from ..formats import gguf as G
        from ..ops.linear import GgufLinear

        m = DenseModel(cfg, device, 0, 1, workspace)
        H = cfg.hidden_size
        f32 = lambda name: gf.tensor(name).to(device=m.device, dtype=torch.float32).contiguous() if name in gf.tensors else None
        for i in range(cfg.num_hidden_layers):
            p = f"blk.{i}."
            rr = lambda stem: gf.raw_rows(p + stem + ".weight")
            qkv = GgufLinear([rr("attn_q"), rr("attn_k"), rr("attn_v")], H, m.device, f"L{i}.qkv", workspace=m.ws)
            o = GgufLinear([rr("attn_output")], cfg.num_attention_heads * cfg.head_dim, m.device, f"L{i}.o", workspace=m.ws)
            gu = GgufLinear([rr("ffn_gate"), rr("ffn_up")], H, m.device, f"L{i}.gate_up", swiglu=True, workspace=m.ws)
            dn = GgufLinear([rr("ffn_down")], cfg.intermediate_size, m.device, f"L{i}.down", workspace=m.ws)
            m.layers.append(DenseLayer(f32(p + "attn_norm.weight"), f32(p + "ffn_norm.weight"), qkv, o, gu, dn,
                                       f32(p + "attn_q_norm.weight"), f32(p + "attn_k_norm.weight")))
        m.embed = gf.tensor("token_embd.weight").to(device=m.device, dtype=torch.bfloat16).contiguous()
        m.final_norm = f32("output_norm.weight")
        if "output.weight" in gf.tensors and gf.tensors["output.weight"][1] in G.NATIVE_TYPES:
            m.lm_head = GgufLinear([gf.raw_rows("output.weight")], H, m.device, "lm_head", workspace=m.ws)
        elif "output.weight" in gf.tensors:
            m.lm_head = BF16Linear(gf.tensor("output.weight"), m.device, "lm_head(bf16)")
        else:
            m.lm_head = BF16Linear(m.embed, m.device, "lm_head(tied)")
        return m

    def set_embeddings(self, embed: torch.Tensor, final_norm: torch.Tensor, lm_head: Optional[torch.Tensor]):
        dev = self.device
        self.embed = embed.to(device=dev, dtype=torch.bfloat16).contiguous()
        self.final_norm = final_norm.to(device=dev, dtype=torch.float32).contiguous()
        if lm_head is None or self.cfg.tie_word_embeddings:
            # tied: the head aliases the embedding table and is never quantized (grimoire.cpp:3492-3495)
            self.lm_head = BF16Linear(self.embed, dev, "lm_head(tied)")
        else:
            self.lm_head = self._linear(self._quant(lm_head), "lm_head")

    @staticmethod
    def random(cfg: ModelConfig, device, seed: int = 0, tp_rank: int = 0, tp_world: int = 1, std: float = 0.02,
               gen_device=None, workspace: Optional[Workspace] = None, pp_rank: int = 0, pp_world: int = 1) -> "DenseModel":
        """Random-init weights N(0, std) of the named architecture, quantized to int4 (the synthetic
        checkpoints of the benchmarks).  Every rank draws the same logical matrices and keeps its
        shard, so TP results can be compared with a single-GPU run token for token."""
        m = DenseModel(cfg, device, tp_rank, tp_world, workspace, pp_rank, pp_world)
        gdev = torch.device(gen_device or device)
        g = torch.Generator(device=gdev)
        H, D = cfg.hidden_size, cfg.head_dim
        qrows = cfg.num_attention_heads * D * (2 if cfg.attn_output_gate else 1)

        def rnd(n, k, tag):
            g.manual_seed(seed * 1000003 + tag)
            return torch.randn(n, k, generator=g, device=gdev, dtype=torch.float32) * std

        ones = torch.ones(H)
        for i in range(m.layer_begin, m.layer_end):
            t = i * 16
            m.add_layer_from_dense(rnd(qrows, H, t + 1), rnd(cfg.kv_size, H, t + 2), rnd(cfg.kv_size, H, t + 3),
                                   rnd(H, cfg.num_attention_heads * D, t + 4), rnd(cfg.intermediate_size, H, t + 5),
                                   rnd(cfg.intermediate_size, H, t + 6), rnd(H, cfg.intermediate_size, t + 7),
                                   ones if not cfg.norm_zero_centered else torch.zeros(H),
                                   ones if not cfg.norm_zero_centered else torch.zeros(H),
                                   torch.ones(D) if cfg.qk_norm else None, torch.ones(D) if cfg.qk_norm else None)
        emb = rnd(cfg.vocab_size, H, 900001)
        head = None if cfg.tie_word_embeddings else rnd(cfg.vocab_size, H, 900002)
        m.set_embeddings(emb, ones if not cfg.norm_zero_centered else torch.zeros(H), head)
        return m

    @staticmethod
    def from_state_dict(cfg: ModelConfig, sd: dict, device, tp_rank: int = 0, tp_world: int = 1,
                        workspace: Optional[Workspace] = None, pp_rank: int = 0, pp_world: int = 1) -> "DenseModel":
        """Build from HF-named full-precision tensors (``[out][in]``), quantizing to int4."""
        m = DenseModel(cfg, device, tp_rank, tp_world, workspace, pp_rank, pp_world)
        for i in range(m.layer_begin, m.layer_end):
            p = f"model.layers.{i}."
            g = lambda k: sd.get(p + k)
            m.add_layer_from_dense(g("self_attn.q_proj.weight"), g("self_attn.k_proj.weight"), g("self_attn.v_proj.weight"),
                                   g("self_attn.o_proj.weight"), g("mlp.gate_proj.weight"), g("mlp.up_proj.weight"),
                                   g("mlp.down_proj.weight"), g("input_layernorm.weight"),
                                   g("post_attention_layernorm.weight"), g("self_attn.q_norm.weight"),
                                   g("self_attn.k_norm.weight"))
        m.set_embeddings(sd["model.embed_tokens.weight"], sd["model.norm.weight"], sd.get("lm_head.weight"))
        return m

    @staticmethod
    def from_checkpoint(path, device, tp_rank: int = 0, tp_world: int = 1, workspace: Optional[Workspace] = None,
                        lm_head_bf16: bool = False, pp_rank: int = 0, pp_world: int = 1, proj: str = "int4") -> "DenseModel":
        """Load a HF directory (safetensors shards; bf16 / GPTQ / compressed-tensors / fp8 / NVFP4
        projections) and serve it with int4-g128 projections.  Stored int4 is repacked, anything
        else is dequantized and quantized on the host (Grimoire::build, grimoire.cpp:7133-10637)."""
        from ..formats.checkpoint import Checkpoint

        ck = Checkpoint(path) if isinstance(path, (str, bytes)) or hasattr(path, "__fspath__") else path    # or any tensor resolver
        cfg = ck.cfg
        if proj in ("mxfp4", "fp8") or proj in _ROWQ_PROJ:
            import dataclasses

            cfg = dataclasses.replace(cfg, quant=proj)
        m = DenseModel(cfg, device, tp_rank, tp_world, workspace, pp_rank, pp_world)
        for i in range(m.layer_begin, m.layer_end):
            p = f"{ck.prefix}layers.{i}."
            lin = lambda k: ck.linear(p + k)
            m.add_layer_from_dense(lin("self_attn.q_proj"), lin("self_attn.k_proj"), lin("self_attn.v_proj"),
                                   lin("self_attn.o_proj"), lin("mlp.gate_proj"), lin("mlp.up_proj"), lin("mlp.down_proj"),
                                   ck.plain(p + "input_layernorm.weight"), ck.plain(p + "post_attention_layernorm.weight"),
                                   ck.plain(p + "self_attn.q_norm.weight"), ck.plain(p + "self_attn.k_norm.weight"))
        head = None if cfg.tie_word_embeddings else ck.linear("lm_head")
        emb = ck.embedding()
        m.set_embeddings(emb, ck.plain(ck.prefix + "norm.weight"), head)
        if lm_head_bf16 and head is not None:
            hw = head.dequant() if isinstance(head, QuantWeight) else head
            m.lm_head = BF16Linear(hw, device, "lm_head(bf16)")
        return m

    def weight_bytes(self) -> int:
        n = self.lm_head.nbytes()
        for l in self.layers:
            n += l.qkv.nbytes() + l.o.nbytes() + l.gate_up.nbytes() + l.down.nbytes()
        return n

    def make_buffers(self, max_rows: int, max_logit_rows: int, dense_kv_tokens: int = 0) -> Buffers:
        b = Buffers(self.cfg, self.geom, self.I, max_rows, max_logit_rows, self.device, dense_kv_tokens)
        self.add_tap_rows(b)
        return b

    def add_tap_rows(self, b: Buffers) -> None:
        if self.tap_index and getattr(b, "taps", None) is None:
            b.taps = torch.zeros(b.max_rows, len(self.tap_index), self.cfg.hidden_size, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------------------------------
    # forward over M rows
    # ------------------------------------------------------------------------------------------
    def _row_parallel(self, lin, x, h):
        if self.tp_world == 1:
            lin(x, h, "add_f32")
        else:
            self.tp.row_parallel_add(lin, x, h)

    def forward_prefill_sp(self, rb: RowBatch, buf: Buffers, kv_layers, block_table) -> torch.Tensor:
        """Prefill chunk under tensor parallelism with the fused GEMM -> reduce-scatter and
        all-gather -> GEMM kernels; the residual stream and the norms live on this rank's M/W token
        shard (sequence parallelism).  Same math as ``forward`` up to bf16 partial sums on the wire."""
        cfg, geom, tp = self.cfg, self.geom, self.tp
        M, H = rb.tokens.shape[0], cfg.hidden_size
        W, r = self.tp_world, self.tp_rank
        R = M // W
        eps, off = cfg.rms_norm_eps, cfg.norm_offset
        tp.sp_setup(M, H)
        hs = tp.sp_hs[:R]
        K.embed(rb.tokens[r * R: (r + 1) * R], self.embed, hs)
        qkv, q, attn, act = buf.qkv[:M], buf.q[:M], buf.attn[:M], buf.act[:M]
        gate = buf.gate[:M] if buf.gate is not None else None
        T = rb.q_pos0 + M
        tl = trace.timeline.on
        for li, L in enumerate(self.layers):
            kvl = kv_layers[li]
            if tl: trace.mark("reduce+norm+allgather")
            x_full, agc, age = tp.sp_reduce_norm_allgather(hs, L.in_norm, eps, off, reduce=li > 0, M=M)
            if tl: trace.mark("qkv gemm (dequant + ag-wait)")
            tp.sp_gemm_allgathered(L.qkv, x_full, agc, age, qkv, "bf16")
            if tl: trace.mark("rope + kv write")
            if rb.q_pos0 > 0:
                K.gather_kv_dense(kvl, block_table[rb.seq_slot], rb.q_pos0, buf.dense_k, buf.dense_v)
            K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm,
                           gate, buf.dense_k[rb.q_pos0: T], buf.dense_v[rb.q_pos0: T])
            if tl: trace.mark("flash prefill")
            K.flash_prefill(q, buf.dense_k, buf.dense_v, geom, attn, rb.q_pos0, gate)
            if tl: trace.mark("o gemm + rs push")
            tp.sp_gemm_reduce_scatter(L.o, attn, M, H)
            if tl: trace.mark("reduce+norm+allgather")
            x_full, agc, age = tp.sp_reduce_norm_allgather(hs, L.post_norm, eps, off, reduce=True, M=M)
            if tl: trace.mark("gate_up gemm (dequant + ag-wait)")
            tp.sp_gemm_allgathered(L.gate_up, x_full, agc, age, act, "swiglu")
            if tl: trace.mark("down gemm + rs push")
            tp.sp_gemm_reduce_scatter(L.down, act, M, H)
        if tl: trace.mark("tail")
        tp.sp_reduce_norm_allgather(hs, None, eps, off, reduce=True, M=M)
        # the rows that need logits live on their owners: collect them on every rank
        rows = rb.logits_rows if rb.logits_rows is not None else torch.arange(M, device=self.device)
        n = rows.shape[0]
        sel = torch.zeros(n, H, dtype=torch.float32, device=self.device)
        mine = (rows >= r * R) & (rows < (r + 1) * R)
        if bool(mine.any()):
            sel[mine] = hs.index_select(0, rows[mine] - r * R)
        torch.distributed.all_reduce(sel, group=tp.group)
        return self._head(sel, buf, n, rb)

    def _mega_ready(self) -> bool:
        from ..ops import linear as _lin

        if _lin.BATCH_INVARIANT:
            return False                # every height on the batch-invariant kernels (speculative decoding is on)
        ok = getattr(self, "_mega_ok", None)
        if ok is None:
            from ..ops import mega

            ok = self._mega_ok = mega.dense_supported(self)
        return ok

    def forward_mega(self, rb: RowBatch, buf: Buffers, kv_layers, block_table) -> torch.Tensor:
        """One decode token through the persistent phase kernel (ops/mega.py): two launches per layer -- attention, then
        o_proj | gate_up | down | the next layer's q|k|v inside one kernel -- with the same rounding points as ``forward``."""
        from ..ops import mega

        cfg, geom = self.cfg, self.geom
        tab = mega.table_for(self, buf)
        h, qkv, q, attn = buf.h[:1], buf.qkv[:1], buf.q[:1], buf.attn[:1]
        K.embed(rb.tokens, self.embed, h)
        tab.run(0, 1)
        n = tab.n_layers
        for li, L in enumerate(self.layers):
            kvl = kv_layers[li]
            if not K.paged_decode_attn_fused(qkv, self.inv_freq, L.q_norm, L.k_norm, rb.row_seq, rb.row_pos, block_table, kvl, geom,
                                             attn, rb.splits, self.ws, prefetch=True):
                K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, None)
                K.paged_decode_attn(q, rb.row_seq, rb.row_pos, block_table, kvl, geom, attn, rb.splits, self.ws, None)
            last = li == n - 1
            tab.run(1 + 4 * li, 4 if (not last or tab.head_in_table) else 3)
        if not tab.head_in_table:
            return self._head(h, buf, 1, rb)
        logits = buf.logits[:1]
        if self.head_split is not None and rb.full_logits:
            self.tp.gather_head(logits)
        return logits

    def forward_prefill_cp(self, rb: RowBatch, buf: Buffers, kv_layers, block_table) -> torch.Tensor:
        """Prefill chunk under context parallelism (parallel/cp.py): this rank runs its share of the chunk's rows (one early
        and one late piece, so that causal attention costs every rank the same) through every layer; per layer the ranks exchange the chunk's raw k | v rows, every rank appends the whole chunk's K / V to its
        own cache, and the local query rows attend over past and present keys.  Same arithmetic per row as ``forward``."""
        cfg, geom, cp = self.cfg, self.geom, self.cp
        M = rb.tokens.shape[0]
        a, b = cp.local_rows(M)              # exchange order: this rank's rows are contiguous there
        segs, perm = cp.layout(M)            # chunk rows behind them (two pieces under the balanced split)
        n = b - a
        eps, off = cfg.rms_norm_eps, cfg.norm_offset
        h, x = buf.h[:n], buf.x[:n]
        qkv, q, attn, act = buf.qkv[:M], buf.q[:M], buf.attn[:n], buf.act[:n]
        gate = buf.gate[:M] if buf.gate is not None else None
        qsz = geom.Hq * geom.D * (2 if geom.q_gated else 1)
        if perm is None:
            toks, row_pos, row_seq = rb.tokens[a:b], rb.row_pos, rb.row_seq
        else:
            toks = rb.tokens.index_select(0, perm[a:b])
            row_pos, row_seq = rb.row_pos.index_select(0, perm), rb.row_seq.index_select(0, perm)
        K.embed(toks, self.embed, h)
        T = rb.q_pos0 + M
        cp.stats["chunks"] += 1
        for li, L in enumerate(self.layers):
            kvl = kv_layers[li]
            tl = trace.timeline.on
            if tl: trace.mark("norm + qkv gemm")
            self._norm_linear(L.qkv, h, L.in_norm, x, qkv[a:b], "bf16", eps, off)
            if tl: trace.mark("k|v exchange")
            cp.exchange_kv(qkv, M, qsz, li & 1)
            if tl: trace.mark("rope + kv write")
            if rb.q_pos0 > 0:
                K.gather_kv_dense(kvl, block_table[rb.seq_slot], rb.q_pos0, buf.dense_k, buf.dense_v)
            # norm + RoPE + cache append for the whole chunk's keys (dense K / V land by position, whatever the row order);
            # queries for the local rows only
            K.rope_kvwrite(qkv, row_pos, row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm,
                           gate, buf.dense_k[rb.q_pos0: T], buf.dense_v[rb.q_pos0: T], dense_pos0=rb.q_pos0, q_rows=(a, n))
            if tl: trace.mark("flash prefill")
            o0 = 0
            for g0, cnt in segs:
                K.flash_prefill(q[a + o0: a + o0 + cnt], buf.dense_k, buf.dense_v, geom, attn[o0: o0 + cnt], rb.q_pos0 + g0,
                                None if gate is None else gate[a + o0: a + o0 + cnt])
                o0 += cnt
            if tl: trace.mark("o gemm")
            L.o(attn, h, "add_f32")
            if tl: trace.mark("norm + gate_up gemm")
            self._norm_linear(L.gate_up, h, L.post_norm, x, act, "swiglu", eps, off)
            if tl: trace.mark("down gemm")
            L.down(act, h, "add_f32")
        if trace.timeline.on: trace.mark("tail")
        # rows that need logits live on their owners: collect them on every rank
        rows = rb.logits_rows if rb.logits_rows is not None else torch.arange(M, device=self.device)
        nl = rows.shape[0]
        sel = torch.zeros(nl, cfg.hidden_size, dtype=torch.float32, device=self.device)
        owner, local = cp.owner_index(rows.long(), M)
        mine = owner == cp.rank
        if bool(mine.any()):
            sel[mine] = h.index_select(0, local[mine])
        torch.distributed.all_reduce(sel, group=cp.group)
        return self._head(sel, buf, nl, rb)

    def forward_ulysses(self, rb: RowBatch, buf: Buffers, kv_layers, block_table) -> torch.Tensor:
        """Head-parallel attention over whole-model replicas (parallel/ulysses.py).  ``self.geom`` and the KV cache hold this
        rank's heads only.  A prompt chunk whose rows divide over the ranks is row-split outside attention (two all-to-alls per
        layer); every other pass runs its projections replicated and all-gathers the attention output."""
        cfg, geom, up = self.cfg, self.geom, self.up
        M = rb.tokens.shape[0]
        eps, off = cfg.rms_norm_eps, cfg.norm_offset
        prefill = rb.mode == "prefill"
        if prefill and rb.segments is not None:
            raise NotImplementedError("several prompts in one pass are not built for the head / sequence exchange")
        split = prefill and up.split_ready(M)
        a, b = up.local_rows(M) if split else (0, M)
        n = b - a
        h, x, act = buf.h[:n], buf.x[:n], buf.act[:n]
        qkv_h, q, attn_h = buf.qkv[:M], buf.q[:M], buf.attn[:M]                  # local-head layouts, all M rows
        qw_full = up.full.Hq * up.full.D
        qkv_full = up.scratch("qkv_full", n, qw_full + 2 * up.full.Hkv * up.full.D)
        K.embed(rb.tokens[a:b], self.embed, h)
        T = rb.q_pos0 + M
        up.stats["split_chunks" if split else "replicated_passes"] += 1
        for li, L in enumerate(self.layers):
            kvl = kv_layers[li]
            self._norm_linear(L.qkv, h, L.in_norm, x, qkv_full, "bf16", eps, off)
            if split:
                qkv_h.copy_(up.rows_to_heads(qkv_full, M))
            else:
                qkv_h.copy_(up.head_columns(qkv_full, up.rank))
            if prefill:
                if rb.q_pos0 > 0:
                    K.gather_kv_dense(kvl, block_table[rb.seq_slot], rb.q_pos0, buf.dense_k, buf.dense_v)
                K.rope_kvwrite(qkv_h, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, None,
                               buf.dense_k[rb.q_pos0: T], buf.dense_v[rb.q_pos0: T])
                K.flash_prefill(q, buf.dense_k, buf.dense_v, geom, attn_h, rb.q_pos0, None)
            else:
                K.rope_kvwrite(qkv_h, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, None)
                if not (rb.verify is not None and K.paged_verify_attn(q, rb.verify[0], rb.verify[1], block_table, kvl, geom, attn_h,
                                                                      rb.splits, self.ws, None)):
                    K.paged_decode_attn(q, rb.row_seq, rb.row_pos, block_table, kvl, geom, attn_h, rb.splits, self.ws, None)
            attn = up.heads_to_rows(attn_h, M) if split else up.gather_heads(attn_h)
            L.o(attn, h, "add_f32")
            self._norm_linear(L.gate_up, h, L.post_norm, x, act, "swiglu", eps, off)
            L.down(act, h, "add_f32")
        rows = rb.logits_rows if rb.logits_rows is not None else torch.arange(M, device=self.device)
        nl = rows.shape[0]
        if not split:
            hsel = h.index_select(0, rows.long()) if nl != M else h
            return self._head(hsel, buf, nl, rb)
        sel = torch.zeros(nl, cfg.hidden_size, dtype=torch.float32, device=self.device)
        mine = (rows >= a) & (rows < b)
        if bool(mine.any()):
            sel[mine] = h.index_select(0, (rows[mine] - a).long())
        torch.distributed.all_reduce(sel, group=up.group)
        return self._head(sel, buf, nl, rb)

    def forward(self, rb: RowBatch, buf: Buffers, kv_layers, block_table) -> torch.Tensor:
        """Run all layers for the rows of ``rb``; returns fp32 logits [rows needing logits][V]."""
        if getattr(self, "up", None) is not None:
            return self.forward_ulysses(rb, buf, kv_layers, block_table)
        if (rb.mode == "prefill" and rb.segments is None and getattr(self, "cp", None) is not None and self.cp.ready(rb.tokens.shape[0])):
            return self.forward_prefill_cp(rb, buf, kv_layers, block_table)
        if (rb.mode == "prefill" and rb.segments is None and self.tp is not None and self.pp_world == 1 and getattr(self.tp, "sp_ready", None)
                and isinstance(self.layers[0].qkv, (W4Linear, RowQLinear)) and self.tp.sp_ready(rb.tokens.shape[0]) and self.tp.sp_enabled):
            return self.forward_prefill_sp(rb, buf, kv_layers, block_table)
        cfg, geom = self.cfg, self.geom
        M = rb.tokens.shape[0]
        if M == 1 and rb.mode == "decode" and not trace.timeline.on and self._mega_ready():
            return self.forward_mega(rb, buf, kv_layers, block_table)
        eps, off = cfg.rms_norm_eps, cfg.norm_offset
        h, x = buf.h[:M], buf.x[:M]
        qkv, q, attn, act = buf.qkv[:M], buf.q[:M], buf.attn[:M], buf.act[:M]
        gate = buf.gate[:M] if buf.gate is not None else None
        first_stage, last_stage = self.pp_rank == 0, self.pp_rank == self.pp_world - 1
        if first_stage:
            K.embed(rb.tokens, self.embed, h)
        else:
            self.pp.recv_hidden(h)          # [rows][H] from the previous stage
        prefill = rb.mode == "prefill"
        T = rb.q_pos0 + M
        tl = trace.timeline.on
        for li, L in enumerate(self.layers):
            kvl = kv_layers[li]
            if tl: trace.mark("norm+qkv")
            self._norm_linear(L.qkv, h, L.in_norm, x, qkv, "bf16", eps, off)
            if tl: trace.mark("rope+attn")
            if prefill and rb.segments is not None:
                # several fresh prompts in one pass: the projections see all M rows at once, attention runs per prompt
                # over that prompt's slice of the dense K / V rows
                K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm,
                               gate, buf.dense_k[:M], buf.dense_v[:M])
                for r0, n in rb.segments:
                    K.flash_prefill(q[r0: r0 + n], buf.dense_k[r0: r0 + n], buf.dense_v[r0: r0 + n], geom, attn[r0: r0 + n], 0,
                                    None if gate is None else gate[r0: r0 + n])
            elif prefill:
                if rb.q_pos0 > 0:
                    K.gather_kv_dense(kvl, block_table[rb.seq_slot], rb.q_pos0, buf.dense_k, buf.dense_v)
                K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm,
                               gate, buf.dense_k[rb.q_pos0: T], buf.dense_v[rb.q_pos0: T])
                K.flash_prefill(q, buf.dense_k, buf.dense_v, geom, attn, rb.q_pos0, gate)
            elif not ((M == 1 or rb.distinct) and gate is None and K.paged_decode_attn_fused(qkv, self.inv_freq, L.q_norm, L.k_norm, rb.row_seq, rb.row_pos,
                                                                          block_table, kvl, geom, attn, rb.splits, self.ws, prefetch=True)):
                K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, gate)
                if not (rb.verify is not None and K.paged_verify_attn(q, rb.verify[0], rb.verify[1], block_table, kvl, geom, attn,
                                                                      rb.splits, self.ws, gate)):
                    K.paged_decode_attn(q, rb.row_seq, rb.row_pos, block_table, kvl, geom, attn, rb.splits, self.ws, gate)
            if tl: trace.mark("o_proj")
            self._row_parallel(L.o, attn, h)
            if tl: trace.mark("norm+gate_up")
            self._norm_linear(L.gate_up, h, L.post_norm, x, act, "swiglu", eps, off)
            if tl: trace.mark("down")
            self._row_parallel(L.down, act, h)
            if self.tap_index:
                j = self.tap_index.get(self.layer_begin + li)
                if j is not None:            # residual stream after this layer, kept per row for a block drafter
                    buf.taps[:M, j].copy_(h)
        if tl: trace.mark("head")
        if not last_stage:
            self.pp.send_hidden(h)
            return None
        # head
        if rb.logits_rows is None:
            hsel, n = h, M
        else:
            n = rb.logits_rows.shape[0]
            hsel = h.index_select(0, rb.logits_rows) if n != M else h
        logits = self._head(hsel, buf, n, rb)
        if tl: trace.mark("end")
        return logits
