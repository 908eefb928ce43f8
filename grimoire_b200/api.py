"""Public API: the handles a front end needs.

Mirrors include/b70/grimoire_api.hpp:191-243 -- ``grimoire_new/load`` -> ``Grimoire.load``,
``grimoire_serve_generate(_batch)`` -> ``Grimoire.generate`` / ``generate_batch``,
``grimoire_scheduler_new/width/generate`` -> ``Grimoire.scheduler()`` and ``Scheduler.generate``,
``grimoire_prefix_slots_used`` -> ``prefix_slots_used``; the rank-worker entry points live in
``parallel/control.py`` (``worker_loop``, ``broadcast_request``, ``shutdown``).
"""
from __future__ import annotations

import os
import time
from typing import Callable, Optional, Sequence

import torch

from .config import EngineConfig
from .engine.engine import Engine, EngineLimits
from .engine.generation import CopyDrafter, GenerationOptions, SpecStats, generate_tokens
from .engine.sampling import SamplingOptions
from .models.config import PRESETS, ModelConfig
from .models.dense import DenseModel


class UnsupportedModel(ValueError):
    pass


# --proj values with a runtime projection: int4 g128 (default; 'native' keeps a stored int4 / MXFP4 / fp8 checkpoint's own
# format), MXFP4, block-scaled fp8 ('fp8'), and the byte-per-weight formats with per-row or per-32 scales
_SERVED_PROJ = ("int4", "native", "mxfp4", "fp8", "int8", "bf16", "mxfp8", "fp8_e4m3", "fp8_e5m2")


def is_hybrid(cfg: ModelConfig) -> bool:
    """Configurations served by ``HybridModel``: any linear-attention (Gated DeltaNet) layer or an MoE FFN."""
    from .models.config import LINEAR_ATTN

    return cfg.is_moe or any(t == LINEAR_ATTN for t in cfg.layer_types)


def unsupported_reason(cfg: ModelConfig, ec: EngineConfig) -> Optional[str]:
    """Refusal by name before any weight is read (unsupported_reason, grimoire.cpp:6969)."""
    if cfg.head_dim not in (64, 128, 256):
        return f"head_dim {cfg.head_dim} is not supported (64, 128, 256)"
    if cfg.is_sandwich:
        from .models.gemma4 import unsupported_gemma4

        if ec.tp_world > 1 or ec.pp_world > 1 or ec.ep_world > 1:
            return "the gemma4 / muse families are served on one GPU (no tensor / pipeline / expert parallel path is built for them)"
        return unsupported_gemma4(cfg)
    if is_hybrid(cfg):
        if not cfg.is_moe and ec.ep_world > 1:
            return "expert parallelism needs an MoE FFN"
        if cfg.is_k2 and ec.ep_world > 1:
            return "the K2-Horizon family is served on one GPU (its router is not built into the expert-parallel chain)"
        if cfg.is_qwen4_exp and ec.ep_world > 1:
            return "the Qwen4-Exp family is served on one GPU (its residual streams are not built into the expert-parallel chain)"
        if ec.tp_world > 1 or ec.pp_world > 1:
            return "the hybrid (DeltaNet + MoE) family scales by expert parallelism (multi EP); tensor / pipeline stages are not built for it"
        if cfg.num_experts % max(1, ec.ep_world):
            return f"expert parallel {ec.ep_world} does not divide {cfg.num_experts} experts"
        if cfg.hidden_size % 128 or cfg.moe_intermediate_size % 128 or (not cfg.is_moe and cfg.intermediate_size % 128):
            return "block-scaled fp8 / int4 g128 projections need widths that are multiples of 128"
        return None
    if ec.ep_world > 1:
        return "expert parallelism needs an MoE model"
    if ec.tp_world > 1:
        if cfg.num_attention_heads % ec.tp_world or cfg.num_key_value_heads % ec.tp_world:
            return f"tensor parallel {ec.tp_world} does not divide {cfg.num_attention_heads} q / {cfg.num_key_value_heads} kv heads"
        if cfg.intermediate_size and (cfg.intermediate_size // ec.tp_world) % cfg.quant_group:
            return "FFN slice per rank is not a multiple of the quantisation group"
    if ec.pp_world > cfg.num_hidden_layers:
        return f"pipeline parallel {ec.pp_world} exceeds {cfg.num_hidden_layers} layers"
    return None


def _find_artifact(path: str) -> Optional[str]:
    """``model-v3.grm`` itself, or a bundle directory that holds one."""
    if path.endswith(".grm") and os.path.isfile(path):
        return path
    cand = os.path.join(path, "model-v3.grm")
    return cand if os.path.isfile(cand) else None


class Grimoire:
    def __init__(self, model, engine: Engine, tokenizer=None, config: Optional[EngineConfig] = None, name: str = ""):
        self.model, self.engine, self.tokenizer = model, engine, tokenizer
        self.config = config or EngineConfig()
        self.name = name or self.config.model
        self.drafter = None            # models.mtp.MtpDrafter when the checkpoint carries a draft head and GRIMOIRE_MTP=1
        self._sched = None

    # ---- construction ----
    @classmethod
    def load(cls, ec: EngineConfig, device: Optional[str] = None, tp=None, pp=None, ep_group=None, up_group=None) -> "Grimoire":
        """Build model + engine for ``ec.model``: ``synthetic:<preset>``, a HF directory (dense or hybrid family), a
        ``.gguf`` file, or a pre-quantised artifact (``model-v3.grm`` / its bundle directory).  ``tp`` / ``pp`` are this
        rank's TensorParallel / PipelineParallel objects, ``ep_group`` the expert-parallel process group."""
        from .models.hybrid import HybridModel

        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        tok = None
        mtp_src = None                    # (state-dict-like getter, config) for the draft head
        ck_dir = None
        if ec.proj == "fp8-e5m2" or ec.proj == "fp8-e4m3":
            ec.proj = ec.proj.replace("-", "_")
        if ec.model.startswith("synthetic:"):
            preset = ec.model.split(":", 1)[1]
            if preset not in PRESETS:
                raise UnsupportedModel(f"unknown synthetic preset {preset!r}; choose from {sorted(PRESETS)}")
            cfg = PRESETS[preset]()
            why = unsupported_reason(cfg, ec)
            if why:
                raise UnsupportedModel(why)
            if cfg.is_sandwich:
                from .models.gemma4 import Gemma4Model, MuseModel

                model = (MuseModel if cfg.is_muse else Gemma4Model).random(cfg, dev, seed=0)
            elif cfg.is_qwen4_exp:
                from .models.qwen4_exp import Qwen4ExpModel

                model = Qwen4ExpModel.random(cfg, dev, seed=0, max_slots=ec.seq_slots)
            elif is_hybrid(cfg):
                model = HybridModel.random(cfg, dev, seed=0, max_slots=ec.seq_slots, ep_rank=ec.ep_rank, ep_world=ec.ep_world)
            else:
                model = DenseModel.random(cfg, dev, seed=0, tp_rank=ec.tp_rank, tp_world=ec.tp_world, pp_rank=ec.pp_rank,
                                          pp_world=ec.pp_world)
        else:
            from .tokenizer import Tokenizer

            if ec.proj not in _SERVED_PROJ:
                raise UnsupportedModel(f"--proj {ec.proj}: this build serves {sorted(_SERVED_PROJ)}")
            art = _find_artifact(ec.model)
            if art is not None:
                from .formats.artifact import load_artifact_model

                ck_dir = os.path.dirname(art)
                cfg = ModelConfig.from_dir(ck_dir)
                why = unsupported_reason(cfg, ec)
                if why:
                    raise UnsupportedModel(why)
                model, mtp_src = load_artifact_model(art, cfg, dev, ec)
            elif ec.model.endswith(".gguf"):
                # GGUF: config and tokenizer from the metadata.  --proj native on one rank keeps the file's blocks and runs
                # the projections over the raw bytes (when every projection's block type is served); otherwise tensors
                # are dequantised block by block and re-quantised to the serving format
                import dataclasses
                import json as _json
                import tempfile
                from .formats import gguf as G

                gf = G.GGUFFile(ec.model)
                cfg = G.config_from_gguf(gf)
                if ec.proj not in ("int4", "native"):
                    cfg = dataclasses.replace(cfg, quant=ec.proj)
                why = unsupported_reason(cfg, ec)
                if why:
                    raise UnsupportedModel(why)
                if cfg.is_gemma4:
                    from .models.gemma4 import Gemma4Model

                    model = Gemma4Model.from_state_dict(cfg, G.state_dict_from_gguf(gf), dev)
                elif is_hybrid(cfg):
                    # qwen35 / qwen35moe / qwen3moe files: the converter's tensor transforms are undone on the way in
                    from .models.hybrid import _DictSource

                    model_src = _DictSource(cfg, G.state_dict_from_gguf(gf, cfg))
                    model = HybridModel.from_checkpoint(model_src, dev, max_slots=ec.seq_slots,
                                                        ep_rank=ec.ep_rank, ep_world=ec.ep_world,
                                                        expert_heat=os.environ.get("GRIMOIRE_EXPERT_HEAT", ""),
                                                        proj=None if cfg.is_moe else {"int4": "int4", "fp8": "fp8"}.get(ec.proj))
                    if ec.mtp and cfg.mtp_num_hidden_layers > 0 and not cfg.is_moe and "mtp.fc.weight" in model_src.sd:
                        mtp_src = model_src              # the file's nextn block under the mtp.* names
                elif ec.proj == "native" and ec.tp_world == 1 and ec.pp_world == 1 and G.native_ok(gf, cfg):
                    model = DenseModel.from_gguf_native(cfg, gf, dev)
                else:
                    model = DenseModel.from_state_dict(cfg, G.state_dict_from_gguf(gf), dev, ec.tp_rank, ec.tp_world, pp_rank=ec.pp_rank,
                                                       pp_world=ec.pp_world)
                tj = G.tokenizer_json_from_gguf(gf)
                if tj is not None:
                    tdir = tempfile.mkdtemp(prefix="grimoire_tok_")
                    with open(os.path.join(tdir, "tokenizer.json"), "w") as f:
                        _json.dump(tj, f)
                    with open(os.path.join(tdir, "tokenizer_config.json"), "w") as f:
                        _json.dump(G.tokenizer_config_from_gguf(gf), f)
                    tok = Tokenizer(tdir)
                gf.close()
            else:
                ck_dir = ec.model
                cfg = ModelConfig.from_dir(ec.model)
                why = unsupported_reason(cfg, ec)
                if why:
                    raise UnsupportedModel(why)
                if cfg.is_sandwich:
                    from .models.gemma4 import Gemma4Model, MuseModel

                    model = (MuseModel if cfg.is_muse else Gemma4Model).from_checkpoint(ec.model, dev)
                elif cfg.is_qwen4_exp:
                    from .models.qwen4_exp import Qwen4ExpModel

                    model = Qwen4ExpModel.from_checkpoint(ec.model, dev, max_slots=ec.seq_slots)
                elif is_hybrid(cfg):
                    model = HybridModel.from_checkpoint(ec.model, dev, max_slots=ec.seq_slots, ep_rank=ec.ep_rank, ep_world=ec.ep_world,
                                                        expert_heat=os.environ.get("GRIMOIRE_EXPERT_HEAT", ""),
                                                        vram_experts=int(os.environ.get("GRIMOIRE_EXPERT_VRAM_PER_LAYER", "0") or 0),
                                                        proj=None if cfg.is_moe else {"int4": "int4", "fp8": "fp8"}.get(ec.proj))
                    if ec.mtp and cfg.mtp_num_hidden_layers > 0 and not cfg.is_moe and ec.ep_world == 1:
                        from .formats.checkpoint import Checkpoint

                        ck = Checkpoint(ec.model)
                        if ck.has("mtp.fc.weight"):
                            mtp_src = ck                 # the 27B-style hybrid's draft layer: full attention + dense FFN
                else:
                    model = DenseModel.from_checkpoint(ec.model, dev, ec.tp_rank, ec.tp_world, lm_head_bf16=bool(ec.lm_head_bf16),
                                                       proj=ec.proj, pp_rank=ec.pp_rank, pp_world=ec.pp_world)
                    if ec.mtp and cfg.mtp_num_hidden_layers > 0:
                        from .formats.checkpoint import Checkpoint

                        ck = Checkpoint(ec.model)
                        if ck.has("mtp.fc.weight"):
                            mtp_src = ck
            if ck_dir and tok is None and os.path.exists(os.path.join(ck_dir, "tokenizer.json")):
                tok = Tokenizer(ck_dir)
        hybrid = isinstance(model, HybridModel)
        if hybrid and getattr(model, "vram_experts", 0) and int(os.environ.get("GRIMOIRE_EXPERT_SWAPS", "0") or 0) > 0:
            model.enable_expert_swaps(int(os.environ["GRIMOIRE_EXPERT_SWAPS"]))      # hot host experts move onto the device as traffic shifts
        if hybrid and os.environ.get("GRIMOIRE_EXPERT_HITS"):
            model.record_expert_hits(os.environ["GRIMOIRE_EXPERT_HITS"])     # the file GRIMOIRE_EXPERT_HEAT reads at the next load
        if tp is not None:
            tp.attach(model, max_rows=max(ec.prefill_chunk, 64))
            if not hybrid and pp is None:
                tp.split_head(model)             # 1/W of the lm_head per rank; tokens by (value, index) exchange
        if pp is not None:
            pp.attach(model)
        if hybrid and ep_group is not None and ec.ep_world > 1:
            model.attach_ep(ep_group, max_rows=max(ec.prefill_chunk, 64))
        if up_group is not None:
            # head / sequence exchange over whole-model replicas: the KV pool below is sized from the (now local) head geometry
            from .parallel.ulysses import UlyssesParallel

            if hybrid or cfg.is_sandwich or ec.tp_world > 1 or ec.pp_world > 1:
                raise UnsupportedModel("the head / sequence exchange (multi UP) runs over whole replicas of the dense decoder family")
            UlyssesParallel(up_group, dev).attach(model)
        # draft head: on a single-stage, single-rank dense model or dense-FFN hybrid (the reference drafts on the last stage)
        want_mtp = mtp_src is not None and ec.tp_world == 1 and ec.pp_world == 1
        lim = EngineLimits(max_slots=ec.seq_slots, max_ctx=ec.ctx, prefill_chunk=ec.prefill_chunk, max_decode_rows=64,
                           kv_pages=ec.kv_pages, extra_kv_layers=1 if want_mtp else 0)
        eng = Engine(model, lim)
        if ec.prefix_cache and not cfg.is_qwen4_exp:       # that family's n-gram history and convolution tails are not snapshotted
            eng.enable_prefix_cache()
        g = cls(model, eng, tok, ec)
        if want_mtp:
            from .models.mtp import MtpDrafter, MtpHead

            g.drafter = MtpDrafter(eng, MtpHead.from_checkpoint(model, mtp_src, draft_vocab=ec.mtp_draft_vocab))
        elif ec.dflash_model:
            # --dflash-model: a block drafter over the target's residual taps (dense family, one GPU)
            if hybrid or ec.tp_world > 1 or ec.pp_world > 1:
                raise UnsupportedModel("the block drafter (--dflash-model) runs beside a single-GPU dense target")
            from .models.dflash_drafter import load_dflash

            g.drafter = load_dflash(ec.dflash_model, eng)
        g.banner()
        return g

    def banner(self) -> str:
        """Capability matrix: what is ACTUALLY active (grimoire.cpp:10488-10625)."""
        ec, m = self.config, self.model
        lines = [
            f"[grimoire-b200] model={self.name or 'synthetic'} layers={m.cfg.num_hidden_layers} hidden={m.cfg.hidden_size} "
            f"heads={m.cfg.num_attention_heads}/{m.cfg.num_key_value_heads}x{m.cfg.head_dim} vocab={m.cfg.vocab_size}",
            f"  parallel   : tp={m.tp_world} (fused all-reduce={'on' if getattr(m, 'tp', None) and m.tp.fused else 'off'}) pp={ec.pp_world} "
            f"ep={getattr(m, 'ep_world', 1)} dp={ec.dp_world}",
            f"  weights    : {'block-scaled fp8 (e4m3, 1x128)' if getattr(m, 'kv_layer_count', None) is not None else ec.proj + ' g' + str(m.cfg.quant_group)} "
            f"({m.weight_bytes() / 1e9:.2f} GB on this rank), draft head={type(self.drafter).__name__ if self.drafter is not None else 'none'}",
            f"  kv cache   : int8 paged, {self.engine.kv.num_pages} pages x 16 tokens, {self.engine.kv.bytes_per_token()} B/token",
            f"  batching   : width {ec.width()}, prefill chunk {ec.prefill_chunk}, interleave chunk {ec.interleave_chunk}",
            f"  speculation: copy drafts={'on' if ec.copy_drafts else 'off'} depth table {ec.spec_depth_table()}",
            f"  prefix     : {'on' if self.engine.prefix_cache is not None else 'off'}",
            f"  norms      : {'zero-centred (1+w)' if m.cfg.norm_zero_centered else 'plain w'}",
        ]
        text = "\n".join(lines)
        print(text, flush=True)
        return text

    # ---- single request path (CLI, workers) ----
    def generate(self, prompt_ids: Sequence[int], max_new: int, eos: Optional[int] = None, eos2: Optional[int] = None,
                 on_token: Optional[Callable[[int], bool]] = None, draft_depth: int = 0, stats: Optional[SpecStats] = None):
        drafter = None
        if draft_depth:
            drafter = self.drafter if self.drafter is not None else CopyDrafter()
        opts = GenerationOptions(max_new=max_new, eos=eos, eos2=eos2, draft_depth=draft_depth, drafter=drafter,
                                 stats=stats or SpecStats())
        return generate_tokens(self.engine, list(prompt_ids), opts, on_token)

    def generate_batch(self, prompts: Sequence[Sequence[int]], max_new: int, eos: Optional[int] = None):
        """Several prompts through the scheduler at once; returns a list of (tokens, reason)."""
        import threading

        s = self.scheduler()
        res = [None] * len(prompts)

        def work(i):
            out, why, _ = s.generate(list(prompts[i]), max_new, eos)
            res[i] = (out, why)

        ts = [threading.Thread(target=work, args=(i,)) for i in range(len(prompts))]
        [t.start() for t in ts]
        [t.join() for t in ts]
        return res

    def scheduler(self):
        if self._sched is None:
            from .sched.scheduler import Scheduler

            ec = self.config
            spec = self.drafter is not None or (ec.copy_drafts and getattr(self.model, "supports_verify_rows", True))
            self._sched = Scheduler(self.engine, width=ec.width(), interleave_chunk=ec.interleave_chunk,
                                    prefill_chunk=ec.prefill_chunk, hold_ms=ec.admit_hold_ms, hold_long_ms=ec.admit_hold_long_ms,
                                    depths=ec.spec_depth_table() if spec else (0,), spec_rows=ec.spec_rows,
                                    copy_drafts=bool(ec.copy_drafts) and spec, drafter=self.drafter)
        return self._sched

    def prefix_slots_used(self) -> int:
        return len(self.engine.prefix_cache.entries) if self.engine.prefix_cache is not None else 0

    def close(self) -> None:
        if self._sched is not None:
            self._sched.shutdown()
            self._sched = None
        save = getattr(self.model, "save_expert_hits", None)
        if save is not None:
            save()

    # ---- CLI helpers: load report / micro benchmarks / scoring ----
    def bench_prefill(self, n_tokens: int, repeats: int = 2) -> float:
        """tokens/s reading a random prompt of n_tokens (grimoire_bench_prefill, grimoire.cpp:12905)."""
        g = torch.Generator().manual_seed(0)
        ids = torch.randint(0, self.model.cfg.vocab_size, (n_tokens,), generator=g).tolist()
        best = 0.0
        for _ in range(repeats + 1):
            s = self.engine.open()
            t0 = time.perf_counter()
            self.engine.prefill(s, ids)
            if self.engine.device.type == "cuda":
                torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            self.engine.release(s)
            best = max(best, n_tokens / dt)
        return best

    def bench_decode(self, n_tokens: int = 64, prompt: int = 128) -> float:
        """tokens/s of plain greedy decode (grimoire_bench_decode, grimoire.cpp:13190)."""
        g = torch.Generator().manual_seed(0)
        ids = torch.randint(0, self.model.cfg.vocab_size, (prompt,), generator=g).tolist()
        self.engine.generate(ids, 8)
        t0 = time.perf_counter()
        self.engine.generate(ids, n_tokens)
        return n_tokens / (time.perf_counter() - t0)

    def score_ids(self, ids: Sequence[int]) -> torch.Tensor:
        """fp32 logits for every position of ``ids`` (``--score-ids/--score-out``: accuracy checks
        against another implementation's logits)."""
        out = []
        s = self.engine.open()
        try:
            lg = self.engine.prefill(s, [ids[0]])
            out.append(lg.float().cpu())
            for i in range(1, len(ids)):
                _, l2 = self.engine.decode_rows([ids[i]], [s], [s.length], use_graph=False, return_logits=True)
                self.engine.commit_rows([s], [ids[i]], [s.length])
                out.append(l2[0].float().cpu().clone())
        finally:
            self.engine.release(s)
        return torch.stack(out)

    def perplexity(self, ids: Sequence[int], ctx: int = 512, chunks: int = 0, dump: str = "", selfcheck: bool = False,
                   kld_base: str = "") -> dict:
        """Perplexity over complete ``ctx``-token chunks, teacher-forced one row per step from a fresh conversation, scoring
        the second half of each chunk (positions ctx/2 .. ctx-2 predict their successors) with a running mean and its standard
        error (``--ppl FILE --ppl-ctx --ppl-chunks --ppl-dump --ppl-selfcheck``, grimoire_perplexity grimoire.cpp:23734-23905).
        ``dump``: a TSV line per scored token -- chunk, position, target, its log-probability, the best token and its
        log-probability, then the eight best ``id:logprob``.  ``selfcheck``: the decode logits of the first chunk's last
        scored position against a batched prefill of the same prefix.  ``kld_base``: a llama-perplexity
        ``--kl-divergence-base`` file; the chunks, their tokens and the context length come from it (``ids`` is unused), and
        the result carries the KL-divergence / probability statistics against its rows under ``"kld"``."""
        import math

        V = self.model.cfg.vocab_size
        base = kstats = None
        if kld_base:
            from .utils.kld import KldBase, KldStats

            base, kstats = KldBase(kld_base), KldStats()
            if base.vocab != V:
                raise ValueError(f"vocabulary mismatch (base {base.vocab}, model {V})")
            if chunks > base.chunks:
                raise ValueError(f"more chunks asked than the base file has ({base.chunks})")
            ctx = base.ctx
            ids = [int(t) for c in range(base.chunks) for t in base.read_chunk(c)[0]]
        count = len(ids) // ctx
        if chunks:
            count = min(count, chunks)
        if count < 1:
            raise ValueError(f"{len(ids)} tokens, no complete {ctx}-token chunk")
        if any(t < 0 or t >= V for t in ids[: count * ctx]):
            raise ValueError("a token id lies outside the model's vocabulary")
        if dump and V < 8:
            raise ValueError("the dump lists eight candidates: the vocabulary is smaller")
        out = open(dump, "w") if dump else None
        scored, mean, m2 = 0, 0.0, 0.0
        res: dict = {}
        try:
            for c in range(count):
                w = list(ids[c * ctx: (c + 1) * ctx])
                lg = self.score_ids(w[:-1]).double()                    # row p predicts token p + 1
                if base is not None:
                    _, sc, mn, q = base.read_chunk(c)
                    kstats.add_rows(lg[ctx // 2: ctx - 1].float().numpy(), sc, mn, q, w[ctx // 2 + 1: ctx])
                for pos in range(ctx // 2, ctx - 1):
                    row = lg[pos]
                    if not bool(torch.isfinite(row).all()):
                        raise ValueError(f"non-finite logits at position {pos}")
                    lp = row - torch.logsumexp(row, 0)
                    nll = -float(lp[w[pos + 1]])
                    scored += 1
                    delta = nll - mean
                    mean += delta / scored
                    m2 += delta * (nll - mean)
                    if out is not None:
                        top = torch.topk(lp, 8)
                        best = int(top.indices[0])
                        out.write("\t".join([str(c + 1), str(pos), str(w[pos + 1]), f"{-nll:.12g}", str(best), f"{float(lp[best]):.12g}"]
                                            + [f"{int(i)}:{float(v):.12g}" for v, i in zip(top.values, top.indices)]) + "\n")
                if selfcheck and c == 0:
                    s = self.engine.open()
                    try:
                        pre = self.engine.prefill(s, w[:-1]).double().cpu()
                    finally:
                        self.engine.release(s)
                    if not bool(torch.isfinite(pre).all()):
                        raise ValueError("non-finite prefill logits")
                    res["selfcheck_max_abs_diff"] = float((pre - lg[ctx - 2]).abs().max())
        finally:
            if out is not None:
                out.close()
        ppl = math.exp(mean)
        se = math.sqrt(m2 / (scored - 1) / scored) if scored > 1 else 0.0
        res.update({"ppl": ppl, "ppl_stderr": ppl * se, "tokens": scored, "chunks": count, "nll": mean * scored})
        if kstats is not None:
            res["kld"] = kstats.summary()
            res["kld_report"] = kstats.report()
        return res
