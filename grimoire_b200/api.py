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


def unsupported_reason(cfg: ModelConfig, ec: EngineConfig) -> Optional[str]:
    """Refusal by name before any weight is read (unsupported_reason, grimoire.cpp:6969)."""
    if ec.tp_world > 1:
        if cfg.num_attention_heads % ec.tp_world or cfg.num_key_value_heads % ec.tp_world:
            return f"tensor parallel {ec.tp_world} does not divide {cfg.num_attention_heads} q / {cfg.num_key_value_heads} kv heads"
        if cfg.intermediate_size and (cfg.intermediate_size // ec.tp_world) % cfg.quant_group:
            return "FFN slice per rank is not a multiple of the quantisation group"
    if cfg.head_dim not in (64, 128, 256):
        return f"head_dim {cfg.head_dim} is not supported (64, 128, 256)"
    return None


class Grimoire:
    def __init__(self, model, engine: Engine, tokenizer=None, config: Optional[EngineConfig] = None, name: str = ""):
        self.model, self.engine, self.tokenizer = model, engine, tokenizer
        self.config = config or EngineConfig()
        self.name = name or self.config.model
        self._sched = None

    # ---- construction ----
    @classmethod
    def load(cls, ec: EngineConfig, device: Optional[str] = None, tp=None) -> "Grimoire":
        dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        tok = None
        if ec.model.startswith("synthetic:"):
            preset = ec.model.split(":", 1)[1]
            if preset not in PRESETS:
                raise UnsupportedModel(f"unknown synthetic preset {preset!r}; choose from {sorted(PRESETS)}")
            cfg = PRESETS[preset]()
            why = unsupported_reason(cfg, ec)
            if why:
                raise UnsupportedModel(why)
            model = DenseModel.random(cfg, dev, seed=0, tp_rank=ec.tp_rank, tp_world=ec.tp_world)
        else:
            from .tokenizer import Tokenizer

            if ec.proj == "fp8-e5m2" or ec.proj == "fp8-e4m3":
                ec.proj = ec.proj.replace("-", "_")
            if ec.proj not in _SERVED_PROJ:
                raise UnsupportedModel(f"--proj {ec.proj}: this build serves {sorted(_SERVED_PROJ)}")
            if ec.model.endswith(".gguf"):
                # GGUF: config and tokenizer from the metadata, tensors dequantised block by block and re-quantised
                # to the serving format (the reference's native GGUF path keeps the file's blocks; this one does not)
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
                model = DenseModel.from_state_dict(cfg, G.state_dict_from_gguf(gf), dev, ec.tp_rank, ec.tp_world)
                tj = G.tokenizer_json_from_gguf(gf)
                if tj is not None:
                    tdir = tempfile.mkdtemp(prefix="grimoire_tok_")
                    with open(os.path.join(tdir, "tokenizer.json"), "w") as f:
                        _json.dump(tj, f)
                    tok = Tokenizer(tdir)
                gf.close()
            else:
                cfg = ModelConfig.from_dir(ec.model)
                why = unsupported_reason(cfg, ec)
                if why:
                    raise UnsupportedModel(why)
                model = DenseModel.from_checkpoint(ec.model, dev, ec.tp_rank, ec.tp_world, lm_head_bf16=bool(ec.lm_head_bf16),
                                                   proj=ec.proj)
                if os.path.exists(os.path.join(ec.model, "tokenizer.json")):
                    tok = Tokenizer(ec.model)
        if tp is not None:
            tp.attach(model, max_rows=max(ec.prefill_chunk, 64))
        lim = EngineLimits(max_slots=ec.seq_slots, max_ctx=ec.ctx, prefill_chunk=ec.prefill_chunk, max_decode_rows=64,
                           kv_pages=ec.kv_pages)
        eng = Engine(model, lim)
        if ec.prefix_cache:
            eng.enable_prefix_cache()
        g = cls(model, eng, tok, ec)
        g.banner()
        return g

    def banner(self) -> str:
        """Capability matrix: what is ACTUALLY active (grimoire.cpp:10488-10625)."""
        ec, m = self.config, self.model
        lines = [
            f"[grimoire-b200] model={self.name or 'synthetic'} layers={m.cfg.num_hidden_layers} hidden={m.cfg.hidden_size} "
            f"heads={m.cfg.num_attention_heads}/{m.cfg.num_key_value_heads}x{m.cfg.head_dim} vocab={m.cfg.vocab_size}",
            f"  parallel   : tp={m.tp_world} (fused all-reduce={'on' if getattr(m, 'tp', None) and m.tp.fused else 'off'}) pp={ec.pp_world} dp={ec.dp_world}",
            f"  weights    : int4 g{m.cfg.quant_group} ({m.weight_bytes() / 1e9:.2f} GB on this rank), lm_head={'tied bf16' if m.cfg.tie_word_embeddings else 'int4'}",
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
        opts = GenerationOptions(max_new=max_new, eos=eos, eos2=eos2, draft_depth=draft_depth,
                                 drafter=CopyDrafter() if draft_depth else None, stats=stats or SpecStats())
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
            self._sched = Scheduler(self.engine, width=ec.width(), interleave_chunk=ec.interleave_chunk,
                                    prefill_chunk=ec.prefill_chunk, hold_ms=ec.admit_hold_ms, hold_long_ms=ec.admit_hold_long_ms,
                                    depths=ec.spec_depth_table() if ec.copy_drafts else (0,), spec_rows=ec.spec_rows,
                                    copy_drafts=bool(ec.copy_drafts))
        return self._sched

    def prefix_slots_used(self) -> int:
        return len(self.engine.prefix_cache.entries) if self.engine.prefix_cache is not None else 0

    def close(self) -> None:
        if self._sched is not None:
            self._sched.shutdown()
            self._sched = None

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

    def perplexity(self, ids: Sequence[int], ctx: int = 512, chunks: int = 0) -> dict:
        """Perplexity over fixed windows (``--ppl FILE --ppl-ctx --ppl-chunks``, grimoire_perplexity
        grimoire.cpp:23734)."""
        import math

        nll, n = 0.0, 0
        windows = [ids[i: i + ctx] for i in range(0, len(ids) - 1, ctx)]
        if chunks:
            windows = windows[:chunks]
        for w in windows:
            if len(w) < 2:
                continue
            lg = self.score_ids(w)
            lp = torch.log_softmax(lg[:-1].double(), dim=-1)
            tgt = torch.tensor(w[1:])
            nll -= float(lp[torch.arange(len(w) - 1), tgt].sum())
            n += len(w) - 1
        return {"ppl": math.exp(nll / max(n, 1)), "tokens": n, "nll": nll}
