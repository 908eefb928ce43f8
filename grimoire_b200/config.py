"""Typed engine configuration filled from the CLI flags and the user-facing ``GRIMOIRE_*`` variables.

The reference has no config file: a handful of flags on ``grimoire`` / ``grimoire-server``
(tools/grimoire_server.cpp:148-184, tools/grimoire_main.cpp:66-167) plus 419 environment variables
read with ``getenv`` at the point of use.  Here the same flag names and the user-facing variables
land in one validated dataclass; kernel A/B switches become ``--kernel-override key=value`` and an
unknown ``GRIMOIRE_*`` name is reported instead of being silently ignored.
"""
from __future__ import annotations

import argparse
import os
import sys
from dataclasses import dataclass, field, fields
from typing import Optional

from .formats.codecs import PROJ_NAMES

# variable -> (field, type)
_ENV = {
    "GRIMOIRE_SEQ_SLOTS": ("seq_slots", int),
    "GRIMOIRE_MAX_BATCH": ("max_batch", int),
    "GRIMOIRE_MTP": ("mtp", int),
    "GRIMOIRE_MTP_K": ("mtp_k", int),
    "GRIMOIRE_MTP_DRAFT_VOCAB": ("mtp_draft_vocab", int),
    "GRIMOIRE_KV_POOL": ("kv_pool", int),
    "GRIMOIRE_KV_PAGES": ("kv_pages", int),
    "GRIMOIRE_PREFIX_CACHE": ("prefix_cache", int),
    "GRIMOIRE_PREFILL_CHUNK": ("prefill_chunk", int),
    "GRIMOIRE_INTERLEAVE_CHUNK": ("interleave_chunk", int),
    "GRIMOIRE_TP_RANK": ("tp_rank", int),
    "GRIMOIRE_TP_WORLD_SIZE": ("tp_world", int),
    "GRIMOIRE_PP_RANK": ("pp_rank", int),
    "GRIMOIRE_PP_WORLD_SIZE": ("pp_world", int),
    "GRIMOIRE_DP_WORLD_SIZE": ("dp_world", int),
    "GRIMOIRE_EP_WORLD_SIZE": ("ep_world", int),
    "GRIMOIRE_EP_RANK": ("ep_rank", int),
    "GRIMOIRE_CP_WORLD_SIZE": ("cp_world", int),
    "GRIMOIRE_SPEC_ROWS": ("spec_rows", int),
    "GRIMOIRE_SPEC_DEPTHS": ("spec_depths", str),
    "GRIMOIRE_SPEC_MAX_SEQS": ("spec_max_seqs", int),
    "GRIMOIRE_SPEC_STATS": ("spec_stats", int),
    "GRIMOIRE_COPY": ("copy_drafts", int),
    "GRIMOIRE_LM_HEAD_BF16": ("lm_head_bf16", int),
    "GRIMOIRE_ADMIT_HOLD_MS": ("admit_hold_ms", float),
    "GRIMOIRE_ADMIT_HOLD_LONG_MS": ("admit_hold_long_ms", float),
    "GRIMOIRE_TP_FUSED": ("tp_fused", int),
    "GRIMOIRE_TIMELINE": ("timeline", int),
    "GRIMOIRE_DEBUG": ("debug", int),
    "GRIMOIRE_STEP_LOG": ("step_log", str),
}
# read elsewhere at the point of use (documented, not part of EngineConfig)
_KNOWN_OTHER = {"GRIMOIRE_CP_BALANCED", "GRIMOIRE_FLASH_WS", "GRIMOIRE_GDN_SOLO", "GRIMOIRE_GDN_MMA", "GRIMOIRE_DFLASH_M", "GRIMOIRE_EXPERT_HEAT", "GRIMOIRE_EXPERT_HITS", "GRIMOIRE_EXPERT_VRAM_PER_LAYER", "GRIMOIRE_EXPERT_SWAPS", "GRIMOIRE_ROUTE_TRACE", "GRIMOIRE_CPU_EXPERT_THREADS", "GRIMOIRE_PDL", "GRIMOIRE_TP_HEAD_SPLIT", "GRIMOIRE_W4_BF16_CACHE_GB", "GRIMOIRE_W4_TC", "GRIMOIRE_VERIFY_ATTN", "GRIMOIRE_VERIFY_ATTN_MIN_CTX", "GRIMOIRE_CP_FUSED", "GRIMOIRE_NO_AUTOBUILD", "GRIMOIRE_HOST_LIB", "GRIMOIRE_MEGA", "GRIMOIRE_MEGA_COOP", "GRIMOIRE_MEGA_SPIN", "GRIMOIRE_MEGA_SLOTS", "GRIMOIRE_MEGA_TUNE", "GRIMOIRE_GGUF_GOLDEN_DIR", "GRIMOIRE_TP_SPIN", "GRIMOIRE_TP_SOCKET", "GRIMOIRE_PP_SOCKET"}


@dataclass
class EngineConfig:
    model: str = ""
    proj: str = "int4"                 # --proj {int4,int8,mxfp4,mxfp8,fp8,fp8_e5m2,bf16,native}
    ctx: int = 8192                    # --ctx
    port: int = 8000                   # --port
    host: str = "0.0.0.0"              # --host
    dflash_model: str = ""             # --dflash-model
    defer_moe_gather: bool = False
    bf16_qkv: bool = False
    bf16_dn_qkv: bool = False
    # scheduling
    seq_slots: int = 8
    max_batch: int = 8
    prefill_chunk: int = 4096
    interleave_chunk: int = 1024
    admit_hold_ms: float = 8.0
    admit_hold_long_ms: float = 100.0
    kv_pool: int = 1
    kv_pages: int = 0
    prefix_cache: int = 1
    # speculation
    mtp: int = 1
    mtp_k: int = 4
    mtp_draft_vocab: int = 0
    spec_rows: int = 32
    spec_depths: str = "15,5,4,3"
    spec_max_seqs: int = 16
    spec_stats: int = 0
    copy_drafts: int = 1
    lm_head_bf16: int = 0
    # parallel layout
    tp_rank: int = 0
    tp_world: int = 1
    pp_rank: int = 0
    pp_world: int = 1
    dp_world: int = 1
    ep_world: int = 1
    ep_rank: int = 0
    cp_world: int = 1
    tp_fused: int = 1
    # diagnostics
    timeline: int = 0
    debug: int = 0
    step_log: str = ""
    trace: bool = False
    kernel_override: dict = field(default_factory=dict)
    unknown_env: list = field(default_factory=list)

    def validate(self) -> "EngineConfig":
        if self.proj not in PROJ_NAMES and self.proj != "native":
            raise ValueError(f"--proj {self.proj!r}: expected one of {sorted(PROJ_NAMES)} or 'native'")
        if self.ctx < 16:
            raise ValueError("--ctx must be at least 16")
        if not (1 <= self.port <= 65535):
            raise ValueError("--port out of range")
        for name in ("seq_slots", "max_batch", "prefill_chunk", "tp_world", "pp_world", "dp_world", "ep_world", "cp_world"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be >= 1")
        if not (0 <= self.tp_rank < self.tp_world) or not (0 <= self.pp_rank < self.pp_world) or not (0 <= self.ep_rank < self.ep_world):
            raise ValueError("rank outside its world size")
        if self.mtp_k < 0 or self.mtp_k > 16:
            raise ValueError("GRIMOIRE_MTP_K must be in 0..16")
        return self

    def spec_depth_table(self) -> list[int]:
        """Draft depth by number of live conversations (index 0 = one user), the reference's
        "15,5,4,3,..." table (grimoire.cpp:11401-11431); the last entry repeats."""
        vals = [int(v) for v in self.spec_depths.split(",") if v.strip()]
        return vals or [self.mtp_k]

    def width(self) -> int:
        return max(1, min(self.max_batch, self.seq_slots))


def add_engine_flags(ap: argparse.ArgumentParser) -> None:
    ap.add_argument("--model", "-m", default="", help="HF directory, .gguf file or pre-quantized artifact")
    ap.add_argument("--proj", default="int4", help="projection format: int4 int8 mxfp4 mxfp8 fp8 (block-scaled) fp8_e4m3 fp8_e5m2 bf16 native")
    ap.add_argument("--ctx", type=int, default=8192, help="context cap per request")
    ap.add_argument("--dflash-model", default="", help="optional block drafter checkpoint")
    ap.add_argument("--defer-moe-gather", action="store_true")
    ap.add_argument("--bf16-qkv", action="store_true")
    ap.add_argument("--bf16-dn-qkv", action="store_true")
    ap.add_argument("--trace", action="store_true", help="record one steady decode step and one prefill chunk")
    ap.add_argument("--kernel-override", action="append", default=[], metavar="KEY=VALUE")


def from_args(ns: argparse.Namespace, env: Optional[dict] = None, warn=None) -> EngineConfig:
    env = os.environ if env is None else env
    cfg = EngineConfig()
    names = {f.name for f in fields(EngineConfig)}
    for k, v in vars(ns).items():
        if k in names and v is not None and k != "kernel_override":
            setattr(cfg, k, v)
    for item in getattr(ns, "kernel_override", []) or []:
        if "=" not in item:
            raise ValueError(f"--kernel-override {item!r}: expected KEY=VALUE")
        k, v = item.split("=", 1)
        cfg.kernel_override[k] = v
    for var, val in env.items():
        if not var.startswith("GRIMOIRE_"):
            continue
        if var in _ENV:
            name, typ = _ENV[var]
            try:
                setattr(cfg, name, typ(val))
            except ValueError as e:
                raise ValueError(f"{var}={val!r}: {e}") from None
        elif var not in _KNOWN_OTHER:
            cfg.unknown_env.append(var)
    if cfg.unknown_env:
        msg = "unknown GRIMOIRE_* variables ignored: " + ", ".join(sorted(cfg.unknown_env))
        (warn or (lambda m: print(m, file=sys.stderr)))(msg)
    return cfg.validate()
