"""Pre-quantized model artifact ("model-v3.grm") and the offline quantizer / inspector CLIs.

Role of the reference's native v3 container and ``grimoire-quantize`` (include/b70/native_model.hpp,
src/native_model.cpp:157-230, tools/b70_compile_model.cpp:205-213, docs/native-quantizer-v3.md):
``grimoire quantize SRC OUT --format {int4,bf16,fp8,fp8-e5m2,int8,mxfp4,mxfp8} --policy
{experts,linear} [--bundle]`` reads a HF checkpoint one tensor at a time (round to nearest), and
writes one mmap-able file: a 48-byte header, 288-byte tensor records and 4096-byte aligned payload
/ scale / zero regions.  ``--bundle`` copies config, tokenizer files and a manifest next to it.
"""
from __future__ import annotations

import argparse
import json
import mmap
import shutil
import struct
from pathlib import Path
from typing import Iterable, Optional, Union

import torch

from . import codecs as C
from .codecs import Fmt
from .quantize import QuantWeight, quantize

MAGIC = b"GRMB200\0"
VERSION = 3
HEADER = struct.Struct("<8sIIQQ16x")          # magic, version, n_tensors, records_offset, data_offset  (48 bytes)
RECORD = struct.Struct("<192sIIQQIIQQQQQQf12x")  # 288 bytes
ALIGN = 4096
ENC_RAW = 0          # unquantized tensor (dtype in `fmt`: 0 f32, 1 bf16, 2 f16)
_RAW_DT = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}
_RAW_ID = {v: k for k, v in _RAW_DT.items()}
assert HEADER.size == 48 and RECORD.size == 288

Entry = Union[torch.Tensor, QuantWeight]


def _pad(f, align=ALIGN):
    pos = f.tell()
    f.write(b"\0" * ((align - pos % align) % align))
    return f.tell()


def write_artifact(path: str | Path, entries: Iterable[tuple[str, Entry]]) -> int:
    """Stream (name, tensor-or-QuantWeight) pairs into an artifact; returns the tensor count."""
    path = Path(path)
    records = []
    with open(path, "wb") as f:
        f.write(b"\0" * HEADER.size)
        data_offset = _pad(f)
        for name, e in entries:
            nb = name.encode()
            if len(nb) >= 192:
                raise ValueError(f"tensor name too long: {name}")

            def blob(t: Optional[torch.Tensor]):
                if t is None:
                    return 0, 0
                off = _pad(f)
                raw = t.detach().cpu().contiguous().view(torch.uint8).reshape(-1).numpy().tobytes()
                f.write(raw)
                return off, len(raw)

            if isinstance(e, QuantWeight):
                po, pl = blob(e.payload)
                so, sl = blob(e.scales)
                zo, zl = blob(e.zeros)
                records.append(RECORD.pack(nb, 1 + int(e.fmt), int(e.fmt), e.N, e.K, e.group, 0, po, pl, so, sl, zo, zl,
                                           float(e.global_scale)))
            else:
                t = e.detach()
                if t.dtype not in _RAW_ID:
                    t = t.float()
                po, pl = blob(t)
                shape = list(t.shape) + [1, 1]
                records.append(RECORD.pack(nb, ENC_RAW, _RAW_ID[t.dtype], shape[0], shape[1] if t.dim() > 1 else 0, t.dim(), 0,
                                           po, pl, 0, 0, 0, 0, 1.0))
        records_offset = _pad(f)
        for r in records:
            f.write(r)
        f.seek(0)
        f.write(HEADER.pack(MAGIC, VERSION, len(records), records_offset, data_offset))
    return len(records)


class Artifact:
    """mmap reader: ``get(name)`` returns a tensor (raw entries) or a QuantWeight (quantized ones)."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        magic, ver, n, rec_off, data_off = HEADER.unpack_from(self._mm, 0)
        if magic != MAGIC:
            raise ValueError(f"{path}: not a grimoire-b200 artifact")
        if ver != VERSION:
            raise ValueError(f"{path}: artifact version {ver}, expected {VERSION}")
        if rec_off + n * RECORD.size > len(self._mm):
            raise ValueError(f"{path}: record table out of range")
        self.records = {}
        for i in range(n):
            r = RECORD.unpack_from(self._mm, rec_off + i * RECORD.size)
            name = r[0].split(b"\0", 1)[0].decode()
            for off, ln in ((r[7], r[8]), (r[9], r[10]), (r[11], r[12])):
                if off + ln > len(self._mm):
                    raise ValueError(f"{path}: region of {name} out of range")
            self.records[name] = r

    def keys(self):
        return self.records.keys()

    def _bytes(self, off, ln) -> torch.Tensor:
        return torch.frombuffer(self._mm, dtype=torch.uint8, count=ln, offset=off).clone() if ln else torch.empty(0, dtype=torch.uint8)

    def get(self, name: str) -> Entry:
        r = self.records[name]
        enc, fmt, N, K, group = r[1], r[2], r[3], r[4], r[5]
        if enc == ENC_RAW:
            t = self._bytes(r[7], r[8]).view(_RAW_DT[fmt])
            ndim = group
            return t.reshape(N, K) if ndim == 2 else t.reshape(-1) if ndim <= 1 else t
        f = Fmt(fmt)
        pay = self._bytes(r[7], r[8]).reshape(N, -1)
        sc = self._bytes(r[9], r[10])
        zr = self._bytes(r[11], r[12])
        if f == Fmt.INT4:
            scales, zeros = sc.view(torch.float16).reshape(N, -1), zr.reshape(N, -1)
        elif f in (Fmt.INT8, Fmt.FP8_E4M3, Fmt.FP8_E5M2):
            scales, zeros = sc.view(torch.float32).reshape(N), None
        elif f == Fmt.FP8_BLOCK:
            scales, zeros = sc.view(torch.float32).reshape(N, -1), None
        elif f == Fmt.BF16:
            scales, zeros = None, None
        else:
            scales, zeros = sc.reshape(N, -1), None
        return QuantWeight(f, N, K, pay, scales=scales, zeros=zeros, group=group, global_scale=r[13])

    def describe(self) -> list[dict]:
        out = []
        for name, r in self.records.items():
            out.append({"name": name, "encoding": "raw" if r[1] == ENC_RAW else Fmt(r[2]).name.lower(), "shape": [r[3], r[4]],
                        "group": r[5] if r[1] != ENC_RAW else 0, "payload_bytes": r[8], "scale_bytes": r[10]})
        return out

    def close(self):
        self._mm.close()
        self._f.close()


class ArtifactSource:
    """Tensor resolver over an artifact with the interface the model loaders use (``cfg``, ``prefix``, ``has``,
    ``tensor``, ``plain``, ``linear``, ``embedding``): the counterpart of NativeModel::view feeding Grimoire::build
    (src/native_model.cpp:157-260).  Quantised entries come back as QuantWeights and are served in their stored format
    when it matches the projection format, raw entries as tensors."""

    def __init__(self, art: "Artifact", cfg):
        self.art, self.cfg = art, cfg
        keys = set(art.keys())
        self._keys = keys
        self.prefix = "model.language_model." if any(k.startswith("model.language_model.") for k in keys) else "model."

    def has(self, name: str) -> bool:
        return name in self._keys

    def tensor(self, name: str):
        if name not in self._keys:
            return None
        e = self.art.get(name)
        return e.dequant() if isinstance(e, QuantWeight) else e

    def plain(self, name: str):
        t = self.tensor(name)
        return None if t is None else t.float()

    def linear(self, base: str):
        name = base + ".weight"
        if name not in self._keys:
            return None
        e = self.art.get(name)
        return e if isinstance(e, QuantWeight) else e.float()

    def embedding(self):
        t = self.plain(self.prefix + "embed_tokens.weight")
        if t is None:
            raise KeyError(self.prefix + "embed_tokens.weight")
        return t


def load_artifact_model(path: str | Path, cfg, device, ec):
    """Build the model of a pre-quantised artifact (``model-v3.grm`` next to its ``config.json``).  Returns (model,
    resolver for the draft head or None)."""
    from ..models.dense import DenseModel
    from ..models.hybrid import HybridModel
    from ..models.config import LINEAR_ATTN

    src = ArtifactSource(Artifact(path), cfg)
    if cfg.is_moe or any(t == LINEAR_ATTN for t in cfg.layer_types):
        model = HybridModel.from_checkpoint(src, device, max_slots=ec.seq_slots, ep_rank=ec.ep_rank, ep_world=ec.ep_world)
        return model, None
    # the artifact's own format wins unless --proj names another one
    stored = {Fmt(r[2]) for r in src.art.records.values() if r[1] != ENC_RAW}
    proj = ec.proj
    if proj in ("int4", "native") and len(stored) == 1:
        only = next(iter(stored))
        proj = {Fmt.INT4: "int4", Fmt.MXFP4: "mxfp4", Fmt.FP8_BLOCK: "fp8", Fmt.INT8: "int8", Fmt.BF16: "bf16", Fmt.MXFP8: "mxfp8",
                Fmt.FP8_E4M3: "fp8_e4m3", Fmt.FP8_E5M2: "fp8_e5m2"}.get(only, proj)
    model = DenseModel.from_checkpoint(src, device, ec.tp_rank, ec.tp_world, lm_head_bf16=bool(ec.lm_head_bf16), proj=proj,
                                       pp_rank=ec.pp_rank, pp_world=ec.pp_world)
    mtp = src if (ec.mtp and cfg.mtp_num_hidden_layers > 0 and src.has("mtp.fc.weight")) else None
    return model, mtp


_FORMATS = {"int4": Fmt.INT4, "bf16": Fmt.BF16, "fp8": Fmt.FP8_E4M3, "fp8-e4m3": Fmt.FP8_E4M3, "fp8-e5m2": Fmt.FP8_E5M2,
            "int8": Fmt.INT8, "mxfp4": Fmt.MXFP4, "mxfp8": Fmt.MXFP8, "fp8-block": Fmt.FP8_BLOCK, "nvfp4": Fmt.NVFP4}
_LINEAR = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "in_proj_qkv", "in_proj_z", "out_proj")


def _wants_quant(name: str, policy: str) -> bool:
    from .checkpoint import NEVER_QUANTIZE

    if any(k in name for k in NEVER_QUANTIZE) and "experts" not in name:
        return False
    if policy == "experts":
        return ".experts." in name
    return any(name.endswith(p + ".weight") or f".{p}." in name for p in _LINEAR) or ".experts." in name or name == "lm_head.weight"


def quantize_checkpoint(src: str | Path, out: str | Path, fmt: Fmt, policy: str = "linear", bundle: bool = False,
                        imatrix: Optional[str] = None) -> dict:
    from .checkpoint import Checkpoint
    from .imatrix import importance_for, read_imatrix

    ck = Checkpoint(src)
    out = Path(out)
    target = out / "model-v3.grm" if bundle or out.suffix == "" else out
    target.parent.mkdir(parents=True, exist_ok=True)
    im = read_imatrix(imatrix) if imatrix else None
    stats = {"quantized": 0, "raw": 0}

    def stream():
        seen = set()
        for name in sorted(ck.dir.keys()):
            base = name.rsplit(".", 1)[0]
            if name.endswith((".qweight", ".weight_packed")) or (name.endswith(".weight") and base not in seen):
                if base in seen:
                    continue
                seen.add(base)
                wname = base + ".weight"
                if _wants_quant(wname, policy):
                    srcw = ck.linear(base)
                    if isinstance(srcw, QuantWeight) and srcw.fmt == fmt:
                        qw = srcw
                    else:
                        dense = srcw.dequant() if isinstance(srcw, QuantWeight) else srcw
                        imp = importance_for(im, wname) if im else None
                        qw = quantize(dense, fmt, search=imp is not None, importance=imp) if fmt == Fmt.INT4 else quantize(dense, fmt)
                    stats["quantized"] += 1
                    yield wname, qw
                    continue
                t = ck.tensor(wname)
                if t is not None:
                    stats["raw"] += 1
                    yield wname, t if t.dtype in _RAW_ID else t.float()
            elif not name.endswith((".qzeros", ".scales", ".g_idx", ".weight_scale", ".weight_scale_inv", ".weight_scale_2",
                                    ".weight_global_scale", ".weight_shape", ".weight_zero_point", ".weight")):
                stats["raw"] += 1
                t = ck.tensor(name)
                yield name, t if t.dtype in _RAW_ID else t.float()

    n = write_artifact(target, stream())
    if bundle:
        for fn in ("config.json", "tokenizer.json", "tokenizer_config.json", "generation_config.json"):
            if (Path(src) / fn).exists():
                shutil.copy(Path(src) / fn, out / fn)
        (out / "manifest.json").write_text(json.dumps({"format": fmt.name.lower(), "policy": policy, "tensors": n, "source": str(src),
                                                       "artifact": target.name, "version": VERSION}, indent=1))
    stats["tensors"] = n
    stats["path"] = str(target)
    return stats


def quantize_cli(argv) -> int:
    ap = argparse.ArgumentParser(prog="grimoire quantize")
    ap.add_argument("src")
    ap.add_argument("out")
    ap.add_argument("--format", default="int4", choices=sorted(_FORMATS))
    ap.add_argument("--policy", default="linear", choices=["experts", "linear"])
    ap.add_argument("--bundle", action="store_true")
    ap.add_argument("--imatrix", default=None)
    ns = ap.parse_args(argv)
    print(json.dumps(quantize_checkpoint(ns.src, ns.out, _FORMATS[ns.format], ns.policy, ns.bundle, ns.imatrix)))
    return 0


def inspect_cli(argv) -> int:
    ap = argparse.ArgumentParser(prog="grimoire inspect")
    ap.add_argument("artifact")
    ns = ap.parse_args(argv)
    a = Artifact(ns.artifact)
    for d in a.describe():
        print(json.dumps(d))
    return 0
