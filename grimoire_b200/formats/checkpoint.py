"""Checkpoint reading: HF directory -> logical weights (fp32 or native quantized) per tensor name.

Covers what the reference's Qwen35Model::load / linear_ref do (src/qwen35_loader.cpp:161-1611):
name prefix detection (``model.language_model.`` vs ``model.``), and the quantized suffix zoo --
GPTQ triples (group size from the scales shape), compressed-tensors ``weight_packed`` /
``weight_scale`` (+ ``weight_global_scale`` => NVFP4, which DIVIDES by the global scale), modelopt
NVFP4 (``weight`` U8 + ``weight_scale`` + ``weight_scale_2``, which MULTIPLIES), FP8 with
``weight_scale_inv`` (128x128 blocks, multiplies) or ``weight_scale`` [N,1], int8 embedding side
tensors, plain bf16/f16/f32.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Optional, Union

import torch

from ..models.config import ModelConfig
from . import codecs as C
from . import gptq
from .codecs import Fmt
from .quantize import QuantWeight, quantize
from .safetensors_io import CheckpointDir

LinearSource = Union[torch.Tensor, QuantWeight]

# tensors that are never quantized (keep_qwen_bf16, src/qwen35_loader.cpp:129-159)
NEVER_QUANTIZE = ("norm", "embed_tokens", "A_log", "dt_bias", "conv1d", "mlp.gate.weight", "shared_expert_gate",
                  "in_proj_a", "in_proj_b")


class Checkpoint:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        self.dir = CheckpointDir(self.path)
        self.config_json = json.loads((self.path / "config.json").read_text())
        self.cfg = ModelConfig.from_hf(self.config_json)
        keys = set(self.dir.keys())
        self.prefix = "model.language_model." if any(k.startswith("model.language_model.") for k in keys) else "model."
        self._keys = keys
        qc = self.config_json.get("quantization_config") or {}
        self.quant_method = qc.get("quant_method", "")

    def has(self, name: str) -> bool:
        return name in self._keys

    def tensor(self, name: str) -> Optional[torch.Tensor]:
        return self.dir.get(name) if name in self._keys else None

    def plain(self, name: str) -> Optional[torch.Tensor]:
        """An unquantized tensor as fp32 (norm weights, embeddings, small gates)."""
        t = self.tensor(name)
        return None if t is None else t.float()

    # ------------------------------------------------------------------------------------------
    def linear(self, base: str) -> Optional[LinearSource]:
        """Resolve ``<base>.weight`` in whatever form the checkpoint stores it.

        Returns a QuantWeight when the stored form maps 1:1 onto a runtime format (GPTQ int4,
        MXFP4, NVFP4, block fp8, per-row fp8), else an fp32 ``[out][in]`` tensor."""
        k = self._keys
        if base + ".qweight" in k:
            return gptq.gptq_unpack(self.dir.get(base + ".qweight"), self.dir.get(base + ".qzeros"),
                                    self.dir.get(base + ".scales"), self.tensor(base + ".g_idx"))
        if base + ".weight_packed" in k:
            packed = self.dir.get(base + ".weight_packed")
            scale = self.dir.get(base + ".weight_scale")
            if base + ".weight_global_scale" in k:         # compressed-tensors NVFP4: divide
                g = float(self.dir.get(base + ".weight_global_scale").float().reshape(-1)[0])
                pay = packed.view(torch.uint8)
                N, K = pay.shape[0], pay.shape[1] * 2
                return QuantWeight(Fmt.NVFP4, N, K, pay.contiguous(), scales=scale.view(torch.uint8).reshape(N, K // 16).contiguous(),
                                   group=16, global_scale=1.0 / g)
            if packed.dtype == torch.uint8 and scale.dtype == torch.uint8:     # MXFP4: e2m1 + e8m0 / 32
                N, K = packed.shape[0], packed.shape[1] * 2
                return QuantWeight(Fmt.MXFP4, N, K, packed.contiguous(), scales=scale.reshape(N, K // 32).contiguous(), group=32)
            if packed.dtype == torch.int32:                # compressed-tensors int4: 8 codes per word along IN, symmetric (code - 8)
                N = packed.shape[0]
                shape = self.tensor(base + ".weight_shape")
                K = int(shape[1]) if shape is not None else packed.shape[1] * 8
                q = gptq._unpack_i32_nibbles(packed, 1)[:, :K]
                group = K // scale.shape[1]
                zp = self.tensor(base + ".weight_zero_point")
                zeros = torch.full((N, K // group), 8, dtype=torch.uint8) if zp is None else \
                    gptq._unpack_i32_nibbles(zp.t().contiguous(), 1).t()[:N, : K // group].to(torch.uint8)
                return QuantWeight(Fmt.INT4, N, K, C.pack_nibbles(q.to(torch.uint8)), scales=scale.half().contiguous(), zeros=zeros, group=group)
        w = self.tensor(base + ".weight")
        if w is None:
            return None
        if w.dtype == torch.uint8 and base + ".weight_scale_2" in k:          # modelopt NVFP4: multiply
            N, K = w.shape[0], w.shape[1] * 2
            g = float(self.dir.get(base + ".weight_scale_2").float().reshape(-1)[0])
            return QuantWeight(Fmt.NVFP4, N, K, w.contiguous(), scales=self.dir.get(base + ".weight_scale").view(torch.uint8).reshape(N, K // 16).contiguous(),
                               group=16, global_scale=g)
        if w.dtype == torch.float8_e4m3fn:
            N, K = w.shape
            if base + ".weight_scale_inv" in k:            # 128x128 blocks, multiply
                s = self.dir.get(base + ".weight_scale_inv").float()
                rows = s.repeat_interleave(128, dim=0)[:N]                       # -> [N][K/128] (1x128 runtime blocks)
                return QuantWeight(Fmt.FP8_BLOCK, N, K, w.view(torch.uint8).contiguous(), scales=rows.contiguous(), group=128)
            if base + ".weight_scale" in k:
                s = self.dir.get(base + ".weight_scale").float().reshape(-1)
                s = s.expand(N) if s.numel() == 1 else s
                return QuantWeight(Fmt.FP8_E4M3, N, K, w.view(torch.uint8).contiguous(), scales=s.contiguous())
            return w.float()
        return w.float()

    def embedding(self) -> torch.Tensor:
        """Token embedding table as fp32, including the int8 + per-row scale side form
        (include/b70/int8_embedding.hpp)."""
        name = self.prefix + "embed_tokens.weight"
        t = self.tensor(name)
        if t is not None and t.dtype == torch.int8 and self.has(self.prefix + "embed_tokens.weight_scale"):
            # both gathered operands are bf16 in the source model: the scale is rounded to bf16, and so is the product
            scale = self.dir.get(self.prefix + "embed_tokens.weight_scale").bfloat16().float().reshape(-1, 1)
            return (t.float() * scale).bfloat16().float()
        if t is None:
            raise KeyError(name)
        return t.float()


def to_runtime(src: LinearSource, proj: Fmt, group: int = C.INT4_GROUP) -> QuantWeight:
    """Bring a resolved linear to the runtime projection format ``proj``.  A stored form that
    already is ``proj`` is used as is (a GPTQ checkpoint served with ``--proj int4`` is repacked,
    not requantized); anything else is dequantized and requantized on the host."""
    if isinstance(src, QuantWeight):
        if src.fmt == proj:
            return src
        src = src.dequant()
    return quantize(src, proj, group=group)
