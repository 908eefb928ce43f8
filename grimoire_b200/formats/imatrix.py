"""Importance matrices: per-input-channel activation statistics that steer int4 rounding.

Reads the llama.cpp ``.imatrix`` / ``.dat`` container the reference consumes
(include/b70/imatrix.hpp, src/quantize.cpp:354-437): a count, then per entry a name, a call count
and a float vector of summed squared activations.  ``importance_for`` maps a HF projection name to
its vector; ``quantize(..., search=True, importance=v)`` weights the clipping-range search with it.
"""
from __future__ import annotations

import struct
from pathlib import Path
from typing import Optional

import torch

# llama.cpp tensor-name stems -> HF projection names
_GGML_TO_HF = {"attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
               "attn_output": "self_attn.o_proj", "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj"}


def read_imatrix(path: str | Path) -> dict[str, torch.Tensor]:
    data = Path(path).read_bytes()
    off = 0
    (n,) = struct.unpack_from("<i", data, off)
    off += 4
    if n < 0 or n > 1 << 20:
        raise ValueError("imatrix: implausible entry count")
    out = {}
    for _ in range(n):
        (ln,) = struct.unpack_from("<i", data, off)
        off += 4
        if ln < 0 or off + ln > len(data):
            raise ValueError("imatrix: truncated name")
        name = data[off: off + ln].decode("utf-8", errors="replace")
        off += ln
        ncall, nval = struct.unpack_from("<ii", data, off)
        off += 8
        if nval < 0 or off + 4 * nval > len(data):
            raise ValueError("imatrix: truncated values")
        vals = torch.frombuffer(bytearray(data[off: off + 4 * nval]), dtype=torch.float32).clone()
        off += 4 * nval
        out[name] = vals / max(ncall, 1)
    return out


def write_imatrix(path: str | Path, entries: dict[str, torch.Tensor], ncall: int = 1) -> None:
    with open(path, "wb") as f:
        f.write(struct.pack("<i", len(entries)))
        for name, v in entries.items():
            b = name.encode()
            f.write(struct.pack("<i", len(b)))
            f.write(b)
            f.write(struct.pack("<ii", ncall, v.numel()))
            f.write((v.float() * ncall).numpy().tobytes())


def importance_for(im: dict[str, torch.Tensor], hf_name: str) -> Optional[torch.Tensor]:
    """``model.layers.3.mlp.down_proj.weight`` -> the vector stored as ``blk.3.ffn_down.weight``."""
    parts = hf_name.split(".")
    if "layers" not in parts:
        return None
    layer = parts[parts.index("layers") + 1]
    for ggml, hf in _GGML_TO_HF.items():
        if hf in hf_name:
            return im.get(f"blk.{layer}.{ggml}.weight")
    return None
