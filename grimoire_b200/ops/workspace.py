"""Per-device scratch shared by the kernels of one engine (grow-only, like the reference's
grow-only prefill scratch cache, grimoire.cpp:11103-11161).

Holds: the bf16 buffer the int4 weights are dequantized into for a tcgen05 prefill GEMM, the
split-K partial buffer + arrival counters of the small-M kernel, and the split-KV partials +
counters of paged decode attention.  Counters are zeroed once at allocation; every kernel that
uses them leaves them at zero.
"""
from __future__ import annotations

import torch


class Workspace:
    def __init__(self, device):
        self.device = torch.device(device)
        self._bufs: dict[str, torch.Tensor] = {}

    def get(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        t = self._bufs.get(name)
        if t is None or t.numel() < numel or t.dtype != dtype:
            if t is not None and torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
                raise RuntimeError(f"workspace buffer {name!r} would grow during CUDA graph capture")
            t = (torch.zeros if zero else torch.empty)(max(numel, 1), dtype=dtype, device=self.device)
            self._bufs[name] = t
        return t

    def reserve(self, name: str, numel: int, dtype: torch.dtype, zero: bool = False) -> None:
        self.get(name, numel, dtype, zero)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._bufs.values())


_default: dict[str, Workspace] = {}


def default_workspace(device) -> Workspace:
    key = str(torch.device(device))
    if key not in _default:
        _default[key] = Workspace(device)
    return _default[key]
