"""Tracing and diagnosis helpers.

* **Device timeline** (``GRIMOIRE_TIMELINE=1`` or ``timeline.enable()``): ``mark(tag)`` records a CUDA
  event on the current stream; a region's time is the gap between consecutive marks on the in-order
  stream, so marking costs no synchronisation.  ``dump()`` synchronises once and returns microseconds
  per tag (summed over layers) for the marks since the last ``reset()``.  This is the reference's
  marker-kernel timeline (``mark()`` / ``dump_timeline()``, grimoire.cpp:3823-3850, :25138-25170)
  with events instead of 1-thread kernels.  Marks are skipped while a CUDA graph is being captured.
* **Fenced host timers** (``FencedTimer``): wall time of a region with a device synchronise on both
  sides -- diagnosis only, it serialises the pipeline (GRIMOIRE_SPEC_TIME and friends,
  include/b70/generation.hpp:47-53).
* **Numeric probe** (``probe(tag, tensor)`` under ``GRIMOIRE_DEBUG=1``): rms / max / nan / inf of a
  buffer, plus with ``GRIMOIRE_PROBE_EXACT=1`` an FNV-1a hash of its bits and the first 4 values
  (grimoire.cpp:25172-25200), for bisecting divergence between two builds or ranks.
* **Launch counting**: ``launches()`` returns the number of native kernel launches issued so far
  (every launcher goes through ``_native.check``); the difference across a step is the per-step count
  (the reference counts ``urEnqueueKernelLaunch`` with tools/count_launches.sh).
"""
from __future__ import annotations

import os
import time
from collections import OrderedDict
from typing import Optional

import torch

from .. import _native


class Timeline:
    def __init__(self):
        self.on = os.environ.get("GRIMOIRE_TIMELINE", "0") not in ("", "0")
        self._marks: list[tuple[str, object]] = []

    def enable(self, on: bool = True) -> None:
        self.on = on
        self._marks.clear()

    def reset(self) -> None:
        self._marks.clear()

    def mark(self, tag: str) -> None:
        """End the previous region and start region ``tag`` on the current stream."""
        if not self.on:
            return
        if torch.cuda.is_available():
            if torch.cuda.is_current_stream_capturing():
                return
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((tag, ev))
        else:
            self._marks.append((tag, time.perf_counter()))

    def dump(self, per_mark: bool = False):
        """Microseconds per tag since the last reset (``per_mark``: the raw sequence instead).  The last
        mark closes the timeline; tag it "end"."""
        if torch.cuda.is_available() and self._marks:
            torch.cuda.synchronize()
        seq = []
        for (tag, a), (_, b) in zip(self._marks, self._marks[1:]):
            us = a.elapsed_time(b) * 1000.0 if hasattr(a, "elapsed_time") else (b - a) * 1e6
            seq.append((tag, us))
        if per_mark:
            return seq
        out: "OrderedDict[str, float]" = OrderedDict()
        for tag, us in seq:
            out[tag] = out.get(tag, 0.0) + us
        return out

    def format(self) -> str:
        d = self.dump()
        total = sum(d.values()) or 1.0
        return "\n".join(f"{tag:>14s} {us:10.1f} us {100.0 * us / total:5.1f} %" for tag, us in d.items())


timeline = Timeline()
mark = timeline.mark


class FencedTimer:
    """``with FencedTimer(store, "verify"): ...`` adds the fenced wall time (seconds) to store[name]."""

    def __init__(self, store: dict, name: str, enabled: bool = True):
        self.store, self.name, self.enabled = store, name, enabled

    def __enter__(self):
        if self.enabled:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.enabled:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self.store[self.name] = self.store.get(self.name, 0.0) + time.perf_counter() - self.t0
        return False


def fnv1a(data: bytes) -> int:
    h = 0xCBF29CE484222325
    for b in data:
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def probe_stats(t: torch.Tensor, exact: bool = False) -> dict:
    """rms / max|x| / nan / inf counts (and an exact bit hash) of a tensor, on whichever device it lives."""
    f = t.detach().float()
    finite = torch.isfinite(f)
    ok = torch.where(finite, f, torch.zeros_like(f))
    out = {"n": f.numel(), "rms": float(ok.pow(2).mean().sqrt()) if f.numel() else 0.0, "max": float(ok.abs().max()) if f.numel() else 0.0,
           "nan": int(torch.isnan(f).sum()), "inf": int(torch.isinf(f).sum())}
    if exact:
        raw = t.detach().contiguous().cpu().view(torch.uint8).numpy().tobytes()
        out["fnv1a"] = f"{fnv1a(raw):016x}"
        out["head"] = [float(v) for v in f.flatten()[:4].tolist()]
    return out


def probe(tag: str, t: Optional[torch.Tensor], file=None) -> Optional[dict]:
    """Print the probe line when GRIMOIRE_DEBUG is set; returns the stats (None when disabled)."""
    if t is None or os.environ.get("GRIMOIRE_DEBUG", "0") in ("", "0"):
        return None
    st = probe_stats(t, exact=os.environ.get("GRIMOIRE_PROBE_EXACT", "0") not in ("", "0"))
    extra = f" fnv={st['fnv1a']} head={st['head']}" if "fnv1a" in st else ""
    print(f"[probe] {tag}: n={st['n']} rms={st['rms']:.6g} max={st['max']:.6g} nan={st['nan']} inf={st['inf']}{extra}", file=file, flush=True)
    return st


def launches() -> int:
    return _native.launch_count
