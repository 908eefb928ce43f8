"""Expert routing statistics and placement.

The reference keeps a decayed per-(layer, expert) heat, credited from every routing decision, and
uses it to decide which experts live in VRAM and which in pinned host memory, swapping a bounded
number per step with hysteresis (include/b70/expert_heat.hpp:22-100; upload_tiered_experts
grimoire.cpp:18373; hit file GRIMOIRE_EXPERT_HITS updated every 256 tokens, tm_save_hits :14300).

On a 180 GB part every expert of the 80B model is resident, so the same statistics drive a different
decision here: **which rank owns which expert** under expert parallelism.  ``balanced_placement``
spreads the hot experts of each layer evenly over the ranks (equal expert counts per rank, greedy
longest-processing-time on heat), which evens out the rows each rank's grouped GEMM receives.  The
two-tier swap proposal is kept (``propose_swaps``) for deployments that oversubscribe HBM with KV
slots and park cold experts in pinned memory.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Sequence

import numpy as np


@dataclass
class HeatParams:
    decay: float = 0.95          # applied to a layer's heats each time that layer is credited
    hysteresis: float = 1.25     # promote only when hot >= cold * hysteresis + min_gain
    min_gain: float = 1.5
    credit_cap: float = 512.0    # most selections one call credits (a prompt chunk must not own the set)
    moves_per_step: int = 32


@dataclass(frozen=True)
class Swap:
    promote_layer: int
    promote_expert: int
    demote_layer: int
    demote_expert: int


class ExpertHeat:
    def __init__(self, layers: int, experts: int, params: HeatParams | None = None):
        self.L, self.E, self.p = layers, experts, params or HeatParams()
        self.h = np.zeros((layers, experts), dtype=np.float32)
        self.hits = np.zeros((layers, experts), dtype=np.int64)     # undecayed, what the hit file stores
        self.tokens_since_save = 0

    def credit(self, layer: int, ids: Sequence[int]) -> None:
        """One call of ``layer``: its routed expert ids (out-of-range ids such as -1 are skipped)."""
        if not 0 <= layer < self.L:
            return
        ids = np.asarray(ids, dtype=np.int64).reshape(-1)
        n = ids.size
        self.h[layer] *= np.float32(self.p.decay)
        if n == 0:
            return
        w = np.float32(self.p.credit_cap / n if n > self.p.credit_cap else 1.0)
        ok = ids[(ids >= 0) & (ids < self.E)]
        np.add.at(self.h[layer], ok, w)
        np.add.at(self.hits[layer], ok, 1)

    def propose_swaps(self, resident: Callable[[int, int], bool], movable: Callable[[int, int], bool]) -> list[Swap]:
        """Hottest non-resident experts against the coldest resident ones, at most ``moves_per_step``,
        while hot >= cold * hysteresis + min_gain; ties broken by (layer, expert)."""
        hot, cold = [], []
        for l in range(self.L):
            for e in range(self.E):
                if not movable(l, e):
                    continue
                x = float(self.h[l, e])
                if resident(l, e):
                    cold.append((x, l, e))
                elif x > 0.0:
                    hot.append((x, l, e))
        hot.sort(key=lambda u: (-u[0], u[1], u[2]))
        cold.sort(key=lambda u: (u[0], u[1], u[2]))
        out = []
        for (hh, hl, he), (ch, cl, ce) in zip(hot[: self.p.moves_per_step], cold[: self.p.moves_per_step]):
            if not hh >= ch * self.p.hysteresis + self.p.min_gain:
                break
            out.append(Swap(hl, he, cl, ce))
        return out

    # ---- persistence (one JSON object; rewritten atomically) ----
    def save(self, path: str) -> None:
        tmp = path + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"layers": self.L, "experts": self.E, "hits": self.hits.tolist()}, f)
        os.replace(tmp, path)
        self.tokens_since_save = 0

    def load(self, path: str) -> bool:
        try:
            with open(path) as f:
                d = json.load(f)
        except (OSError, ValueError):
            return False
        if d.get("layers") != self.L or d.get("experts") != self.E:
            return False
        self.hits = np.asarray(d["hits"], dtype=np.int64)
        tot = np.maximum(self.hits.sum(axis=1, keepdims=True), 1)
        self.h = (self.hits / tot * self.p.credit_cap).astype(np.float32)      # warm start in credit units
        return True

    def on_tokens(self, n: int, path: str = "", every: int = 256) -> None:
        self.tokens_since_save += n
        if path and self.tokens_since_save >= every:
            self.save(path)


def balanced_placement(heat_row: Sequence[float], world: int) -> list[int]:
    """Permutation ``perm`` of one layer's experts such that rank r owns experts
    perm[r*E/W : (r+1)*E/W] and the summed heat per rank is as even as a greedy pass gets it
    (hottest first onto the least-loaded rank that still has room).  Deterministic."""
    E = len(heat_row)
    if E % world:
        raise ValueError("experts do not split evenly")
    per = E // world
    order = sorted(range(E), key=lambda e: (-float(heat_row[e]), e))
    load, members = [0.0] * world, [[] for _ in range(world)]
    for e in order:
        r = min((r for r in range(world) if len(members[r]) < per), key=lambda r: (load[r], r))
        members[r].append(e)
        load[r] += float(heat_row[e])
    return [e for r in range(world) for e in sorted(members[r])]


def rank_loads(heat_row: Sequence[float], perm: Sequence[int], world: int) -> list[float]:
    per = len(perm) // world
    return [float(sum(heat_row[e] for e in perm[r * per: (r + 1) * per])) for r in range(world)]
