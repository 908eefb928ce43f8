"""Prefix cache over the paged KV pool.

Role of the reference's PrefixCache / prefix_reuse / save_prefix(_head) (grimoire.cpp:3340-3484,
:10731-11047, :11908-12035): a finished conversation's KV stays resident, a new prompt reuses the
longest matching *prefix*, and a prompt-head snapshot (KV + last-token logits) makes an identical
prompt cost zero prefill rows (105K-token repeat: 54.4 s -> 0.39 s, README.md:235).

Mechanism here: KV is paged, so an entry is a list of page ids whose reference counts the cache
holds; reuse = pointing the new slot's block table at the shared full pages (no copy), plus a copy
of the one partial tail page when the whole entry is reused (copy-on-write of 16 tokens).  Entries
are evicted least-recently-used when the pool runs short.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from ..ops.core import PAGE
from .kv import KvPool, SeqSlot


@dataclass
class PrefixEntry:
    tokens: list[int]
    pages: list[int]
    head_logits: Optional[torch.Tensor] = None     # logits after the last token (prompt-head snapshot)
    stamp: int = 0
    extra: dict = field(default_factory=dict)      # recurrent-state snapshots for hybrid models


class PrefixCache:
    def __init__(self, kv: KvPool, max_entries: int = 16):
        self.kv = kv
        self.max_entries = max_entries
        self.entries: list[PrefixEntry] = []
        self._clock = itertools.count(1)
        self.hits = 0
        self.tokens_reused = 0
        self.last_extra: dict = {}          # ``extra`` of the entry the last successful ``reuse`` attached
        kv.reclaim = self.make_room         # a live decode that needs a page evicts cached entries before it fails

    # ---- store ----
    def store(self, seq: SeqSlot, head_logits: Optional[torch.Tensor] = None, extra: Optional[dict] = None) -> None:
        """Keep the sequence's cached positions alive after the slot is released."""
        n = min(seq.length, len(seq.tokens))
        if n < PAGE:
            return
        npg = (n + PAGE - 1) // PAGE
        pages = list(seq.pages[:npg])
        for pg in pages:
            self.kv.refcount[pg] += 1
        ent = PrefixEntry(list(seq.tokens[:n]), pages, None if head_logits is None else head_logits.detach().clone(),
                          next(self._clock), extra or {})
        # drop an older entry that this one extends
        for old in list(self.entries):
            if len(old.tokens) <= n and old.tokens == ent.tokens[: len(old.tokens)]:
                self._drop(old)
        self.entries.append(ent)
        while len(self.entries) > self.max_entries:
            self.evict_one()

    def _drop(self, ent: PrefixEntry) -> None:
        self.entries.remove(ent)
        for pg in ent.pages:
            self.kv.refcount[pg] -= 1
            if self.kv.refcount[pg] == 0:
                self.kv.free.append(pg)

    def evict_one(self) -> bool:
        if not self.entries:
            return False
        self._drop(min(self.entries, key=lambda e: e.stamp))
        return True

    def make_room(self, pages_needed: int) -> None:
        while self.kv.pages_free() < pages_needed and self.evict_one():
            pass

    # ---- lookup ----
    def match(self, prompt: Sequence[int]):
        """Longest common prefix over the entries -> (entry, matched tokens)."""
        best, best_n = None, 0
        for ent in self.entries:
            n = 0
            lim = min(len(ent.tokens), len(prompt))
            while n < lim and ent.tokens[n] == prompt[n]:
                n += 1
            if n > best_n:
                best, best_n = ent, n
        return best, best_n

    def reuse(self, seq: SeqSlot, prompt: Sequence[int]):
        """Attach cached pages to a fresh slot.  Returns (tokens reused, head logits or None).
        At least one prompt token is always left to prefill unless the entry carries the logits of
        exactly this prompt."""
        self.last_extra = {}
        if seq.length or seq.pages:
            return 0, None
        ent, n = self.match(prompt)
        if ent is None:
            return 0, None
        exact = n == len(prompt) == len(ent.tokens) and ent.head_logits is not None
        # the whole entry is a prefix of the prompt: its partial tail page can be copied and appended to
        whole = n == len(ent.tokens) and (exact or len(prompt) > n)
        recurrent = ent.extra.get("recurrent") is not None
        if recurrent and not whole:
            # a recurrent state exists only for the entry's last position: a shorter match cannot resume from it
            return 0, None
        if not exact:
            n = min(n, len(prompt) - 1)
        n_full = n // PAGE
        if n_full == 0 and not whole:
            return 0, None
        kv = self.kv
        if whole and n > n_full * PAGE and not kv.free:
            self.make_room(1)
        if recurrent and n > n_full * PAGE and not kv.free:
            return 0, None                 # the tail page cannot be copied: KV and state would disagree
        for i in range(n_full):
            pg = ent.pages[i]
            kv.refcount[pg] += 1
            kv.table_host[seq.slot, i] = pg
            seq.pages.append(pg)
        reused = n_full * PAGE
        if whole and n > reused and kv.free:
            # copy-on-write of the entry's partial tail page so this conversation can append to it
            new = kv.free.pop()
            kv.refcount[new] = 1
            src = ent.pages[n_full]
            for L in kv.layers:
                L.k[new].copy_(L.k[src]); L.v[new].copy_(L.v[src]); L.ks[new].copy_(L.ks[src]); L.vs[new].copy_(L.vs[src])
            kv.table_host[seq.slot, n_full] = new
            seq.pages.append(new)
            reused = n
        kv._sync_row(seq.slot)
        seq.length = reused
        seq.tokens = list(prompt[:reused])
        ent.stamp = next(self._clock)
        self.last_extra = ent.extra
        self.hits += 1
        self.tokens_reused += reused
        return reused, (ent.head_logits if (exact and reused == len(prompt)) else None)
