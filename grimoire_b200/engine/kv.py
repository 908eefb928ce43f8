"""Pooled paged KV cache: 16-token int8 pages shared by every conversation slot.

Plays the role of the reference's per-slot KV views + on-demand virtual-memory pool
(bind_seq_slot grimoire.cpp:11872; KvVirtualPool src/kv_vmm.hpp; ensure_kv/admit_kv/release_kv
grimoire.cpp:12036-12070) with a different mechanism: one page pool per layer, a block table per
slot on the device, reference-counted pages so a cached prefix can be shared between slots
(prefix snapshot = page-table refcounts), and no per-slot context reservation.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..ops.core import PAGE, KvLayer


class OutOfPages(RuntimeError):
    pass


@dataclass
class SeqSlot:
    slot: int
    length: int = 0                 # tokens whose K/V are in the cache
    pages: list[int] = field(default_factory=list)
    tokens: list[int] = field(default_factory=list)   # token ids behind the cached positions


class KvPool:
    """Page allocator + per-slot block tables for ``n_layers`` attention layers."""

    def __init__(self, n_layers: int, Hkv: int, D: int, num_pages: int, max_slots: int, max_ctx: int, device):
        self.device = torch.device(device)
        self.num_pages = num_pages
        self.max_slots = max_slots
        self.max_pages_per_seq = (max_ctx + PAGE - 1) // PAGE
        self.layers = [KvLayer.alloc(num_pages, Hkv, D, device) for _ in range(n_layers)]
        self.refcount = [0] * num_pages
        self.free = list(range(num_pages - 1, -1, -1))
        # block table lives on the device (kernels index it) with a pinned host mirror
        self.table_host = torch.full((max_slots, self.max_pages_per_seq), -1, dtype=torch.int32)
        if self.device.type == "cuda":
            self.table_host = self.table_host.pin_memory()
        self.table = self.table_host.to(self.device)
        self.slots: dict[int, SeqSlot] = {}
        # called with the number of pages still missing when the free list runs dry (the prefix cache evicts entries)
        self.reclaim = None

    # ---- accounting ----
    def pages_free(self) -> int:
        return len(self.free)

    def pages_used(self) -> int:
        return self.num_pages - len(self.free)

    def bytes_per_token(self) -> int:
        return sum(l.bytes_per_token() for l in self.layers)

    # ---- slots ----
    def open_slot(self, slot: Optional[int] = None) -> SeqSlot:
        if slot is None:
            for s in range(self.max_slots):
                if s not in self.slots:
                    slot = s
                    break
            else:
                raise OutOfPages("no free conversation slot")
        if slot in self.slots:
            raise ValueError(f"slot {slot} already open")
        self.slots[slot] = SeqSlot(slot)
        return self.slots[slot]

    def ensure(self, seq: SeqSlot, new_length: int) -> None:
        """Make sure pages exist for positions < new_length (admit_kv / ensure_kv)."""
        need = (new_length + PAGE - 1) // PAGE
        if need > self.max_pages_per_seq:
            raise OutOfPages(f"context {new_length} exceeds the per-request cap")
        grew = False
        if need - len(seq.pages) > len(self.free) and self.reclaim is not None:
            self.reclaim(need - len(seq.pages))
        if need - len(seq.pages) > len(self.free):
            # nothing is mapped for a request that cannot be served in full: the caller parks or fails this one only
            raise OutOfPages(f"KV page pool exhausted ({need - len(seq.pages)} pages wanted, {len(self.free)} free)")
        while len(seq.pages) < need:
            pg = self.free.pop()
            self.refcount[pg] = 1
            self.table_host[seq.slot, len(seq.pages)] = pg
            seq.pages.append(pg)
            grew = True
        if grew:
            self._sync_row(seq.slot)

    def _sync_row(self, slot: int) -> None:
        self.table[slot].copy_(self.table_host[slot], non_blocking=True)

    def release(self, seq: SeqSlot) -> None:
        for pg in seq.pages:
            self.refcount[pg] -= 1
            if self.refcount[pg] == 0:
                self.free.append(pg)
        self.table_host[seq.slot].fill_(-1)
        self._sync_row(seq.slot)
        seq.pages.clear()
        seq.length = 0
        seq.tokens.clear()
        self.slots.pop(seq.slot, None)

    def truncate(self, seq: SeqSlot, length: int) -> None:
        """Drop cached positions >= length (speculative rollback keeps whole pages it still needs)."""
        keep = (length + PAGE - 1) // PAGE
        while len(seq.pages) > keep:
            pg = seq.pages.pop()
            self.table_host[seq.slot, len(seq.pages)] = -1
            self.refcount[pg] -= 1
            if self.refcount[pg] == 0:
                self.free.append(pg)
        seq.length = min(seq.length, length)
        del seq.tokens[length:]
        self._sync_row(seq.slot)

    def share_prefix(self, src: SeqSlot, dst: SeqSlot, n_tokens: int) -> int:
        """Point ``dst`` at the first whole pages of ``src`` (copy-on-write is not needed: only
        full pages are shared and new tokens go to fresh pages).  Returns the tokens shared."""
        n_pages = min(n_tokens // PAGE, len(src.pages))
        for i in range(n_pages):
            pg = src.pages[i]
            self.refcount[pg] += 1
            self.table_host[dst.slot, i] = pg
            dst.pages.append(pg)
        dst.length = n_pages * PAGE
        dst.tokens = list(src.tokens[: dst.length])
        if n_pages:
            self._sync_row(dst.slot)
        return dst.length
