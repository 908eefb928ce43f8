"""SentencePiece-style BPE tokenizers shipped as ``tokenizer.json`` (Llama-2 / Mistral / Gemma families).

Differences from the byte-level BPE core (csrc/host/tokenizer.cpp): the text is not mapped to bytes first -- spaces become
"▁" (optionally with one prepended), the symbols are Unicode characters, merges run over the whole segment between
special tokens (no regular-expression pre-tokenizer), and a character the vocabulary does not hold falls back to its UTF-8
bytes as ``<0xNN>`` tokens.  The reference parses the same two flavours (src/tokenizer.cpp:427 SPM pieces, :1627 Gemma);
here this path is Python (prompt tokenisation is off the token loop) with a heap-ordered merge queue, O(n log n) in the
segment length.
"""
from __future__ import annotations

import heapq
import re
import unicodedata
from typing import Optional, Sequence

SPACE = "▁"


def is_spm_bpe(meta: dict) -> bool:
    """True for a BPE ``tokenizer.json`` that is NOT byte-level: byte fallback pieces or a Metaspace / space-replacing
    normalizer and no ByteLevel pre-tokenizer."""
    model = meta.get("model") or {}
    if model.get("type") != "BPE":
        return False

    def kinds(node):
        if not node:
            return []
        return [node.get("type")] + [k for n in node.get("pretokenizers", []) + node.get("normalizers", []) for k in kinds(n)]

    if "ByteLevel" in kinds(meta.get("pre_tokenizer")):
        return False
    return bool(model.get("byte_fallback")) or "Metaspace" in kinds(meta.get("pre_tokenizer")) or SPACE in str(meta.get("normalizer"))


class _ScoreRanks:
    """Merge priorities taken from piece scores: rank(a, b) = -score(a + b) when a + b is a piece (ties: the lower id)."""

    def __init__(self, vocab: dict, scores: Sequence[float]):
        self.vocab, self.scores = vocab, scores

    def get(self, pair):
        i = self.vocab.get(pair[0] + pair[1])
        if i is None or i >= len(self.scores):
            return None
        return (-float(self.scores[i]), i)

    def __bool__(self):
        return True


class SpmBpe:
    def __init__(self, meta: dict):
        model = meta["model"]
        self.vocab: dict[str, int] = dict(model["vocab"])
        self.inv: dict[int, str] = {i: t for t, i in self.vocab.items()}
        self.ranks: dict[tuple[str, str], int] = {}
        for r, m in enumerate(model.get("merges", [])):
            a, b = m if isinstance(m, (list, tuple)) else m.split(" ", 1)
            self.ranks[(a, b)] = r
        if not self.ranks and model.get("scores"):
            # SentencePiece pieces with scores and no merge list (GGUF "llama" tokenizers): two neighbours merge when their
            # concatenation is a piece, the best-scored piece first (src/tokenizer.cpp:427 on)
            self.ranks = _ScoreRanks(self.vocab, model["scores"])
        self.byte_fallback = bool(model.get("byte_fallback"))
        self.unk = self.vocab.get(model.get("unk_token") or "<unk>", -1)
        self.special: dict[str, int] = {}
        self.special_ids: set[int] = set()
        for t in meta.get("added_tokens", []):
            self.vocab.setdefault(t["content"], t["id"])
            self.inv[t["id"]] = t["content"]
            if t.get("special", True):
                self.special[t["content"]] = t["id"]
                self.special_ids.add(t["id"])
        self._split = re.compile("(" + "|".join(re.escape(t) for t in sorted(self.special, key=len, reverse=True)) + ")") if self.special else None
        # normalizer: Prepend / Replace(" " -> "▁") / NFC / NFKC, in order; a Metaspace pre-tokenizer means both
        self.steps: list[tuple[str, str, str]] = []
        self._collect(meta.get("normalizer"))
        pre = meta.get("pre_tokenizer") or {}
        metas = [pre] + pre.get("pretokenizers", [])
        for n in metas:
            if n.get("type") == "Metaspace":
                if n.get("prepend_scheme", "always") != "never" and n.get("add_prefix_space", True):
                    self.steps.append(("prepend", SPACE, ""))
                self.steps.append(("replace", " ", n.get("replacement", SPACE)))
        self.strip_prefix = any(k == "prepend" for k, _, _ in self.steps)
        self.vocab_size = max(self.inv) + 1 if self.inv else 0

    def _collect(self, node: Optional[dict]) -> None:
        if not node:
            return
        t = node.get("type")
        if t == "Sequence":
            for n in node.get("normalizers", []):
                self._collect(n)
        elif t == "Prepend":
            self.steps.append(("prepend", node.get("prepend", SPACE), ""))
        elif t == "Replace":
            pat = node.get("pattern", {})
            if "String" in pat:
                self.steps.append(("replace", pat["String"], node.get("content", "")))
        elif t in ("NFC", "NFKC", "NFD", "NFKD"):
            self.steps.append(("unicode", t, ""))

    # ------------------------------------------------------------------------------------------
    def _normalize(self, text: str) -> str:
        for kind, a, b in self.steps:
            if kind == "prepend":
                text = a + text if text else text
            elif kind == "replace":
                text = text.replace(a, b)
            else:
                text = unicodedata.normalize(a, text)
        return text

    def _symbols(self, seg: str) -> list[str]:
        out = []
        for ch in seg:
            if ch in self.vocab or not self.byte_fallback:
                out.append(ch)
            else:
                out.extend(f"<0x{b:02X}>" for b in ch.encode("utf-8"))
        return out

    def _merge(self, sym: list[str]) -> list[str]:
        """Greedy lowest-rank-first merging with a heap over a doubly linked list of symbols."""
        n = len(sym)
        if n < 2:
            return sym
        prev = list(range(-1, n - 1))
        nxt = list(range(1, n + 1))
        nxt[-1] = -1
        alive = [True] * n
        heap = []
        for i in range(n - 1):
            r = self.ranks.get((sym[i], sym[i + 1]))
            if r is not None:
                heap.append((r, i, sym[i], sym[i + 1]))
        heapq.heapify(heap)
        while heap:
            r, i, a, b = heapq.heappop(heap)
            j = nxt[i] if alive[i] else -1
            if j < 0 or not alive[j] or sym[i] != a or sym[j] != b:
                continue                                   # stale entry
            sym[i] = a + b
            alive[j] = False
            nxt[i] = nxt[j]
            if nxt[j] >= 0:
                prev[nxt[j]] = i
            p, q = prev[i], nxt[i]
            if p >= 0:
                rr = self.ranks.get((sym[p], sym[i]))
                if rr is not None:
                    heapq.heappush(heap, (rr, p, sym[p], sym[i]))
            if q >= 0:
                rr = self.ranks.get((sym[i], sym[q]))
                if rr is not None:
                    heapq.heappush(heap, (rr, i, sym[i], sym[q]))
        return [s for s, ok in zip(sym, alive) if ok]

    def encode(self, text: str, allow_special: bool = True) -> list[int]:
        parts = self._split.split(text) if (allow_special and self._split) else [text]
        ids: list[int] = []
        first = True
        for part in parts:
            if not part:
                continue
            if allow_special and part in self.special:
                ids.append(self.special[part])
                continue
            seg = self._normalize(part) if first or not self.strip_prefix else self._normalize_no_prepend(part)
            first = False
            for tok in self._merge(self._symbols(seg)):
                i = self.vocab.get(tok)
                if i is None:
                    if self.byte_fallback:
                        ids.extend(self.vocab.get(f"<0x{b:02X}>", self.unk) for b in tok.encode("utf-8"))
                    else:
                        ids.append(self.unk)
                else:
                    ids.append(i)
        return ids

    def _normalize_no_prepend(self, text: str) -> str:
        for kind, a, b in self.steps:
            if kind == "replace":
                text = text.replace(a, b)
            elif kind == "unicode":
                text = unicodedata.normalize(a, text)
        return text

    def decode_bytes(self, ids: Sequence[int], skip_special: bool = True) -> bytes:
        out = bytearray()
        for i in ids:
            if skip_special and i in self.special_ids:
                continue
            t = self.inv.get(int(i))
            if t is None:
                continue
            if len(t) == 6 and t.startswith("<0x") and t.endswith(">"):
                try:
                    out.append(int(t[3:5], 16))
                    continue
                except ValueError:
                    pass
            out.extend(t.replace(SPACE, " ").encode("utf-8"))
        if self.strip_prefix and out[:1] == b" ":
            del out[0]
        return bytes(out)

    def token_id(self, token: str) -> int:
        return self.vocab.get(token, -1)
