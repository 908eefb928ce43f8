"""Tokenizer front end: the C++ byte-level BPE core (csrc/host/tokenizer.cpp) plus NFC
normalisation, special-token lookup and chat templates.

Reference: include/b70/tokenizer.hpp + src/tokenizer.cpp (load / encode / decode / special_id /
eos / eos2 / apply_chat_template; ChatML-Qwen tool template, reasoning switch).
"""
from __future__ import annotations

import ctypes
import json
import unicodedata
from pathlib import Path
from typing import Optional, Sequence

from . import _native

IM_START, IM_END, EOT = "<|im_start|>", "<|im_end|>", "<|endoftext|>"


class Tokenizer:
    def __init__(self, path: str | Path):
        p = Path(path)
        self.dir = p if p.is_dir() else p.parent
        tj = p / "tokenizer.json" if p.is_dir() else p
        self._spm = None
        meta0 = json.loads(tj.read_text())
        from .tokenizer_spm import SpmBpe, is_spm_bpe

        if is_spm_bpe(meta0):
            # SentencePiece-style BPE (spaces as U+2581, byte fallback pieces): Python path, see tokenizer_spm.py
            self._spm = SpmBpe(meta0)
            self._h, self._lib = None, None
            self.nfc = False
            self.cfg = {}
            tc = self.dir / "tokenizer_config.json"
            if tc.exists():
                try:
                    self.cfg = json.loads(tc.read_text())
                except json.JSONDecodeError:
                    self.cfg = {}
            self.vocab_size = self._spm.vocab_size
            return
        lib = _native.host()
        lib.grm_tok_load.restype = ctypes.c_void_p
        err = ctypes.create_string_buffer(512)
        h = lib.grm_tok_load(str(tj).encode(), err, 512)
        if not h:
            raise ValueError(err.value.decode(errors="replace"))
        self._h, self._lib = ctypes.c_void_p(h), lib
        meta = json.loads(tj.read_text())
        norm = meta.get("normalizer") or {}
        kinds = [norm.get("type")] + [n.get("type") for n in norm.get("normalizers", [])] if norm else []
        self.nfc = "NFC" in kinds
        self.cfg = {}
        tc = self.dir / "tokenizer_config.json"
        if tc.exists():
            try:
                self.cfg = json.loads(tc.read_text())
            except json.JSONDecodeError:
                self.cfg = {}
        self.vocab_size = lib.grm_tok_vocab_size(self._h)

    @classmethod
    def load(cls, path) -> "Tokenizer":
        return cls(path)

    def __del__(self):
        try:
            if self._h:
                self._lib.grm_tok_free(self._h)
                self._h = None
        except Exception:
            pass

    # ---- core ----
    def encode(self, text: str, allow_special: bool = True) -> list[int]:
        if self._spm is not None:
            return self._spm.encode(text, allow_special)
        if self.nfc:
            text = unicodedata.normalize("NFC", text)
        raw = text.encode("utf-8")
        cap = len(raw) + 16
        buf = (ctypes.c_int * cap)()
        n = self._lib.grm_tok_encode(self._h, raw, len(raw), buf, cap, 1 if allow_special else 0)
        if n > cap:
            buf = (ctypes.c_int * n)()
            n = self._lib.grm_tok_encode(self._h, raw, len(raw), buf, n, 1 if allow_special else 0)
        return list(buf[:n])

    def decode_bytes(self, ids: Sequence[int], skip_special: bool = True) -> bytes:
        if self._spm is not None:
            return self._spm.decode_bytes(ids, skip_special)
        arr = (ctypes.c_int * len(ids))(*ids)
        cap = 16 * len(ids) + 64
        out = ctypes.create_string_buffer(cap)
        n = self._lib.grm_tok_decode(self._h, arr, len(ids), out, cap, 1 if skip_special else 0)
        if n > cap:
            out = ctypes.create_string_buffer(n)
            n = self._lib.grm_tok_decode(self._h, arr, len(ids), out, n, 1 if skip_special else 0)
        return out.raw[:n]

    def decode(self, ids: Sequence[int], skip_special: bool = True) -> str:
        return self.decode_bytes(ids, skip_special).decode("utf-8", errors="replace")

    def special_id(self, token: str) -> int:
        if self._spm is not None:
            return self._spm.token_id(token)
        return self._lib.grm_tok_token_id(self._h, token.encode())

    def is_special(self, tok_id: int) -> bool:
        if self._spm is not None:
            return tok_id in self._spm.special_ids
        return bool(self._lib.grm_tok_is_special(self._h, tok_id))

    def eos(self) -> Optional[int]:
        name = self.cfg.get("eos_token")
        if isinstance(name, dict):
            name = name.get("content")
        for cand in (name, IM_END, EOT, "</s>", "<eos>"):
            if cand:
                i = self.special_id(cand)
                if i >= 0:
                    return i
        return None

    def eos2(self) -> Optional[int]:
        """Second end token (``<|im_end|>`` / ``<|endoftext|>`` / ``<|eot_id|>``) when distinct from eos."""
        e = self.eos()
        for cand in (IM_END, EOT, "<|eot_id|>", "<end_of_turn>"):
            i = self.special_id(cand)
            if i >= 0 and i != e:
                return i
        return None

    # ---- chat templates ----
    def template_kind(self) -> str:
        if self.special_id(IM_START) >= 0:
            return "chatml"
        if self.special_id("<start_of_turn>") >= 0:
            return "gemma"
        if self.special_id("<|start|>") >= 0:
            return "harmony"
        return "plain"

    def apply_chat_template(self, messages: list[dict], tools: Optional[list] = None, add_generation_prompt: bool = True,
                            enable_thinking: bool = True, reasoning_effort: Optional[str] = None) -> str:
        kind = self.template_kind()
        if kind == "chatml":
            return render_chatml(messages, tools, add_generation_prompt, enable_thinking)
        if kind == "gemma":
            out = "<bos>"
            for m in messages:
                role = "model" if m["role"] == "assistant" else "user"
                out += f"<start_of_turn>{role}\n{_text(m)}<end_of_turn>\n"
            return out + ("<start_of_turn>model\n" if add_generation_prompt else "")
        if kind == "harmony":
            out = ""
            if reasoning_effort:
                out += f"<|start|>system<|message|>Reasoning: {reasoning_effort}<|end|>"
            for m in messages:
                out += f"<|start|>{m['role']}<|message|>{_text(m)}<|end|>"
            return out + ("<|start|>assistant" if add_generation_prompt else "")
        out = "".join(f"{m['role']}: {_text(m)}\n" for m in messages)
        return out + ("assistant: " if add_generation_prompt else "")

    def encode_chat(self, messages, **kw) -> list[int]:
        return self.encode(self.apply_chat_template(messages, **kw), allow_special=True)


def _text(m: dict) -> str:
    c = m.get("content")
    if c is None:
        return ""
    if isinstance(c, list):          # OpenAI content parts
        return "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") in (None, "text"))
    return str(c)


TOOLS_HEAD = ("# Tools\n\nYou may call one or more functions to assist with the user query.\n\n"
              "You are provided with function signatures within <tools></tools> XML tags:\n<tools>")
TOOLS_TAIL = ("\n</tools>\n\nFor each function call, return a json object with function name and arguments within "
              "<tool_call></tool_call> XML tags:\n<tool_call>\n{\"name\": <function-name>, \"arguments\": <args-json-object>}\n"
              "</tool_call>")


def render_chatml(messages: list[dict], tools=None, add_generation_prompt=True, enable_thinking=True) -> str:
    """ChatML with the Qwen tool-calling conventions: tool signatures in the system turn, assistant
    tool calls as <tool_call> JSON blocks, tool results as <tool_response> inside a user turn."""
    out = ""
    msgs = list(messages)
    sys_text = ""
    if msgs and msgs[0]["role"] == "system":
        sys_text = _text(msgs.pop(0))
    if tools:
        out += f"{IM_START}system\n"
        if sys_text:
            out += sys_text + "\n\n"
        out += TOOLS_HEAD
        for t in tools:
            out += "\n" + json.dumps(t, ensure_ascii=False)
        out += TOOLS_TAIL + f"{IM_END}\n"
    elif sys_text:
        out += f"{IM_START}system\n{sys_text}{IM_END}\n"
    i = 0
    while i < len(msgs):
        m = msgs[i]
        role = m["role"]
        if role in ("user", "system"):
            out += f"{IM_START}{role}\n{_text(m)}{IM_END}\n"
        elif role == "assistant":
            out += f"{IM_START}assistant\n{_text(m)}"
            for tc in m.get("tool_calls") or []:
                fn = tc.get("function", tc)
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except json.JSONDecodeError:
                        pass
                out += ("\n" if out and not out.endswith("\n") else "") + "<tool_call>\n" + json.dumps(
                    {"name": fn.get("name"), "arguments": args}, ensure_ascii=False) + "\n</tool_call>"
            out += f"{IM_END}\n"
        elif role == "tool":
            out += f"{IM_START}user"
            while i < len(msgs) and msgs[i]["role"] == "tool":
                out += f"\n<tool_response>\n{_text(msgs[i])}\n</tool_response>"
                i += 1
            out += f"{IM_END}\n"
            continue
        else:
            raise ValueError(f"unknown role {role!r}")
        i += 1
    if add_generation_prompt:
        out += f"{IM_START}assistant\n"
        if not enable_thinking:
            out += "<think>\n\n</think>\n\n"
    return out
