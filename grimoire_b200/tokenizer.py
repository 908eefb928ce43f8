"""Tokenizer front end: the C++ byte-level BPE core (csrc/host/tokenizer.cpp) plus NFC
normalisation, special-token lookup and chat templates.

Reference: include/b70/tokenizer.hpp + src/tokenizer.cpp (load / encode / decode / special_id /
eos / eos2 / apply_chat_template; ChatML-Qwen JSON and XML tool templates with the reasoning-effort line, the
Gemma-4, Muse-Glimmer and K2-Horizon turn formats).
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
    def chat_template_text(self) -> str:
        """The checkpoint's own Jinja template (tokenizer_config.json or chat_template.jinja), read only to recognise which
        of the renderers below it is (set_chat_family, src/tokenizer.cpp:112-128)."""
        t = self.cfg.get("chat_template") if isinstance(self.cfg, dict) else None
        if isinstance(t, list):                      # [{"name": "default", "template": ...}, ...]
            t = next((e.get("template") for e in t if isinstance(e, dict) and e.get("name") in (None, "default")), None)
        if not t:
            f = self.dir / "chat_template.jinja"
            t = f.read_text() if f.exists() else ""
        return t or ""

    def chat_family(self) -> dict:
        """Switches of the Qwen XML-tool template family: ``xml_tools`` (function / parameter blocks instead of JSON tool
        calls), ``effort`` (a reasoning-effort system line), ``think_split`` (past answers carry their <think> block inline),
        ``default_effort`` (the template's declared default)."""
        if getattr(self, "_family", None) is None:
            import re

            t = self.chat_template_text()
            xml = ("<function=example_function_name>" in t and "do not tell the user about function calls" in t
                   and "multi_step_tool=true" in t)
            eff = xml and "Reasoning effort is set to xhigh." in t
            m = re.search(r"\breasoning_effort\s*\|\s*default\s*\(\s*(['\"])(xhigh|medium|low)\1", t) if eff else None
            self._family = {"xml_tools": xml, "effort": eff, "think_split": xml and "content.split('</think>')" in t,
                            "default_effort": m.group(2) if m else "xhigh"}
        return self._family

    def template_kind(self) -> str:
        if self.special_id("<|turn>") >= 0:
            return "gemma4"
        if self.special_id("<|begin_of_text|>") >= 0:
            return "muse"
        if self.special_id("<|ifm|im_start|>") >= 0:
            return "k2"
        if self.special_id(IM_START) >= 0:
            return "chatml_xml" if self.chat_family()["xml_tools"] else "chatml"
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
        if kind == "chatml_xml":
            return render_chatml_xml(messages, tools, enable_thinking, reasoning_effort, self.chat_family())
        if kind in ("gemma4", "muse", "k2"):
            if tools:
                raise ValueError("this model's chat template has no tool-call format this build renders")
            if kind == "gemma4":
                return render_gemma4(messages, thinking=enable_thinking)      # BOS is the encoder's
            return render_muse(messages) if kind == "muse" else render_k2(messages)
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

    def bos(self) -> int:
        """Id of the beginning-of-sequence token (tokenizer_config.json ``bos_token``, else ``<bos>``), or -1."""
        name = self.cfg.get("bos_token") if isinstance(self.cfg, dict) else None
        if isinstance(name, dict):
            name = name.get("content")
        i = self.special_id(name) if name else -1
        return i if i >= 0 else self.special_id("<bos>")

    @property
    def add_bos(self) -> bool:
        """Prompts start with BOS: the tokenizer says so, or it is the Gemma-4 one and says nothing (src/tokenizer.cpp:218-220)."""
        if isinstance(self.cfg, dict) and "add_bos_token" in self.cfg:
            return bool(self.cfg["add_bos_token"])
        return self.template_kind() == "gemma4"

    def with_bos(self, ids: list[int]) -> list[int]:
        b = self.bos()
        return [b] + ids if self.add_bos and b >= 0 and (not ids or ids[0] != b) else ids

    def encode_prompt(self, text: str) -> list[int]:
        """A raw completion prompt: special tokens in the text are honoured, BOS goes first when the tokenizer asks for it."""
        return self.with_bos(self.encode(text, allow_special=True))

    def encode_chat(self, messages, **kw) -> list[int]:
        return self.with_bos(self.encode(self.apply_chat_template(messages, **kw), allow_special=True))


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


# ---- family templates (src/tokenizer.cpp:1869-2135): Gemma-4, Muse-Glimmer, K2-Horizon and the Qwen XML-tool ChatML ----
def render_gemma4(messages: list[dict], thinking: bool = False) -> str:
    """``<|turn>role\n...<turn|>\n`` turns (assistant -> model, contents trimmed), an optional leading system / developer turn
    that also carries the thinking switch, and a closed empty thought channel when thinking is off.  BOS is the encoder's."""
    out, first = "", 0
    system = bool(messages) and messages[0]["role"] in ("system", "developer")
    if thinking or system:
        out += "<|turn>system\n"
        if thinking:
            out += "<|think|>\n"
        if system:
            out += _text(messages[0]).strip()
            first = 1
        out += "<turn|>\n"
    for m in messages[first:]:
        role = "model" if m["role"] == "assistant" else m["role"]
        if role not in ("user", "model", "system", "developer"):
            raise ValueError(f"gemma4 chat role is unsupported: {m['role']}")
        out += f"<|turn>{role}\n{_text(m).strip()}<turn|>\n"
    out += "<|turn>model\n"
    return out if thinking else out + "<|channel>thought\n<channel|>"


def render_muse(messages: list[dict], today: Optional[str] = None) -> str:
    """Muse-Glimmer's Harmony-style turns: ``<|start|>role<|message|>...<|eot|>``, a dated default system message when the
    conversation has none, the reasoning / recipients footer after a given one, past answers addressed ``to=user``."""
    import datetime

    date = today or datetime.date.today().isoformat()
    meta = "\n\nReasoning strength: high.\n\n# Valid recipients: \"self\", \"user\"."
    out = "<|begin_of_text|>"
    if not any(m["role"] == "system" for m in messages):
        out += ("<|start|>system<|message|>You are a helpful AI assistant.\nKnowledge cutoff: 2026-01-04.\n"
                f"Current date: {date}." + meta + "<|eot|>")
    for m in messages:
        if m["role"] == "system":
            out += "<|start|>system<|message|>" + _text(m) + meta + "<|eot|>"
        elif m["role"] == "user":
            out += "<|start|>user<|message|>" + _text(m) + "<|eot|>"
        elif m["role"] == "assistant":
            out += "<|start|>assistant to=user<|message|>" + _text(m) + "<|eot|>"
    return out + "<|start|>assistant"


def render_k2(messages: list[dict]) -> str:
    """K2-Horizon: its own ChatML-like markers, BOS first, no newline between turns, past answers with an empty think block
    and an assistant turn that opens one."""
    out = "<|ifm|begin_of_text|>"
    for m in messages:
        if m["role"] in ("system", "user"):
            out += f"<|ifm|im_start|>{m['role']}\n{_text(m)}<|ifm|im_end|>"
        elif m["role"] == "assistant":
            out += "<|ifm|im_start|>assistant<ifm|think>\n</ifm|think>" + _text(m) + "<|ifm|im_end|>"
    return out + "<|ifm|im_start|>assistant\n<ifm|think>\n"


XML_TOOL_INSTRUCTIONS = (
    "\n\nIf you choose to call a function ONLY reply in the following format with NO suffix:\n\n"
    "<tool_call>\n<function=example_function_name>\n<parameter=example_parameter_1>\nvalue_1\n"
    "</parameter>\n<parameter=example_parameter_2>\nThis is the value for the second parameter\n"
    "that can span\nmultiple lines\n</parameter>\n</function>\n</tool_call>\n\n<IMPORTANT>\n"
    "Reminder:\n- Function calls MUST follow the specified format: an inner <function=...></function> "
    "block must be nested within <tool_call></tool_call> XML tags\n- Required parameters MUST be "
    "specified\n- You may provide optional reasoning for your function call in natural language "
    "BEFORE the function call, but NOT after\n- If there is no function call available, answer the "
    "question like normal with your current knowledge and do not tell the user about function calls\n"
    "</IMPORTANT>")
EFFORT_XHIGH = ("Reasoning effort is set to xhigh. Please think carefully through the task, validate key "
                "assumptions, consider plausible alternatives, and prioritize correctness, consistency, and "
                "clarity in the final answer.")
EFFORT_LOW = ("Reasoning effort is set to low. Keep your thinking brief and focused, moving directly to the "
              "conclusion without unnecessary elaboration.")


def _xml_arg(v) -> str:
    return v if isinstance(v, str) else json.dumps(v, ensure_ascii=False) if isinstance(v, (dict, list)) else str(v)


def render_chatml_xml(messages: list[dict], tools=None, enable_thinking: bool = True, reasoning_effort: Optional[str] = None,
                      family: Optional[dict] = None) -> str:
    """The Qwen XML-tool template, line for line: tools block with the call-format instructions in the system turn, a
    reasoning-effort system line (templates that have one), past assistant turns with their <think> block, tool calls as
    ``<function=..><parameter=..>`` blocks, consecutive tool results grouped into one user turn."""
    fam = family or {"xml_tools": True, "effort": False, "think_split": False, "default_effort": "xhigh"}
    if not messages:
        raise ValueError("No messages provided.")
    ri = ""
    if fam["effort"] and enable_thinking:
        effort = reasoning_effort or fam["default_effort"]
        effort = "xhigh" if effort == "high" else effort
        if effort not in ("xhigh", "medium", "low"):
            raise ValueError(f"Unexpected reasoning effort {effort}. Supported types are xhigh (default), medium, and low.")
        ri = EFFORT_XHIGH if effort == "xhigh" else EFFORT_LOW if effort == "low" else ""
    out = ""
    first_system = messages[0]["role"] == "system"
    if tools:
        out += f"{IM_START}system\n"
        if ri:
            out += ri + "\n\n"
        out += "# Tools\n\nYou have access to the following functions:\n\n<tools>"
        for t in tools:
            out += "\n" + (t if isinstance(t, str) else json.dumps(t, ensure_ascii=False))
        out += "\n</tools>" + XML_TOOL_INSTRUCTIONS
        if first_system and _text(messages[0]).strip():
            out += "\n\n" + _text(messages[0]).strip()
        out += f"{IM_END}\n"
    elif first_system:
        c = _text(messages[0]).strip()
        if not fam["effort"]:
            out += f"{IM_START}system\n{c}{IM_END}\n"
        elif c:
            out += f"{IM_START}system\n" + (ri + "\n\n" if ri else "") + c + f"{IM_END}\n"
        elif ri:
            out += f"{IM_START}system\n{ri}{IM_END}\n"
    elif ri:
        out += f"{IM_START}system\n{ri}{IM_END}\n"

    def is_query(m) -> bool:
        c = _text(m).strip()
        return m["role"] == "user" and not (c.startswith("<tool_response>") and c.endswith("</tool_response>"))

    if not any(is_query(m) for m in messages):
        raise ValueError("No user query found in messages.")
    for i, m in enumerate(messages):
        role, c = m["role"], _text(m).strip()
        if role == "system":
            if i != 0:
                raise ValueError("System message must be at the beginning.")
        elif role == "user":
            out += f"{IM_START}user\n{c}{IM_END}\n"
        elif role == "assistant":
            r = m.get("reasoning_content") or m.get("reasoning") or ""
            if not r and fam["think_split"] and "</think>" in c:
                head = c[: c.find("</think>")].rstrip("\n")
                o = head.rfind("<think>")
                if o >= 0:
                    head = head[o + 7:]
                r = head.lstrip("\n")
                c = c[c.rfind("</think>") + 8:].lstrip("\n")
            out += f"{IM_START}assistant\n<think>\n{r.strip()}\n</think>\n\n{c}"
            for j, tc in enumerate(m.get("tool_calls") or []):
                fn = tc.get("function", tc)
                args = fn.get("arguments", {})
                if isinstance(args, str):
                    try:
                        args = json.loads(args)
                    except json.JSONDecodeError:
                        args = {}
                out += ("" if (j == 0 and not c.strip()) else "\n\n" if j == 0 else "\n") + f"<tool_call>\n<function={fn.get('name')}>\n"
                for k, v in (args or {}).items():
                    out += f"<parameter={k}>\n{_xml_arg(v)}\n</parameter>\n"
                out += "</function>\n</tool_call>"
            out += f"{IM_END}\n"
        elif role == "tool":
            if i > 0 and messages[i - 1]["role"] != "tool":
                out += f"{IM_START}user"
            out += f"\n<tool_response>\n{c}\n</tool_response>"
            if i + 1 == len(messages) or messages[i + 1]["role"] != "tool":
                out += f"{IM_END}\n"
        else:
            raise ValueError("Unexpected message role.")
    return out + f"{IM_START}assistant\n" + ("<think>\n" if enable_thinking else "<think>\n\n</think>\n\n")
