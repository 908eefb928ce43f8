"""OpenAI request validation and response decoding.

Field-for-field parity with the reference's parse_completion_request / ResponseDecoder /
parse_xml_tool_calls (include/b70/http_request.hpp:69-323): unsupported options are refused with a
ValueError (HTTP 400 ``invalid_request_error``) rather than ignored.
"""
from __future__ import annotations

import json
import re
import secrets
from dataclasses import dataclass, field
from typing import Optional

from .engine.sampling import SamplingOptions


class BadRequest(ValueError):
    pass


@dataclass
class CompletionRequest:
    chat: bool
    messages: list = field(default_factory=list)
    prompt: str = ""
    stream: bool = False
    max_tokens: int = 4096
    sampling: SamplingOptions = field(default_factory=SamplingOptions)
    tools: Optional[list] = None
    tool_choice: str = "auto"
    reasoning_effort: Optional[str] = None
    enable_thinking: bool = True
    model: str = ""


def _num(body, key, default, lo=None, hi=None, integer=False):
    v = body.get(key, default)
    if v is None:
        return default
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise BadRequest(f"'{key}' must be a number")
    if integer and int(v) != v:
        raise BadRequest(f"'{key}' must be an integer")
    if (lo is not None and v < lo) or (hi is not None and v > hi):
        raise BadRequest(f"'{key}' out of range")
    return int(v) if integer else float(v)


def parse_completion_request(body: dict, chat: bool) -> CompletionRequest:
    if not isinstance(body, dict):
        raise BadRequest("request body must be a JSON object")
    r = CompletionRequest(chat=chat, model=str(body.get("model", "")))
    r.stream = bool(body.get("stream", False))
    mt = body.get("max_completion_tokens", body.get("max_tokens", 4096))
    if mt is None:
        mt = 4096
    if isinstance(mt, bool) or not isinstance(mt, int) or mt < 1:
        raise BadRequest("'max_tokens' must be a positive integer")
    r.max_tokens = mt
    if _num(body, "n", 1, integer=True) != 1:
        raise BadRequest("only n=1 is supported")
    for pen in ("presence_penalty", "frequency_penalty"):
        if _num(body, pen, 0.0) != 0.0:
            raise BadRequest(f"'{pen}' is not supported")
    for key in ("stop", "logprobs", "top_logprobs", "response_format", "logit_bias"):
        if body.get(key) not in (None, False, [], {}):
            raise BadRequest(f"'{key}' is not supported")
    temperature = _num(body, "temperature", 0.0, lo=0.0, hi=10.0)
    top_p = _num(body, "top_p", 1.0)
    if not (0.0 < top_p <= 1.0):
        raise BadRequest("'top_p' must be in (0, 1]")
    top_k = _num(body, "top_k", 20, lo=1, hi=64, integer=True)
    seed = _num(body, "seed", 0, integer=True)
    r.sampling = SamplingOptions(temperature=temperature, top_k=top_k, top_p=top_p, seed=seed & ((1 << 64) - 1))
    if chat:
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs:
            raise BadRequest("'messages' must be a non-empty array")
        for m in msgs:
            if not isinstance(m, dict) or m.get("role") not in ("system", "user", "assistant", "tool"):
                raise BadRequest("message role must be system, user, assistant or tool")
            c = m.get("content")
            if c is not None and not isinstance(c, (str, list)):
                raise BadRequest("message content must be a string, an array of parts or null")
        r.messages = msgs
        tools = body.get("tools")
        if tools is not None:
            if not isinstance(tools, list):
                raise BadRequest("'tools' must be an array")
            r.tools = tools or None
        tc = body.get("tool_choice", "auto")
        if tc not in ("auto", "none"):
            raise BadRequest("'tool_choice' must be \"auto\" or \"none\"")
        r.tool_choice = tc
        if tc == "none":
            r.tools = None
        re_eff = body.get("reasoning_effort")
        if re_eff is not None and re_eff not in ("low", "medium", "high", "none", "minimal"):
            raise BadRequest("'reasoning_effort' must be low, medium or high")
        r.reasoning_effort = re_eff
        ctk = body.get("chat_template_kwargs") or {}
        if not isinstance(ctk, dict):
            raise BadRequest("'chat_template_kwargs' must be an object")
        r.enable_thinking = bool(ctk.get("enable_thinking", True))
    else:
        p = body.get("prompt")
        if isinstance(p, list) and len(p) == 1 and isinstance(p[0], str):
            p = p[0]
        if not isinstance(p, str) or not p:
            raise BadRequest("'prompt' must be a non-empty string")
        r.prompt = p
    return r


_TOOL_RE = re.compile(r"<tool_call>\s*(.*?)\s*</tool_call>", re.S)
_FUNC_RE = re.compile(r"<function=([^>\s]+)>\s*(.*?)\s*</function>", re.S)
_PARAM_RE = re.compile(r"<parameter=([^>\s]+)>\s*(.*?)\s*</parameter>", re.S)


def parse_xml_tool_calls(text: str) -> tuple[str, list[dict]]:
    """Split generated text into (visible content, tool calls).  Accepts the JSON form
    ``<tool_call>{"name":..,"arguments":{..}}</tool_call>`` and the XML form
    ``<tool_call><function=name><parameter=k>v</parameter></function></tool_call>``."""
    calls = []
    for m in _TOOL_RE.finditer(text):
        body = m.group(1)
        name, args = None, None
        try:
            obj = json.loads(body)
            if isinstance(obj, dict) and "name" in obj:
                name, args = obj["name"], obj.get("arguments", {})
        except json.JSONDecodeError:
            fm = _FUNC_RE.search(body)
            if fm:
                name = fm.group(1)
                args = {}
                for pm in _PARAM_RE.finditer(fm.group(2)):
                    v = pm.group(2)
                    try:
                        args[pm.group(1)] = json.loads(v)
                    except json.JSONDecodeError:
                        args[pm.group(1)] = v
        if name is None:
            continue
        calls.append({"id": "call_" + secrets.token_hex(8), "type": "function",
                      "function": {"name": name, "arguments": args if isinstance(args, str) else json.dumps(args, ensure_ascii=False)}})
    content = _TOOL_RE.sub("", text)
    if calls:
        content = content.rstrip()       # trailing whitespace before a tool call is trimmed
    return content, calls


class ResponseDecoder:
    """Incremental split of the generated text into reasoning / content / tool-call segments.

    ``push(piece)`` returns a list of (kind, text) with kind in {"reasoning", "content"}; text inside
    a ``<tool_call>`` block is held back and returned by ``finish()`` as parsed calls."""

    def __init__(self, thinking: bool, tools: bool, starts_in_think: bool = False):
        self.thinking, self.tools = thinking, tools
        self.in_think = starts_in_think
        self.buf = ""
        self.held = ""
        self.content = ""
        self.reasoning = ""

    def _emit(self, kind, text, out):
        if not text:
            return
        if kind == "reasoning":
            self.reasoning += text
        else:
            self.content += text
        out.append((kind, text))

    def push(self, piece: str) -> list[tuple[str, str]]:
        out: list[tuple[str, str]] = []
        self.buf += piece
        while self.buf:
            if self.held:
                end = self.buf.find("</tool_call>")
                if end < 0:
                    self.held += self.buf
                    self.buf = ""
                    break
                self.held += self.buf[: end + len("</tool_call>")]
                self.buf = self.buf[end + len("</tool_call>"):]
                self._done_calls = getattr(self, "_done_calls", "") + self.held
                self.held = ""
                continue
            tags = []
            if self.thinking:
                tags.append("</think>" if self.in_think else "<think>")
            if self.tools and not self.in_think:
                tags.append("<tool_call>")
            hit, which = -1, None
            for tg in tags:
                i = self.buf.find(tg)
                if i >= 0 and (hit < 0 or i < hit):
                    hit, which = i, tg
            if hit < 0:
                # keep a tail that could be the start of a tag
                keep = 0
                for tg in tags:
                    for k in range(min(len(tg) - 1, len(self.buf)), 0, -1):
                        if self.buf.endswith(tg[:k]):
                            keep = max(keep, k)
                            break
                emit, self.buf = (self.buf[: len(self.buf) - keep], self.buf[len(self.buf) - keep:]) if keep else (self.buf, "")
                self._emit("reasoning" if self.in_think else "content", emit, out)
                break
            self._emit("reasoning" if self.in_think else "content", self.buf[:hit], out)
            self.buf = self.buf[hit + len(which):]
            if which == "<think>":
                self.in_think = True
            elif which == "</think>":
                self.in_think = False
                self.buf = self.buf.lstrip("\n")
            else:
                self.held = "<tool_call>"
        return out

    def finish(self) -> tuple[list[tuple[str, str]], list[dict]]:
        out: list[tuple[str, str]] = []
        if self.buf and not self.held:
            self._emit("reasoning" if self.in_think else "content", self.buf, out)
            self.buf = ""
        _, calls = parse_xml_tool_calls(getattr(self, "_done_calls", ""))
        if calls:
            self.content = self.content.rstrip()
        return out, calls
