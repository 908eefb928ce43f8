"""OpenAI-compatible HTTP server.

Routes, JSON shapes and error types follow tools/grimoire_server.cpp (routes :323-420, SSE
:341-386, non-streaming :387-417, errors :313-322): ``GET /health``, ``GET /v1/models`` (reports the
scheduler width), ``POST /v1/chat/completions``, ``POST /v1/completions``, plus ``GET /metrics``.
One OS thread per connection (ThreadingHTTPServer), tokens are produced by the scheduler thread
and written by the request thread, a client disconnect cancels the job at the next token, SIGTERM /
SIGINT stop accepting, end live generations at the next token and let the step in flight finish.
"""
from __future__ import annotations

import argparse
import json
import signal
import sys
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Optional

from . import config as cfgmod
from .engine.generation import generation_budget
from .http_request import BadRequest, ResponseDecoder, parse_completion_request
from .utils.metrics import Metrics

WARMUP_PROMPTS = (73, 333, 777, 2153)     # start-up warm-up prompt lengths (grimoire_server.cpp:280-302)


def _err(message: str, kind: str) -> bytes:
    return json.dumps({"error": {"message": message, "type": kind}}).encode()


class Handler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"
    server_version = "grimoire-b200"

    def log_message(self, fmt, *args):  # quiet: one line per request is printed by handle_completion
        return

    # ---- helpers ----
    def _send(self, code: int, body: bytes, ctype: str = "application/json") -> None:
        self.send_response(code)
        self.send_header("Content-Type", ctype)
        self.send_header("Content-Length", str(len(body)))
        self.end_headers()
        self.wfile.write(body)

    def do_GET(self):
        app = self.server.app
        if self.path == "/health":
            return self._send(200, b'{"status":"ok"}')
        if self.path == "/v1/models":
            body = {"object": "list", "data": [{"id": app.model_id, "object": "model"}],
                    "grimoire": {"decoding": "greedy,top_k,top_p,temperature", "concurrency": app.sched.width}}
            return self._send(200, json.dumps(body).encode())
        if self.path == "/metrics":
            app.refresh_gauges()
            return self._send(200, app.metrics.render().encode(), "text/plain; version=0.0.4")
        self._send(404, _err("not found", "invalid_request_error"))

    def do_POST(self):
        if self.path not in ("/v1/chat/completions", "/v1/completions"):
            return self._send(404, _err("not found", "invalid_request_error"))
        chat = self.path.endswith("chat/completions")
        try:
            n = int(self.headers.get("Content-Length", "0"))
            raw = self.rfile.read(n) if n > 0 else b""
            try:
                body = json.loads(raw.decode("utf-8"))
            except (json.JSONDecodeError, UnicodeDecodeError) as e:
                raise BadRequest(f"invalid JSON: {e}") from None
            req = parse_completion_request(body, chat)
            self.server.app.handle_completion(self, req)
        except BadRequest as e:
            self.server.app.metrics.inc("requests_failed_total")
            self._send(400, _err(str(e), "invalid_request_error"))
        except ValueError as e:      # prompt too long and other std::invalid_argument-class failures
            self.server.app.metrics.inc("requests_failed_total")
            self._send(400, _err(str(e), "invalid_request_error"))
        except (BrokenPipeError, ConnectionResetError):
            pass
        except Exception as e:       # engine failure
            self.server.app.metrics.inc("requests_failed_total")
            try:
                self._send(500, _err(str(e), "engine_error"))
            except Exception:
                pass


class App:
    def __init__(self, grimoire, metrics: Optional[Metrics] = None):
        self.g = grimoire
        self.tok = grimoire.tokenizer
        self.sched = grimoire.scheduler()
        self.metrics = metrics or Metrics(grimoire.config.step_log)
        self.model_id = grimoire.name or "grimoire-b200"
        self.stopping = threading.Event()

    def refresh_gauges(self) -> None:
        kv = self.g.engine.kv
        self.metrics.set("kv_pages_used", kv.pages_used())
        self.metrics.set("kv_pages_total", kv.num_pages)
        self.metrics.set("running", len(self.sched.jobs))

    def _encode(self, req) -> list[int]:
        if self.tok is None:
            # synthetic models have no tokenizer: accept space-separated token ids
            text = req.prompt if not req.chat else " ".join(str(m.get("content", "")) for m in req.messages)
            try:
                return [int(t) for t in text.split()]
            except ValueError:
                raise BadRequest("this server runs a synthetic model without a tokenizer: send space-separated token ids")
        if req.chat:
            return self.tok.encode_chat(req.messages, tools=req.tools, enable_thinking=req.enable_thinking,
                                        reasoning_effort=req.reasoning_effort)
        return self.tok.encode_prompt(req.prompt)

    def _piece(self, ids: list[int], state: dict) -> str:
        """Incremental detokenisation that never splits a UTF-8 sequence."""
        if self.tok is None:
            return " ".join(str(i) for i in ids) + " "
        state["pending"] += ids
        raw = self.tok.decode_bytes(state["pending"])
        try:
            text = raw.decode("utf-8")
        except UnicodeDecodeError:
            if len(state["pending"]) < 8:
                return ""
            text = raw.decode("utf-8", errors="replace")
        state["pending"] = []
        return text

    def handle_completion(self, h: Handler, req) -> None:
        ids = self._encode(req)
        budget = generation_budget(len(ids), req.max_tokens, self.g.engine.limits.max_ctx)
        eos = self.tok.eos() if self.tok else None
        eos2 = self.tok.eos2() if self.tok else None
        rid = f"cmpl-{time.monotonic_ns()}"
        obj = "chat.completion" if req.chat else "text_completion"
        self.metrics.inc("requests_total")
        self.metrics.inc("prompt_tokens_total", len(ids))
        thinking = bool(req.chat and self.tok is not None and self.tok.special_id("<think>") >= 0)
        dec = ResponseDecoder(thinking=thinking, tools=bool(req.tools), starts_in_think=thinking and req.enable_thinking)
        state = {"pending": []}
        t0 = time.monotonic()
        n_out = [0]
        first = [None]

        if req.stream:
            h.send_response(200)
            h.send_header("Content-Type", "text/event-stream")
            h.send_header("Cache-Control", "no-cache")
            h.send_header("Connection", "close")
            h.end_headers()
            chunk_obj = "chat.completion.chunk" if req.chat else "text_completion"

            def send(delta=None, text=None, finish=None, usage=None) -> bool:
                choice = {"index": 0, "finish_reason": finish}
                if req.chat:
                    choice["delta"] = delta if delta is not None else {}
                else:
                    choice["text"] = text if text is not None else ""
                payload = {"id": rid, "object": chunk_obj, "model": self.model_id, "choices": [choice]}
                if usage is not None:
                    payload["usage"] = usage
                try:
                    h.wfile.write(b"data: " + json.dumps(payload, ensure_ascii=False).encode() + b"\n\n")
                    h.wfile.flush()
                    return True
                except (BrokenPipeError, ConnectionResetError, OSError):
                    return False

            def on_token(t: int) -> bool:
                if self.stopping.is_set():
                    return False
                if first[0] is None:
                    first[0] = time.monotonic()
                    self.metrics.observe_ttft(first[0] - t0)
                n_out[0] += 1
                if t == eos or t == eos2:
                    return True
                piece = self._piece([t], state)
                ok = True
                for kind, text in dec.push(piece) if req.chat else [("content", piece)]:
                    if not text:
                        continue
                    ok = send(delta={"reasoning_content" if kind == "reasoning" else "content": text}, text=text) and ok
                return ok

            try:
                out, why, job = self.sched.generate(ids, budget, eos, eos2, on_token, req.sampling)
            except Exception as e:
                try:
                    h.wfile.write(b"data: " + _err(str(e), "engine_error") + b"\n\n")
                    h.wfile.write(b"data: [DONE]\n\n")
                except Exception:
                    pass
                self.metrics.inc("requests_failed_total")
                return
            tail, calls = dec.finish() if req.chat else ([], [])
            for kind, text in tail:
                send(delta={"reasoning_content" if kind == "reasoning" else "content": text}, text=text)
            if calls:
                why = "tool_calls"
                send(delta={"tool_calls": [dict(c, index=i) for i, c in enumerate(calls)]})
            usage = {"prompt_tokens": len(ids), "completion_tokens": len(out), "total_tokens": len(ids) + len(out)}
            send(delta={}, text="", finish=why, usage=usage)
            try:
                h.wfile.write(b"data: [DONE]\n\n")
                h.wfile.flush()
            except Exception:
                pass
        else:
            def on_token(t: int) -> bool:
                if first[0] is None:
                    first[0] = time.monotonic()
                    self.metrics.observe_ttft(first[0] - t0)
                return not self.stopping.is_set()

            out, why, job = self.sched.generate(ids, budget, eos, eos2, on_token, req.sampling)
            body_ids = [t for t in out if t != eos and t != eos2]
            text = self._piece(body_ids, state) if body_ids else ""
            usage = {"prompt_tokens": len(ids), "completion_tokens": len(out), "total_tokens": len(ids) + len(out)}
            if req.chat:
                dec.push(text)
                _, calls = dec.finish()
                msg = {"role": "assistant", "content": dec.content if (dec.content or not calls) else None}
                if dec.reasoning:
                    msg["reasoning_content"] = dec.reasoning
                if calls:
                    msg["tool_calls"] = calls
                    why = "tool_calls"
                choice = {"index": 0, "message": msg, "finish_reason": why}
            else:
                choice = {"index": 0, "text": text, "finish_reason": why}
            h._send(200, json.dumps({"id": rid, "object": obj, "model": self.model_id, "choices": [choice], "usage": usage},
                                    ensure_ascii=False).encode())
        self.metrics.inc("generation_tokens_total", len(out))
        st = job.stats
        self.metrics.inc("spec_drafted_total", st.drafted)
        self.metrics.inc("spec_accepted_total", st.accepted)
        self.metrics.inc("spec_rounds_total", st.rounds)
        if self.g.config.spec_stats and st.rounds:
            print(f"[{rid}] {st.line()}", flush=True)


def make_server(grimoire, host: str, port: int) -> ThreadingHTTPServer:
    srv = ThreadingHTTPServer((host, port), Handler)
    srv.daemon_threads = True
    srv.app = App(grimoire)
    return srv


def warm_up(grimoire) -> None:
    """Touch every kernel / graph shape before the first request (prompts of 73/333/777/2153 tokens)."""
    import torch

    g = torch.Generator().manual_seed(0)
    for n in WARMUP_PROMPTS:
        if n + 8 >= grimoire.engine.limits.max_ctx:
            break
        ids = torch.randint(0, grimoire.model.cfg.vocab_size, (n,), generator=g).tolist()
        grimoire.generate(ids, 4)


def serve(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="grimoire-server", description="OpenAI-compatible server for grimoire-b200")
    cfgmod.add_engine_flags(ap)
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--no-warmup", action="store_true")
    ns = ap.parse_args(argv)
    if not ns.model:
        ap.error("--model is required (a HF directory, or synthetic:<preset>)")
    ec = cfgmod.from_args(ns)
    from .api import Grimoire

    g = Grimoire.load(ec)
    if not ns.no_warmup:
        warm_up(g)
    srv = make_server(g, ec.host, ec.port)

    def stop(signum, frame):
        # stop accepting, end live generations at the next token, let the step in flight finish
        srv.app.stopping.set()
        threading.Thread(target=srv.shutdown, daemon=True).start()

    signal.signal(signal.SIGTERM, stop)
    signal.signal(signal.SIGINT, stop)
    print(f"[grimoire-b200] listening on {ec.host}:{ec.port} (concurrency {srv.app.sched.width})", flush=True)
    try:
        srv.serve_forever()
    finally:
        g.close()
        srv.server_close()
    return 0


if __name__ == "__main__":
    sys.exit(serve())
