"""HTTP wire contract on a synthetic checkpoint with a real tokenizer (CPU): health, models,
completions, chat completions, SSE streaming, 400s, metrics."""
import http.client
import json
import threading

import pytest

from grimoire_b200.api import Grimoire
from grimoire_b200.config import EngineConfig
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.server import make_server
from tests.fixtures.mini_model import write_checkpoint


@pytest.fixture(scope="module")
def server(tmp_path_factory):
    d = tmp_path_factory.mktemp("srv") / "model"
    cfg = tiny_dense()
    write_checkpoint(d, cfg, seed=1, quant="gptq", tokenizer=True)
    ec = EngineConfig(model=str(d), ctx=256, seq_slots=4, max_batch=4, prefill_chunk=64, admit_hold_ms=1.0).validate()
    g = Grimoire.load(ec, device="cpu")
    srv = make_server(g, "127.0.0.1", 0)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    yield srv
    srv.shutdown()
    g.close()
    srv.server_close()


def _req(srv, method, path, body=None):
    c = http.client.HTTPConnection("127.0.0.1", srv.server_address[1], timeout=120)
    c.request(method, path, None if body is None else json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, r.getheader("Content-Type"), data


def test_health_models_metrics(server):
    assert _req(server, "GET", "/health") == (200, "application/json", b'{"status":"ok"}')
    st, _, data = _req(server, "GET", "/v1/models")
    j = json.loads(data)
    assert st == 200 and j["object"] == "list" and j["data"][0]["object"] == "model"
    assert j["grimoire"] == {"decoding": "greedy,top_k,top_p,temperature", "concurrency": 4}
    st, ctype, data = _req(server, "GET", "/metrics")
    assert st == 200 and ctype.startswith("text/plain") and b"grimoire_kv_pages_total" in data


def test_completion_and_chat_non_streaming(server):
    st, _, data = _req(server, "POST", "/v1/completions", {"prompt": "hello world", "max_tokens": 6})
    j = json.loads(data)
    assert st == 200 and j["object"] == "text_completion" and j["id"].startswith("cmpl-")
    ch = j["choices"][0]
    assert ch["index"] == 0 and isinstance(ch["text"], str) and ch["finish_reason"] in ("length", "stop")
    u = j["usage"]
    assert u["completion_tokens"] <= 6 and u["total_tokens"] == u["prompt_tokens"] + u["completion_tokens"]
    st, _, data = _req(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi there"}], "max_tokens": 5,
                                                                "chat_template_kwargs": {"enable_thinking": False}})
    j = json.loads(data)
    assert st == 200 and j["object"] == "chat.completion" and j["choices"][0]["message"]["role"] == "assistant"


def test_streaming_sse_shape(server):
    c = http.client.HTTPConnection("127.0.0.1", server.server_address[1], timeout=120)
    c.request("POST", "/v1/chat/completions", json.dumps({"messages": [{"role": "user", "content": "hello"}], "max_tokens": 6, "stream": True,
                                                          "chat_template_kwargs": {"enable_thinking": False}}),
              {"Content-Type": "application/json"})
    r = c.getresponse()
    assert r.status == 200 and r.getheader("Content-Type") == "text/event-stream"
    raw = r.read().decode()
    c.close()
    events = [e[len("data: "):] for e in raw.split("\n\n") if e.startswith("data: ")]
    assert events[-1] == "[DONE]"
    chunks = [json.loads(e) for e in events[:-1]]
    assert all(ch["object"] == "chat.completion.chunk" for ch in chunks)
    final = chunks[-1]
    assert final["choices"][0]["delta"] == {} and final["choices"][0]["finish_reason"] in ("length", "stop") and "usage" in final
    assert all(ch["choices"][0]["finish_reason"] is None for ch in chunks[:-1])


def test_errors(server):
    st, _, data = _req(server, "POST", "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "n": 2})
    assert st == 400 and json.loads(data)["error"]["type"] == "invalid_request_error"
    st, _, data = _req(server, "POST", "/v1/completions", {"prompt": "word " * 400, "max_tokens": 4})
    assert st == 400 and "context" in json.loads(data)["error"]["message"]
    st, _, _ = _req(server, "POST", "/v1/nope", {})
    assert st == 404
