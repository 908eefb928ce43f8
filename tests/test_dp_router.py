"""Data-parallel replica router with two in-process replicas (CPU): least-loaded choice with prefix affinity, streaming
passes through unchanged, a lost replica answers 502 once and is skipped afterwards."""
import http.client
import json
import threading

import pytest

from grimoire_b200.api import Grimoire
from grimoire_b200.config import EngineConfig
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.parallel.dp import Replica, Router, make_router_server
from grimoire_b200.server import make_server
from tests.fixtures.mini_model import write_checkpoint


@pytest.fixture(scope="module")
def cluster(tmp_path_factory):
    d = tmp_path_factory.mktemp("dp") / "model"
    write_checkpoint(d, tiny_dense(), seed=1, tokenizer=True)
    servers, gs = [], []
    for _ in range(2):
        ec = EngineConfig(model=str(d), ctx=256, seq_slots=2, max_batch=2, prefill_chunk=64, admit_hold_ms=1.0, mtp=0).validate()
        g = Grimoire.load(ec, device="cpu")
        srv = make_server(g, "127.0.0.1", 0)
        threading.Thread(target=srv.serve_forever, daemon=True).start()
        servers.append(srv); gs.append(g)
    reps = [Replica("127.0.0.1", s.server_address[1]) for s in servers]
    router = make_router_server(reps, "127.0.0.1", 0)
    threading.Thread(target=router.serve_forever, daemon=True).start()
    yield router, reps, servers
    router.shutdown(); router.server_close()
    for s, g in zip(servers, gs):
        try:
            s.shutdown(); s.server_close()
        except Exception:
            pass
        g.close()


def _post(port, body, path="/v1/completions"):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=120)
    c.request("POST", path, json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, r.getheader("Content-Type"), data


def test_router_policy_least_loaded_with_affinity():
    reps = [Replica("h", 1), Replica("h", 2), Replica("h", 3)]
    r = Router(reps, affinity_slack=1)
    body = {"prompt": "the same beginning of a prompt"}
    a = r.pick(body); b = r.pick(body)
    assert a is b                                   # same prefix, same replica (its prefix cache is warm)
    c = r.pick(body)
    assert c is not a                               # the home replica is now busier than the idlest by more than the slack
    reps[reps.index(c)].healthy = False
    d = r.pick({"prompt": "another prompt"})
    assert d.healthy
    for x in (a, b, c, d):
        r.done(x)
    assert sum(x.inflight for x in reps) == 0


def test_requests_flow_through_the_router_and_match_a_replica(cluster):
    router, reps, servers = cluster
    port = router.server_address[1]
    body = {"prompt": "hello world", "max_tokens": 6}
    st, _, via = _post(port, body)
    st2, _, direct = _post(reps[0].port, body)
    assert st == st2 == 200
    assert json.loads(via)["choices"][0]["text"] == json.loads(direct)["choices"][0]["text"]
    st, ctype, raw = _post(port, {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True,
                                  "chat_template_kwargs": {"enable_thinking": False}}, "/v1/chat/completions")
    assert st == 200 and ctype == "text/event-stream" and raw.decode().rstrip().endswith("data: [DONE]")
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=30)
    c.request("GET", "/health")
    assert c.getresponse().status == 200
    c.close()


def test_lost_replica_is_skipped(cluster):
    router, reps, servers = cluster
    port = router.server_address[1]
    servers[1].shutdown(); servers[1].server_close()
    seen = set()
    for i in range(6):
        st, _, data = _post(port, {"prompt": f"prompt number {i} " * 3, "max_tokens": 2})
        seen.add(st)
        assert st in (200, 502)
    assert 200 in seen
    assert not reps[1].check() and reps[0].check()
    st, _, _ = _post(port, {"prompt": "after the loss", "max_tokens": 2})
    assert st == 200
