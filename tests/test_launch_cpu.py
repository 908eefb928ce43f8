"""``grimoire multi PP 2`` / ``multi CP 2`` / ``multi UP 2`` end to end on CPU ranks: the launcher starts two gloo ranks, rank 0 serves HTTP
over a ControlledEngine, rank 1 mirrors the engine calls and runs the second pipeline stage (PP) or its half of every
prompt chunk's rows (CP); the completion must equal the single-process one (tools/test_pp_server.cpp in the reference: same tokens through a two-stage server)."""
import http.client
import json
import os
import signal
import socket
import subprocess
import sys
import time

import pytest

from grimoire_b200.api import Grimoire
from grimoire_b200.config import EngineConfig
from grimoire_b200.models.config import tiny_dense
from tests.fixtures.mini_model import write_checkpoint


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _post(port, body, timeout=120):
    c = http.client.HTTPConnection("127.0.0.1", port, timeout=timeout)
    c.request("POST", "/v1/completions", json.dumps(body), {"Content-Type": "application/json"})
    r = c.getresponse()
    data = r.read()
    c.close()
    return r.status, json.loads(data)


@pytest.mark.parametrize("mode", ["PP", "CP", "UP"])
def test_multi_2_rank_server_matches_single_process(tmp_path, mode):
    d = tmp_path / "model"
    cfg = tiny_dense()
    cfg.num_hidden_layers = 3
    cfg.layer_types = ["full_attention"] * 3
    write_checkpoint(d, cfg, seed=6, tokenizer=True)
    body = {"prompt": "hello world, how are you", "max_tokens": 8}
    # single process answer through the same public path
    from grimoire_b200.server import make_server
    import threading

    ec = EngineConfig(model=str(d), ctx=256, seq_slots=2, max_batch=2, prefill_chunk=64, admit_hold_ms=1.0, copy_drafts=0, mtp=0).validate()
    g = Grimoire.load(ec, device="cpu")
    srv = make_server(g, "127.0.0.1", 0)
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    st, want = _post(srv.server_address[1], body)
    srv.shutdown(); g.close(); srv.server_close()
    assert st == 200
    port, mport = _free_port(), _free_port()
    env = dict(os.environ, GRIMOIRE_SEQ_SLOTS="2", GRIMOIRE_MAX_BATCH="2", GRIMOIRE_PREFILL_CHUNK="64", GRIMOIRE_ADMIT_HOLD_MS="1",
               GRIMOIRE_COPY="0", GRIMOIRE_MTP="0", CUDA_VISIBLE_DEVICES="", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(mport), "-m", "grimoire_b200.parallel.launch", "--mode", mode, "--model", str(d), "--ctx", "256",
           "--host", "127.0.0.1", "--port", str(port)]
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, start_new_session=True)
    try:
        deadline = time.time() + 180
        up = False
        while time.time() < deadline and proc.poll() is None:
            try:
                c = http.client.HTTPConnection("127.0.0.1", port, timeout=2)
                c.request("GET", "/health")
                up = c.getresponse().status == 200
                c.close()
                if up:
                    break
            except OSError:
                time.sleep(0.5)
        assert up, "the two-rank server did not come up: " + (proc.stdout.read() if proc.poll() is not None else "timeout")
        st, got = _post(port, body)
        assert st == 200
        assert got["choices"][0]["text"] == want["choices"][0]["text"]
        assert got["usage"] == want["usage"]
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGTERM)
            try:
                proc.wait(timeout=60)
            except subprocess.TimeoutExpired:
                os.killpg(proc.pid, signal.SIGKILL)
