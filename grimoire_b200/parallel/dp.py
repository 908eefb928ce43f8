"""Data parallelism: N engine replicas (each possibly a TP x PP group) behind ONE front end.

The reference has no replica mode (one engine per process group; users are batched, not
replicated).  On an 8-GPU box replicas multiply throughput for models that fit one GPU (or one TP
group): e.g. DP4 x TP2.  The router is a small reverse proxy: it forwards OpenAI requests to the
replica with the fewest requests in flight, with prefix affinity -- requests whose prompt starts
with the same text go to the same replica so its prefix cache is hit -- and streams the response
back unchanged.  A replica that fails health checks is skipped; requests in flight on it fail with
a 502 and new ones go elsewhere, so a lost replica is not fatal.
"""
from __future__ import annotations

import hashlib
import http.client
import json
import os
import signal
import subprocess
import sys
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer


class Replica:
    def __init__(self, host: str, port: int):
        self.host, self.port = host, port
        self.inflight = 0
        self.healthy = True
        self.served = 0

    def check(self, timeout: float = 2.0) -> bool:
        try:
            c = http.client.HTTPConnection(self.host, self.port, timeout=timeout)
            c.request("GET", "/health")
            ok = c.getresponse().status == 200
            c.close()
        except OSError:
            ok = False
        self.healthy = ok
        return ok


class Router:
    def __init__(self, replicas: list[Replica], affinity_chars: int = 256, affinity_slack: int = 2):
        self.replicas = replicas
        self.lock = threading.Lock()
        self.affinity_chars = affinity_chars
        self.affinity_slack = affinity_slack

    @staticmethod
    def prompt_key(body: dict, n: int) -> str:
        if "messages" in body:
            text = json.dumps(body["messages"], sort_keys=True)
        else:
            text = str(body.get("prompt", ""))
        return hashlib.sha1(text[:n].encode()).hexdigest()

    def pick(self, body: dict) -> Replica:
        with self.lock:
            live = [r for r in self.replicas if r.healthy]
            if not live:
                raise RuntimeError("no healthy replica")
            least = min(r.inflight for r in live)
            home = live[int(self.prompt_key(body, self.affinity_chars), 16) % len(live)]
            # prefix affinity unless the home replica is clearly busier than the idlest one
            r = home if home.inflight <= least + self.affinity_slack else min(live, key=lambda x: x.inflight)
            r.inflight += 1
            return r

    def done(self, r: Replica) -> None:
        with self.lock:
            r.inflight -= 1
            r.served += 1


class ProxyHandler(BaseHTTPRequestHandler):
    protocol_version = "HTTP/1.1"

    def log_message(self, fmt, *args):
        return

    def _relay(self, method: str, body: bytes | None, replica: Replica):
        c = http.client.HTTPConnection(replica.host, replica.port, timeout=3600)
        c.request(method, self.path, body, {"Content-Type": "application/json"} if body is not None else {})
        r = c.getresponse()
        self.send_response(r.status)
        ctype = r.getheader("Content-Type", "application/json")
        self.send_header("Content-Type", ctype)
        if ctype.startswith("text/event-stream"):
            self.send_header("Connection", "close")
            self.end_headers()
            while True:
                chunk = r.read1(65536)
                if not chunk:
                    break
                self.wfile.write(chunk)
                self.wfile.flush()
        else:
            data = r.read()
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)
        c.close()

    def do_GET(self):
        router: Router = self.server.router
        if self.path == "/health":
            ok = any(r.healthy for r in router.replicas)
            data = b'{"status":"ok"}' if ok else b'{"status":"down"}'
            self.send_response(200 if ok else 503)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)
            return
        live = [r for r in router.replicas if r.healthy]
        if not live:
            self.send_error(503)
            return
        self._relay("GET", None, live[0])

    def do_POST(self):
        router: Router = self.server.router
        n = int(self.headers.get("Content-Length", "0"))
        raw = self.rfile.read(n) if n else b""
        try:
            body = json.loads(raw.decode() or "{}")
        except json.JSONDecodeError:
            body = {}
        try:
            rep = router.pick(body if isinstance(body, dict) else {})
        except RuntimeError as e:
            data = json.dumps({"error": {"message": str(e), "type": "engine_error"}}).encode()
            self.send_response(503)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)
            return
        try:
            self._relay("POST", raw, rep)
        except OSError as e:
            rep.healthy = False
            try:
                data = json.dumps({"error": {"message": f"replica lost: {e}", "type": "engine_error"}}).encode()
                self.send_response(502)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)
            except OSError:
                pass
        finally:
            router.done(rep)


def make_router_server(replicas: list[Replica], host: str, port: int) -> ThreadingHTTPServer:
    srv = ThreadingHTTPServer((host, port), ProxyHandler)
    srv.daemon_threads = True
    srv.router = Router(replicas)
    return srv


def run_replicas(n: int, port: int, server_args: list[str], gpus_per_replica: int = 1) -> int:
    """Start n ``serve`` processes on ports port+1.., each pinned to its GPUs, and route on ``port``."""
    procs, reps = [], []
    for i in range(n):
        env = dict(os.environ)
        env["CUDA_VISIBLE_DEVICES"] = ",".join(str(i * gpus_per_replica + k) for k in range(gpus_per_replica))
        p = port + 1 + i
        procs.append(subprocess.Popen([sys.executable, "-m", "grimoire_b200", "serve", "--port", str(p), "--host", "127.0.0.1",
                                       *server_args], env=env))
        reps.append(Replica("127.0.0.1", p))
    deadline = time.time() + 1800
    while time.time() < deadline and not all(r.check() for r in reps):
        if any(p.poll() is not None for p in procs):
            break
        time.sleep(1.0)
    srv = make_router_server(reps, "0.0.0.0", port)

    def stop(signum, frame):
        for p in procs:
            p.send_signal(signal.SIGTERM)
        threading.Thread(target=srv.shutdown, daemon=True).start()

    signal.signal(signal.SIGTERM, stop)
    signal.signal(signal.SIGINT, stop)

    def health_loop():
        while True:
            time.sleep(5.0)
            for r in reps:
                r.check()

    threading.Thread(target=health_loop, daemon=True).start()
    print(f"[grimoire-b200] DP router on :{port} over {n} replicas", flush=True)
    try:
        srv.serve_forever()
    finally:
        for p in procs:
            try:
                p.wait(timeout=60)
            except subprocess.TimeoutExpired:
                p.kill()
        srv.server_close()
    return 0
