"""Serving metrics in the Prometheus text format (``GET /metrics``) and an optional JSONL step log.

The reference only prints to stdout (capability banner, SPEC_STATS lines; it has no Prometheus endpoint and no
structured logs); this adds tok/s counters, a TTFT histogram, queue depth, KV pages in use,
speculative accept length and per-collective byte counters."""
from __future__ import annotations

import json
import threading
import time
from typing import Optional

_BUCKETS = (0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0, 60.0)


class Metrics:
    def __init__(self, step_log: str = ""):
        self.lock = threading.Lock()
        self.counters = {"requests_total": 0, "requests_failed_total": 0, "prompt_tokens_total": 0, "generation_tokens_total": 0,
                         "spec_drafted_total": 0, "spec_accepted_total": 0, "spec_rounds_total": 0, "prefix_tokens_reused_total": 0,
                         "comm_bytes_total": 0}
        self.gauges = {"queue_depth": 0, "running": 0, "kv_pages_used": 0, "kv_pages_total": 0}
        self.ttft = [0] * (len(_BUCKETS) + 1)
        self.ttft_sum = 0.0
        self.ttft_count = 0
        self.started = time.time()
        self._log = open(step_log, "a") if step_log else None

    def inc(self, name: str, v: float = 1) -> None:
        with self.lock:
            self.counters[name] = self.counters.get(name, 0) + v

    def set(self, name: str, v: float) -> None:
        with self.lock:
            self.gauges[name] = v

    def observe_ttft(self, seconds: float) -> None:
        with self.lock:
            for i, b in enumerate(_BUCKETS):
                if seconds <= b:
                    self.ttft[i] += 1
                    break
            else:
                self.ttft[-1] += 1
            self.ttft_sum += seconds
            self.ttft_count += 1

    def step(self, **fields) -> None:
        if self._log is not None:
            fields["t"] = round(time.time() - self.started, 6)
            self._log.write(json.dumps(fields) + "\n")
            self._log.flush()

    def render(self) -> str:
        with self.lock:
            out = []
            for k, v in self.counters.items():
                out += [f"# TYPE grimoire_{k} counter", f"grimoire_{k} {v}"]
            for k, v in self.gauges.items():
                out += [f"# TYPE grimoire_{k} gauge", f"grimoire_{k} {v}"]
            acc = 0
            out.append("# TYPE grimoire_ttft_seconds histogram")
            for b, n in zip(_BUCKETS, self.ttft):
                acc += n
                out.append(f'grimoire_ttft_seconds_bucket{{le="{b}"}} {acc}')
            out.append(f'grimoire_ttft_seconds_bucket{{le="+Inf"}} {acc + self.ttft[-1]}')
            out += [f"grimoire_ttft_seconds_sum {self.ttft_sum}", f"grimoire_ttft_seconds_count {self.ttft_count}"]
            d, a, r = self.counters["spec_drafted_total"], self.counters["spec_accepted_total"], self.counters["spec_rounds_total"]
            out += ["# TYPE grimoire_spec_accept_length gauge", f"grimoire_spec_accept_length {((a + r) / r) if r else 1.0}"]
            return "\n".join(out) + "\n"
