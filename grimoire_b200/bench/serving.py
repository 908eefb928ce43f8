"""Pooled paged-KV serving benchmark on the 27B-class dense int4 model.

    python -m grimoire_b200.bench.serving                       # 8 x (512 in, 128 out), ctx cap 24,576
    python -m grimoire_b200.bench.serving --http                 # the same burst over HTTP (loopback, streaming)
    python -m grimoire_b200.bench.serving --long 131072          # one 131,072-token prompt in 4,096-token chunks + 128 decode

The serving run drives the continuous-batching scheduler exactly as the HTTP server does: N client
threads submit at the same instant, each request is a random prompt of ``--prompt`` tokens with
``--out`` greedy output tokens, the KV cache is the shared page pool under a per-request context
cap.  Reported: aggregate output tok/s over the wall time of the whole burst and p50 time to first
token (submit -> first token delivered to the client), the two figures the reference quotes for its
pooled-KV serving (tools/bench/pp1117/RESULTS-2026-11-20.md:43-45: 150.7 tok/s aggregate and p50 TTFT
2.897 s at 8 users).  Wall-clock here is legitimate: the metric *is* client-observed latency on one
GPU; the device-timed numbers live in bench.py.  Random-init weights, uniform-random tokens.
"""
from __future__ import annotations

import argparse
import json
import statistics
import threading
import time

import torch

from ..engine.engine import Engine, EngineLimits
from ..models.config import dense_27b
from ..models.dense import DenseModel
from ..ops import core as K
from ..sched.scheduler import Scheduler


def run_serving(eng: Engine, users: int, prompt_len: int, out_len: int, vocab: int, rounds: int) -> dict:
    sched = Scheduler(eng, width=max(8, users), prefill_chunk=4096, interleave_chunk=1024)
    g = torch.Generator().manual_seed(7)
    results = []
    try:
        for rnd in range(rounds + 1):                 # the first pass is the warm-up (graph capture, allocator)
            prompts = [torch.randint(0, vocab, (prompt_len,), generator=g).tolist() for _ in range(users)]
            ttft, done, lock = [0.0] * users, [0] * users, threading.Lock()
            start = threading.Barrier(users + 1)

            def client(i):
                first = []
                start.wait()
                t0 = time.perf_counter()

                def on_token(tok):
                    if not first:
                        first.append(time.perf_counter() - t0)
                    return True
                toks, _, _ = sched.generate(prompts[i], out_len, on_token=on_token)
                with lock:
                    ttft[i], done[i] = first[0], len(toks)

            threads = [threading.Thread(target=client, args=(i,)) for i in range(users)]
            for t in threads:
                t.start()
            start.wait()
            t0 = time.perf_counter()
            for t in threads:
                t.join()
            wall = time.perf_counter() - t0
            if rnd:
                results.append({"wall_s": wall, "tokens": sum(done), "tok_s": sum(done) / wall,
                                "p50_ttft_s": statistics.median(ttft), "max_ttft_s": max(ttft)})
    finally:
        sched.shutdown()
    best = max(results, key=lambda r: r["tok_s"])
    return {"users": users, "prompt": prompt_len, "out": out_len, "rounds": rounds,
            "aggregate_tok_s": round(statistics.median(r["tok_s"] for r in results), 1), "best_tok_s": round(best["tok_s"], 1),
            "p50_ttft_s": round(statistics.median(r["p50_ttft_s"] for r in results), 4),
            "max_ttft_s": round(max(r["max_ttft_s"] for r in results), 4)}


def run_serving_http(model, eng: Engine, users: int, prompt_len: int, out_len: int, vocab: int, rounds: int) -> dict:
    """The same burst through the product's front door: an in-process OpenAI-compatible server on a loopback port, one
    streaming ``POST /v1/completions`` per client (the synthetic model takes space-separated token ids as the prompt);
    time to first token is the arrival of the first event that carries text."""
    import http.client

    from ..api import Grimoire
    from ..config import EngineConfig
    from ..server import make_server

    ec = EngineConfig(model="synthetic:dense_27b", ctx=eng.limits.max_ctx, seq_slots=eng.limits.max_slots, max_batch=max(8, users),
                      prefill_chunk=4096, copy_drafts=0, mtp=0)
    g = Grimoire(model, eng, None, ec, name="dense-27b-int4")
    srv = make_server(g, "127.0.0.1", 0)
    port = srv.server_address[1]
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    gen = torch.Generator().manual_seed(7)
    results = []
    try:
        for rnd in range(rounds + 1):
            prompts = [" ".join(str(int(t)) for t in torch.randint(0, vocab, (prompt_len,), generator=gen)) for _ in range(users)]
            ttft, done, lock = [0.0] * users, [0] * users, threading.Lock()
            start = threading.Barrier(users + 1)

            def client(i):
                body = json.dumps({"prompt": prompts[i], "max_tokens": out_len, "stream": True, "temperature": 0}).encode()
                start.wait()
                t0 = time.perf_counter()
                c = http.client.HTTPConnection("127.0.0.1", port, timeout=600)
                c.request("POST", "/v1/completions", body, {"Content-Type": "application/json"})
                r = c.getresponse()
                first, n = None, 0
                for line in r:
                    if not line.startswith(b"data: ") or line.startswith(b"data: [DONE]"):
                        continue
                    ev = json.loads(line[6:])
                    text = ev["choices"][0].get("text") or ""
                    if text:
                        if first is None:
                            first = time.perf_counter() - t0
                        n += len(text.split())
                c.close()
                with lock:
                    ttft[i], done[i] = first if first is not None else float("nan"), n

            threads = [threading.Thread(target=client, args=(i,)) for i in range(users)]
            for t in threads:
                t.start()
            start.wait()
            t0 = time.perf_counter()
            for t in threads:
                t.join()
            wall = time.perf_counter() - t0
            if rnd:
                results.append({"wall_s": wall, "tokens": sum(done), "tok_s": sum(done) / wall,
                                "p50_ttft_s": statistics.median(ttft), "max_ttft_s": max(ttft)})
    finally:
        srv.shutdown()
        g.close()
        srv.server_close()
    best = max(results, key=lambda r: r["tok_s"])
    return {"transport": "http (loopback, SSE)", "users": users, "prompt": prompt_len, "out": out_len, "rounds": rounds,
            "aggregate_tok_s": round(statistics.median(r["tok_s"] for r in results), 1), "best_tok_s": round(best["tok_s"], 1),
            "p50_ttft_s": round(statistics.median(r["p50_ttft_s"] for r in results), 4),
            "max_ttft_s": round(max(r["max_ttft_s"] for r in results), 4)}


def run_long(eng: Engine, prompt_len: int, out_len: int, vocab: int) -> dict:
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, vocab, (prompt_len,), generator=g, dtype=torch.int32)
    s = eng.open()
    warm = eng.open()
    eng.prefill(warm, prompt[:4096])
    eng.release(warm)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    lg = eng.prefill(s, prompt)
    e1.record()
    torch.cuda.synchronize()
    read_ms = e0.elapsed_time(e1)
    graph = eng.build_step_graph([s], [int(lg.argmax())], steps_ahead=out_len + 8)
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(out_len):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    write_ms = e0.elapsed_time(e1) / out_len
    return {"prompt": prompt_len, "chunk": 4096, "read_tok_s": round(prompt_len * 1000.0 / read_ms, 1), "read_s": round(read_ms / 1000.0, 4),
            "write_tok_s": round(1000.0 / write_ms, 1), "write_ms_per_step": round(write_ms, 3)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--users", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--out", type=int, default=128)
    ap.add_argument("--ctx-cap", type=int, default=24576)
    ap.add_argument("--rounds", type=int, default=3)
    ap.add_argument("--layers", type=int, default=64, help="fewer layers is a shape check, not the named configuration")
    ap.add_argument("--long", type=int, default=0, help="long-context variant: prompt length (e.g. 131072)")
    ap.add_argument("--http", action="store_true", help="drive the burst through the HTTP server instead of the scheduler API")
    ns = ap.parse_args(argv)
    cfg = dense_27b(ns.layers) if ns.layers != 64 else dense_27b()
    import os

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cp = None
    if world > 1:
        # several ranks (torch.distributed.run): context parallelism for the long prompt -- whole-model replicas, every
        # 4,096-token chunk's rows split over the ranks, replicated caches and decode
        import torch.distributed as dist

        from ..parallel.cp import ContextParallel

        if not ns.long:
            ap.error("the multi-rank form of this benchmark is the long-context variant (--long)")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        cp = ContextParallel(dist.group.WORLD, dev)
    t0 = time.time()
    model = DenseModel.random(cfg, dev, seed=0)
    if cp is not None:
        cp.attach(model, max_rows=4096)
    torch.cuda.synchronize()
    build_s = time.time() - t0
    if ns.long:
        eng = Engine(model, EngineLimits(max_slots=2, max_ctx=ns.long + ns.out + 64, prefill_chunk=4096, max_decode_rows=8))
        res = {"bench": "long-context", "parallelism": f"cp{world}" if cp is not None else "1 gpu", **run_long(eng, ns.long, ns.out, cfg.vocab_size)}
        if cp is not None:
            import torch.distributed as dist

            t = torch.tensor([res["read_s"], res["write_ms_per_step"]], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)                # device-timed per rank; the slowest rank counts
            res["read_s"], res["write_ms_per_step"] = round(float(t[0]), 4), round(float(t[1]), 3)
            res["read_tok_s"], res["write_tok_s"] = round(ns.long / float(t[0]), 1), round(1000.0 / float(t[1]), 1)
    else:
        # the pool holds what the users can actually use, not users x cap (pages are mapped on demand)
        eng = Engine(model, EngineLimits(max_slots=max(ns.users, 8) + 1, max_ctx=ns.ctx_cap, prefill_chunk=4096, max_decode_rows=32,
                                         kv_pages=(max(ns.users, 8) * (ns.prompt + ns.out + 64) + ns.ctx_cap) // 16 + 16))
        run = (lambda: run_serving_http(model, eng, ns.users, ns.prompt, ns.out, cfg.vocab_size, ns.rounds)) if ns.http else \
            (lambda: run_serving(eng, ns.users, ns.prompt, ns.out, cfg.vocab_size, ns.rounds))
        res = {"bench": "pooled-kv serving", "ctx_cap": ns.ctx_cap, **run()}
    res.update({"model": f"27B dense int4 g128 ({ns.layers} layers)", "build_s": round(build_s, 1), "device_status": list(K.status_read()),
                "data": "synthetic"})
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
