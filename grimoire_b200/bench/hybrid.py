"""Hybrid linear-attention MoE benchmark (80B total / 3B active architecture): prompt read rate and
greedy decode rate on one GPU, device-timed with CUDA events.  ``--layers`` below 48 is a shape
check, not the named configuration."""
from __future__ import annotations

import argparse
import json
import time

import torch

from ..engine.engine import Engine, EngineLimits
from ..models.config import hybrid_moe_80b
from ..models.hybrid import HybridModel
from ..ops import core as K


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--users", type=int, default=1)
    ns = ap.parse_args(argv)
    cfg = hybrid_moe_80b(ns.layers)
    t0 = time.time()
    model = HybridModel.random(cfg, "cuda", seed=0, max_slots=max(ns.users, 2))
    torch.cuda.synchronize()
    build_s = time.time() - t0
    eng = Engine(model, EngineLimits(max_slots=max(ns.users, 2), max_ctx=ns.prompt + ns.decode + 64, prefill_chunk=4096, max_decode_rows=16))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (ns.prompt,), generator=g, dtype=torch.int32) for _ in range(ns.users + 1)]
    s0 = eng.open()
    eng.prefill(s0, prompts[-1])          # warm-up
    eng.release(s0)
    seqs, firsts, pp = [], [], []
    for u in range(ns.users):
        s = eng.open()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        lg = eng.prefill(s, prompts[u])
        e1.record()
        torch.cuda.synchronize()
        pp.append(e0.elapsed_time(e1))
        seqs.append(s)
        firsts.append(int(lg.argmax()))
    graph = eng.build_step_graph(seqs, firsts, steps_ahead=ns.decode + 8)
    for _ in range(4):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(ns.decode):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / ns.decode
    print(json.dumps({"model": f"hybrid-moe {ns.layers}L (48L = 80B/3B-active config)", "prompt": ns.prompt, "users": ns.users,
                      "pp_tok_s": round(ns.prompt * 1000.0 / (sum(pp) / len(pp)), 1), "pp_ms": round(sum(pp) / len(pp), 2),
                      "decode_tok_s": round(ns.users * 1000.0 / ms, 1), "decode_ms_per_step": round(ms, 3),
                      "weights_gb": round(model.weight_bytes() / 1e9, 2), "build_s": round(build_s, 1), "device_status": list(K.status_read())}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
