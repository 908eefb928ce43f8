"""Hybrid linear-attention MoE benchmark (80B total / 3B active architecture): prompt read rate and
greedy decode rate, device-timed with CUDA events (max over ranks).  One GPU, or expert parallel
over the ranks of a ``torchrun`` launch:

    python -m grimoire_b200.bench.hybrid --prompt 4096 --decode 128
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        -m grimoire_b200.bench.hybrid --prompt 4096 --decode 128 [--nccl]

``--nccl`` runs the all-reduce composition instead of the fused dispatch/combine kernels (the
baseline the fused path is compared with).  ``--layers`` below 48 is a shape check, not the named
configuration.  Random weights, uniform-random prompt tokens.
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch
import torch.distributed as dist

from ..engine.engine import Engine, EngineLimits
from ..models.config import hybrid_dense_27b, hybrid_moe_80b
from ..models.hybrid import HybridModel
from ..ops import core as K


def _max_over_ranks(v: float, dev) -> float:
    if not dist.is_initialized():
        return v
    t = torch.tensor([v], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--model", default="moe_80b", choices=["moe_80b", "dense_27b"],
                    help="moe_80b: 512-expert hybrid, block fp8; dense_27b: the 27B hybrid with a dense FFN, int4 (use --layers 64)")
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--prompts", default="", help="comma-separated prompt lengths measured one after the other on one model build "
                                                  "(one JSON line each), e.g. 4096,16384,32768,65536")
    ap.add_argument("--decode", type=int, default=128)
    ap.add_argument("--timeline", action="store_true", help="also print a CUDA-event timeline (us per launch group, summed over "
                    "the layers) of one eager decode step and one prompt chunk")
    ap.add_argument("--users", type=int, default=1)
    ap.add_argument("--nccl", action="store_true", help="all-reduce composition instead of the fused expert-parallel kernels")
    ns = ap.parse_args(argv)
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = hybrid_dense_27b(ns.layers) if ns.model == "dense_27b" else hybrid_moe_80b(ns.layers)
    t0 = time.time()
    model = HybridModel.random(cfg, dev, seed=0, max_slots=max(ns.users, 2), ep_rank=rank, ep_world=world)
    ep = model.attach_ep(dist.group.WORLD, max_rows=4096, fused=not ns.nccl) if world > 1 else None
    torch.cuda.synchronize()
    build_s = time.time() - t0
    lengths = [int(v) for v in ns.prompts.split(",") if v] or [ns.prompt]
    eng = Engine(model, EngineLimits(max_slots=max(ns.users, 2), max_ctx=max(lengths) + ns.decode + 64, prefill_chunk=4096, max_decode_rows=16))
    for plen in lengths:
        ns.prompt = plen
        _measure(ns, eng, model, ep, cfg, world, rank, dev, build_s)
    if world > 1:
        eng.graphs.clear()
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()
    return 0


def _measure(ns, eng, model, ep, cfg, world, rank, dev, build_s) -> None:
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (ns.prompt,), generator=g, dtype=torch.int32) for _ in range(ns.users + 1)]
    s0 = eng.open()
    eng.prefill(s0, prompts[-1])          # warm-up
    eng.release(s0)
    seqs, firsts, pp = [], [], []
    for u in range(ns.users):
        s = eng.open()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        lg = eng.prefill(s, prompts[u])
        e1.record()
        torch.cuda.synchronize()
        pp.append(_max_over_ranks(e0.elapsed_time(e1), dev))
        seqs.append(s)
        firsts.append(int(lg.argmax()))
    use_graph = ep is None or ep.fused
    toks = list(firsts)
    if use_graph:
        graph = eng.build_step_graph(seqs, firsts, steps_ahead=ns.decode + 8)
        step = graph.replay
    else:
        def step():
            nonlocal toks
            pos = [s.length for s in seqs]
            toks = eng.decode_rows(toks, seqs, pos, use_graph=False)
            eng.commit_rows(seqs, toks, pos)
    for _ in range(4):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(ns.decode):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = _max_over_ranks(e0.elapsed_time(e1), dev) / ns.decode
    status = list(K.status_read())
    if rank == 0:
        print(json.dumps({"model": (f"hybrid dense-FFN 27B int4, {ns.layers}L" if ns.model == "dense_27b"
                                    else f"hybrid-moe {ns.layers}L (48L = 80B/3B-active config)"), "n_gpus": world,
                          "parallelism": "single" if world == 1 else (f"ep{world}-nccl-allreduce" if ns.nccl else f"ep{world}-fused"),
                          "prompt": ns.prompt, "users": ns.users,
                          "pp_tok_s": round(ns.prompt * 1000.0 / (sum(pp) / len(pp)), 1), "pp_ms": round(sum(pp) / len(pp), 2),
                          "decode_tok_s": round(ns.users * 1000.0 / ms, 1), "decode_ms_per_step": round(ms, 3),
                          "weights_gb_per_gpu": round(model.weight_bytes() / 1e9, 2), "build_s": round(build_s, 1),
                          "device_status": status}), flush=True)
    if ns.timeline and world == 1:
        from ..utils import trace

        out = {}
        pos = [s.length for s in seqs]
        for _ in range(2):
            eng.decode_rows(toks, seqs, pos, use_graph=False)
        trace.timeline.enable(True)
        eng.decode_rows(toks, seqs, pos, use_graph=False)
        out["decode_step_us"] = {k: round(v, 1) for k, v in trace.timeline.dump().items()}
        trace.timeline.enable(False)
        sx = eng.open()
        trace.timeline.enable(True)
        eng.prefill(sx, prompts[-1][: min(ns.prompt, 4096)])
        out["prefill_chunk_us"] = {k: round(v, 1) for k, v in trace.timeline.dump().items()}
        trace.timeline.enable(False)
        eng.release(sx)
        print(json.dumps({"timeline": out}), flush=True)
    for s in seqs:
        eng.release(s)
    eng.graphs.clear()


if __name__ == "__main__":
    raise SystemExit(main())
