"""Speculative decoding benchmark: 27B-class dense model with MXFP4 weights and a one-layer MTP draft
head, K drafts per round, greedy verify through the multi-row verify attention path.

    python -m grimoire_b200.bench.spec                              # 1 user on 1 GPU: 512 in / 512 out, K = 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29517 \
        -m grimoire_b200.bench.spec                                  # one user per GPU (data-parallel replicas)

The draft head is the target's final layer plus Gaussian noise (sigma 0.01 of the weight scale); with
random-init weights its predictions are rarely the target's, so the accepted length is reported
beside tok/s (mean tokens emitted per verify round = accepted drafts + the bonus token), together
with the plain (non-speculative) decode rate of the same model.  Timing: CUDA events around the whole
generation on the launching stream, max over ranks; the aggregate is users x 512 tokens / that time.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import time

import torch
import torch.distributed as dist

from ..engine.engine import Engine, EngineLimits
from ..ops import linear as _linear
from ..engine.generation import GenerationOptions, OracleDrafter, generate_tokens
from ..models.config import dense_27b
from ..models.dense import DenseModel
from ..models.mtp import MtpDrafter, MtpHead
from ..ops import core as K


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=64, help="fewer layers is a shape check, not the named configuration")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--out", type=int, default=512)
    ap.add_argument("--depth", type=int, default=3)
    ap.add_argument("--quant", default="mxfp4", choices=["mxfp4", "int4"])
    ap.add_argument("--draft-vocab", type=int, default=65536)
    ap.add_argument("--oracle-accept", type=float, default=0.7,
                    help="per-draft acceptance probability of the oracle drafter (0 = skip that measurement)")
    ns = ap.parse_args(argv)
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = dataclasses.replace(dense_27b(ns.layers), quant=ns.quant)
    t0 = time.time()
    model = DenseModel.random(cfg, dev, seed=0)
    eng = Engine(model, EngineLimits(max_slots=2, max_ctx=ns.prompt + ns.out + 64, prefill_chunk=4096, max_decode_rows=8, extra_kv_layers=1))
    drafter = MtpDrafter(eng, MtpHead.random_from_target(model, seed=0, noise=0.01, draft_vocab=ns.draft_vocab))
    torch.cuda.synchronize()
    build_s = time.time() - t0
    g = torch.Generator().manual_seed(100 + rank)
    prompt = torch.randint(0, cfg.vocab_size, (ns.prompt,), generator=g).tolist()

    def timed(depth: int, dr=None):
        opts = GenerationOptions(max_new=ns.out, draft_depth=depth, drafter=(dr or drafter) if depth else None)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        toks, _ = generate_tokens(eng, prompt, opts)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return toks, ms, opts.stats

    generate_tokens(eng, prompt[:64], GenerationOptions(max_new=8, draft_depth=ns.depth, drafter=drafter))   # warm-up: graphs, allocator
    generate_tokens(eng, prompt[:64], GenerationOptions(max_new=8))
    plain, plain_ms, _ = timed(0)
    spec, spec_ms, st = timed(ns.depth)
    oracle = None
    if ns.oracle_accept > 0:
        # the verify path at a realistic accepted length: a drafter that knows the greedy continuation and is wrong with a
        # dialled probability (the random-weight MTP head is never right, so it only measures the cost of rejection)
        od = OracleDrafter(prompt + plain, accept=ns.oracle_accept, vocab=cfg.vocab_size, seed=rank)
        otoks, oms, ost = timed(ns.depth, od)
        oracle = {"accept_probability": ns.oracle_accept, "tok_s": round(world * len(otoks) * 1000.0 / oms, 1),
                  "accepted_length": round(ost.accept_length, 3), "rounds": ost.rounds, "tokens_equal_plain": otoks == plain}
    if rank == 0:
        print(json.dumps({"model": f"27B dense {ns.quant} + MTP head ({ns.layers} layers)", "n_gpus": world, "users": world,
                          "parallelism": "single" if world == 1 else f"dp{world}", "prompt": ns.prompt, "out": ns.out, "draft_depth": ns.depth,
                          "spec_tok_s": round(world * len(spec) * 1000.0 / spec_ms, 1), "accepted_length": round(st.accept_length, 3),
                          "rounds": st.rounds, "drafted": st.drafted, "accepted": st.accepted,
                          "plain_tok_s": round(world * len(plain) * 1000.0 / plain_ms, 1), "tokens_equal_plain": spec == plain,
                          # attaching the drafter switched every height to the batch-invariant kernels (both timed runs)
                          "batch_invariant_kernels": _linear.BATCH_INVARIANT,
                          "oracle_drafter": oracle,
                          "includes_prefill": True, "mtp_bytes": drafter.head.nbytes(), "build_s": round(build_s, 1),
                          "device_status": list(K.status_read()), "data": "synthetic"}), flush=True)
    if world > 1:
        eng.graphs.clear()
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
