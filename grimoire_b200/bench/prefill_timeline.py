"""Per-kernel-group CUDA-event timeline of one 4,096-token prefill chunk of the 27B dense int4 model, on one GPU or under
``torch.distributed.run`` with tensor parallelism (fused sequence-parallel GEMMs, default) or context parallelism (``--cp``):

    python -m grimoire_b200.bench.prefill_timeline
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        -m grimoire_b200.bench.prefill_timeline [--cp]

Events are recorded on the launching stream between the groups of launches the model's forward pass names (utils/trace.py),
summed over the layers, and printed per rank 0 as microseconds per layer; the chunk's wall time from two events around the
whole call is printed beside the sum (the marks themselves cost a few microseconds each).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..engine.engine import Engine, EngineLimits
from ..models.config import dense_27b
from ..models.dense import DenseModel
from ..utils import trace


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--cp", action="store_true", help="context parallelism (whole-model replicas) instead of tensor parallelism")
    ns = ap.parse_args(argv)
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = dense_27b(ns.layers)
    mode = "1 gpu"
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        if ns.cp:
            from ..parallel.cp import ContextParallel

            model = DenseModel.random(cfg, dev, seed=0)
            ContextParallel(dist.group.WORLD, dev).attach(model, max_rows=ns.prompt)
            mode = f"cp{world}"
        else:
            from ..parallel.tp import TensorParallel

            model = DenseModel.random(cfg, dev, seed=0, tp_rank=rank, tp_world=world)
            TensorParallel(dist.group.WORLD, dev).attach(model, max_rows=ns.prompt)
            mode = f"tp{world}"
    else:
        model = DenseModel.random(cfg, dev, seed=0)
    eng = Engine(model, EngineLimits(max_slots=2, max_ctx=ns.prompt + 64, prefill_chunk=ns.prompt, max_decode_rows=8))
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (ns.prompt,), generator=g, dtype=torch.int32) for _ in range(3)]
    s = eng.open()
    eng.prefill(s, prompts[0])                       # warm-up (allocator, resident bf16 weight copies)
    eng.release(s)
    s = eng.open()
    eng.prefill(s, prompts[1])
    eng.release(s)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    trace.timeline.enable(True)
    s = eng.open()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    eng.prefill(s, prompts[2])
    e1.record()
    torch.cuda.synchronize()
    groups = trace.timeline.dump()
    trace.timeline.enable(False)
    total_ms = e0.elapsed_time(e1)
    if rank == 0:
        per_layer = {k: round(v / ns.layers, 1) for k, v in groups.items() if k != "tail"}
        print(json.dumps({"bench": "prefill timeline", "parallelism": mode, "prompt": ns.prompt, "layers": ns.layers,
                          "chunk_ms": round(total_ms, 2), "tok_s": round(ns.prompt * 1000.0 / total_ms, 1),
                          "us_per_layer": per_layer, "sum_us_per_layer": round(sum(per_layer.values()), 1),
                          "tail_us": round(groups.get("tail", 0.0), 1)}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
