"""Rank lockstep through the control channel (gloo, 2 ranks): rank 0 drives a scheduler over a
ControlledEngine with TP=2, rank 1 only mirrors calls; concurrent requests must equal a single
rank, and a closed channel ends the worker with WorkerLost instead of hanging."""
import os
import socket
import threading

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.models.dense import DenseModel
from grimoire_b200.models.synthetic import random_state_dict

LIM = dict(max_slots=3, max_ctx=160, prefill_chunk=64, max_decode_rows=8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompts():
    g = torch.Generator().manual_seed(21)
    return [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (7, 40)]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    from grimoire_b200.parallel.bootstrap import init_parallel
    from grimoire_b200.parallel.control import ControlChannel, ControlledEngine, worker_loop
    from grimoire_b200.parallel.tp import TensorParallel
    from grimoire_b200.sched.scheduler import Scheduler

    lay = init_parallel(tp_world=world, pp_world=1, backend="gloo")
    try:
        cfg = tiny_dense()
        model = DenseModel.from_state_dict(cfg, random_state_dict(cfg, seed=6), "cpu", tp_rank=lay.tp_rank, tp_world=world)
        TensorParallel(lay.tp_group, "cpu").attach(model)
        eng = Engine(model, EngineLimits(**LIM))
        ch = ControlChannel(lay.control_group)
        if rank != 0:
            q.put(("worker", worker_loop(eng, ch)))
            return
        ce = ControlledEngine(eng, ch)
        s = Scheduler(ce, width=2, hold_ms=5.0, use_graph=False)
        res = [None, None]
        def work(i):
            res[i] = s.generate(_prompts()[i], 6)[0]
        ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
        [t.start() for t in ts]
        [t.join(timeout=120) for t in ts]
        s.shutdown()
        ce.shutdown()
        q.put(("front", res))
    finally:
        dist.destroy_process_group()


def test_scheduler_over_control_channel_equals_single_rank():
    cfg = tiny_dense()
    single = Engine(DenseModel.from_state_dict(cfg, random_state_dict(cfg, seed=6), "cpu"), EngineLimits(**LIM))
    want = [single.generate(p, 6) for p in _prompts()]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in procs]
    try:
        got = dict(q.get(timeout=180) for _ in procs)
        [p.join(timeout=60) for p in procs]
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    assert got["front"] == want
    assert got["worker"] > 10           # the worker really mirrored the calls
