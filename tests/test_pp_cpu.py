"""Pipeline parallelism on CPU ranks (gloo): 2 and 3 stages must emit the single-process tokens;
each stage owns only its layers and its share of the KV pool (tools/test_parallel_e2e.cpp,
test_pp_server.cpp in the reference: token-identical output vs one process)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.models.dense import DenseModel
from grimoire_b200.models.synthetic import random_state_dict

LIM = dict(max_slots=2, max_ctx=192, prefill_chunk=32, max_decode_rows=8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cfg():
    c = tiny_dense()
    c.num_hidden_layers = 3
    c.layer_types = ["full_attention"] * 3
    return c


def _prompts():
    g = torch.Generator().manual_seed(11)
    return [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (70, 9, 33)]      # different lengths, chunked


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from grimoire_b200.parallel.pp import PipelineParallel

        cfg = _cfg()
        sd = random_state_dict(cfg, seed=4)
        model = DenseModel.from_state_dict(cfg, sd, "cpu", pp_rank=rank, pp_world=world)
        pp = PipelineParallel(dist.group.WORLD, "cpu")
        pp.attach(model)
        eng = Engine(model, EngineLimits(**LIM))
        outs = [eng.generate(p, 8) for p in _prompts()]          # three requests down a resident pipeline
        q.put((rank, outs, len(model.layers), len(eng.kv.layers), dict(pp.stats)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_pp_tokens_equal_single_process(world):
    cfg = _cfg()
    sd = random_state_dict(cfg, seed=4)
    single_eng = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), EngineLimits(**LIM))
    single = [single_eng.generate(p, 8) for p in _prompts()]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    try:
        res = [q.get(timeout=180) for _ in procs]
        [p.join(timeout=60) for p in procs]
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    layers = 0
    for rank, outs, n_layers, n_kv, stats in res:
        assert outs == single, (rank, outs, single)
        assert n_layers == n_kv and n_layers >= 1
        layers += n_layers
        if rank < world - 1:
            assert stats["sends"] > 0
    assert layers == 3
