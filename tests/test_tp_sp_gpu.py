"""Fused sequence-parallel prefill on 2 GPUs: GEMM -> reduce-scatter push, reduce + norm + all-gather
push on the token shard, all-gather-wait -> GEMM.  The last-token logits must match a single-GPU
prefill of the same weights, through chunks that take the fused path (256 rows) and a ragged tail
that takes the NCCL path."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _setup(world=2):
    """The fused path needs whole 128-row tiles per rank: chunks of 128 * world rows, two of them plus a ragged tail."""
    from grimoire_b200.models.config import small_dense
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = small_dense(layers=3, wide=world > 2)
    sd = random_state_dict(cfg, seed=0)
    g = torch.Generator().manual_seed(3)
    chunk = 128 * world
    prompt = torch.randint(0, cfg.vocab_size, (2 * chunk + 88,), generator=g).tolist()
    return cfg, sd, prompt, chunk


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from grimoire_b200.engine.engine import Engine, EngineLimits
        from grimoire_b200.models.dense import DenseModel
        from grimoire_b200.ops.core import status_read
        from grimoire_b200.parallel.tp import TensorParallel

        cfg, sd, prompt, chunk = _setup(world)
        model = DenseModel.from_state_dict(cfg, sd, dev, tp_rank=rank, tp_world=world)
        tp = TensorParallel(dist.group.WORLD, dev, fused=True)
        tp.attach(model, max_rows=chunk)
        eng = Engine(model, EngineLimits(max_slots=2, max_ctx=len(prompt) + 128, prefill_chunk=chunk, max_decode_rows=16))
        s = eng.open()
        lg = eng.prefill(s, prompt).float().cpu()
        torch.cuda.synchronize()
        q.put((rank, lg, getattr(tp, "_rs_expect", 0), status_read()))
        del eng, model
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_sp_prefill_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.dense import DenseModel

    cfg, sd, prompt, chunk = _setup(world)
    eng = Engine(DenseModel.from_state_dict(cfg, sd, "cuda:0"), EngineLimits(max_slots=2, max_ctx=len(prompt) + 128, prefill_chunk=chunk,
                                                                            max_decode_rows=16))
    want = eng.prefill(eng.open(), prompt).float().cpu()
    del eng
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    try:
        res = [q.get(timeout=240) for _ in procs]
        [p.join(timeout=60) for p in procs]
        codes = [p.exitcode for p in procs]
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    assert codes == [0] * world, codes
    for rank, lg, rs_expect, status in res:
        assert status[0] == 0, status
        assert rs_expect > 0                                    # the fused path really ran
        scale = float(want.abs().max())
        assert float((lg - want).abs().max()) < 0.03 * max(scale, 1.0), (rank, float((lg - want).abs().max()), scale)
        assert int(lg.argmax()) == int(want.argmax())
    assert all(torch.equal(res[0][1], r[1]) for r in res[1:])    # every rank holds identical logits
