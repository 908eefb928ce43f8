"""Context-parallel prompt reading on 2 / 4 / 8 GPUs (skipped on fewer): rows of every chunk split over whole-model
replicas, the chunk's k | v rows pushed to the peers by our copy kernel (and by an all-gather as the baseline); the
last-token logits must match a single-GPU prefill and the status block must stay clean."""
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


def _setup(world):
    from grimoire_b200.models.config import small_dense
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = small_dense(layers=3)
    sd = random_state_dict(cfg, seed=0)
    g = torch.Generator().manual_seed(3)
    chunk = 128 * world          # whole chunks take the balanced two-piece split (64-row pieces), the short tail the plain one
    prompt = torch.randint(0, cfg.vocab_size, (2 * chunk + 5 * world,), generator=g).tolist()
    return cfg, sd, prompt, chunk


def _worker(rank, world, port, q, fused):
    os.environ["GRIMOIRE_CP_BALANCED"] = "1" if world == 2 else "0"      # world 2 takes the balanced two-piece split, the others the default
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from grimoire_b200.engine.engine import Engine, EngineLimits
        from grimoire_b200.models.dense import DenseModel
        from grimoire_b200.ops.core import status_read
        from grimoire_b200.parallel.cp import ContextParallel

        cfg, sd, prompt, chunk = _setup(world)
        model = DenseModel.from_state_dict(cfg, sd, dev)
        cp = ContextParallel(dist.group.WORLD, dev, fused=fused)
        cp.attach(model, max_rows=chunk)
        eng = Engine(model, EngineLimits(max_slots=2, max_ctx=len(prompt) + 64, prefill_chunk=chunk, max_decode_rows=16))
        s = eng.open()
        lg = eng.prefill(s, prompt).float().cpu()
        nxt = eng.decode_rows([int(lg.argmax())], [s], [s.length], use_graph=False)
        torch.cuda.synchronize()
        q.put((rank, lg, nxt, dict(cp.stats), status_read()))
        del eng, model
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fused,world", [(True, 2), (False, 2), (True, 4), (True, 8)])
def test_cp_prefill_matches_single_gpu(fused, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.dense import DenseModel

    cfg, sd, prompt, chunk = _setup(world)
    eng = Engine(DenseModel.from_state_dict(cfg, sd, "cuda:0"), EngineLimits(max_slots=2, max_ctx=len(prompt) + 64, prefill_chunk=chunk,
                                                                            max_decode_rows=16))
    s = eng.open()
    want = eng.prefill(s, prompt).float().cpu()
    nxt0 = eng.decode_rows([int(want.argmax())], [s], [s.length], use_graph=False)
    del eng
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, fused)) for r in range(world)]
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
    scale = max(1.0, float(want.abs().max()))
    for rank, lg, nxt, stats, status in res:
        assert status[0] == 0, status
        assert stats["chunks"] >= 3
        assert float((lg - want).abs().max()) < 0.03 * scale, (rank, float((lg - want).abs().max()), scale)
        assert int(lg.argmax()) == int(want.argmax()) and nxt == nxt0
    assert all(torch.equal(res[0][1], r[1]) for r in res[1:])      # replicas agree bit for bit
