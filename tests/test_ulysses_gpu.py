"""Head / sequence exchange on 2 GPUs (skipped on fewer): whole-model replicas with half of the KV heads each, NCCL
all-to-alls around a head-parallel attention for prompt chunks, an all-gather of the attention output for decode rows; the
last-token logits and the next decode step must match a single-GPU engine and the status block must stay clean."""
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


def _setup():
    from grimoire_b200.models.config import small_dense
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = small_dense(layers=3)
    sd = random_state_dict(cfg, seed=0)
    prompt = torch.randint(0, cfg.vocab_size, (2 * 128 + 11,), generator=torch.Generator().manual_seed(3)).tolist()
    return cfg, sd, prompt


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from grimoire_b200.engine.engine import Engine, EngineLimits
        from grimoire_b200.models.dense import DenseModel
        from grimoire_b200.ops.core import status_read
        from grimoire_b200.parallel.ulysses import UlyssesParallel

        cfg, sd, prompt = _setup()
        model = DenseModel.from_state_dict(cfg, sd, dev)
        up = UlyssesParallel(dist.group.WORLD, dev)
        up.attach(model)
        eng = Engine(model, EngineLimits(max_slots=2, max_ctx=len(prompt) + 64, prefill_chunk=128, max_decode_rows=16))
        s = eng.open()
        lg = eng.prefill(s, prompt).float().cpu()
        nxt = eng.decode_rows([int(lg.argmax())], [s], [s.length], use_graph=False)
        torch.cuda.synchronize()
        q.put((rank, lg, nxt, dict(up.stats), status_read()))
        del eng, model
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


def test_ulysses2_prefill_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.dense import DenseModel

    cfg, sd, prompt = _setup()
    eng = Engine(DenseModel.from_state_dict(cfg, sd, "cuda:0"), EngineLimits(max_slots=2, max_ctx=len(prompt) + 64, prefill_chunk=128,
                                                                            max_decode_rows=16))
    s = eng.open()
    want = eng.prefill(s, prompt).float().cpu()
    nxt0 = eng.decode_rows([int(want.argmax())], [s], [s.length], use_graph=False)
    del eng
    torch.cuda.empty_cache()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    scale = max(1.0, float(want.abs().max()))
    for rank, lg, nxt, stats, status in res:
        assert float((lg - want).abs().max()) < 0.03 * scale, (rank, float((lg - want).abs().max()))
        assert int(lg.argmax()) == int(want.argmax()) and list(nxt) == list(nxt0)
        assert stats["split_chunks"] == 2 and stats["all_to_all"] == 2 * 3 * 2 and status[0] == 0
