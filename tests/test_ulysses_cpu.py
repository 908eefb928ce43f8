"""Head / sequence exchange (parallel/ulysses.py) on CPU ranks (gloo, world 2): every rank holds the whole model and HALF of
the KV heads; prompt chunks are row-split around a head-parallel attention (two all-to-alls per layer), decode rows run
replicated projections and all-gather the attention output.  Logits and generated tokens must equal a single rank's."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.models.dense import DenseModel
from grimoire_b200.models.synthetic import random_state_dict

LIM = dict(max_slots=2, max_ctx=128, prefill_chunk=32, max_decode_rows=8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompt():
    return torch.randint(0, 4096, (71,), generator=torch.Generator().manual_seed(4)).tolist()      # two whole chunks + an odd tail


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from grimoire_b200.parallel.ulysses import UlyssesParallel

        cfg = tiny_dense()
        model = DenseModel.from_state_dict(cfg, random_state_dict(cfg, seed=0), "cpu")
        up = UlyssesParallel(dist.group.WORLD, "cpu")
        up.attach(model)
        eng = Engine(model, EngineLimits(**LIM))
        kv_heads = eng.kv.layers[0].k.shape[1]
        s = eng.open()
        lg = eng.prefill(s, _prompt()).float().clone()
        eng.release(s)
        out = eng.generate(_prompt(), 8)
        q.put((rank, lg, out, dict(up.stats), kv_heads))
    finally:
        dist.destroy_process_group()


def test_ulysses2_prefill_logits_and_tokens_equal_single_rank():
    cfg = tiny_dense()
    eng = Engine(DenseModel.from_state_dict(cfg, random_state_dict(cfg, seed=0), "cpu"), EngineLimits(**LIM))
    s = eng.open()
    want = eng.prefill(s, _prompt()).float().clone()
    eng.release(s)
    single = eng.generate(_prompt(), 8)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, lg, out, stats, kv_heads in res:
        assert kv_heads == cfg.num_key_value_heads // 2                              # the cache holds this rank's heads only
        assert torch.allclose(lg, want, atol=1e-4), (rank, float((lg - want).abs().max()))
        assert out == single
        assert stats["split_chunks"] >= 4 and stats["replicated_passes"] >= 8        # whole chunks split, tail + decode replicated
        assert stats["all_to_all"] == 2 * cfg.num_hidden_layers * stats["split_chunks"]
