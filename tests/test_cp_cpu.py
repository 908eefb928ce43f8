"""Context-parallel prompt reading on CPU ranks (gloo, world 2): every rank runs half of each chunk's rows, the ranks
exchange the chunk's k | v rows per layer and keep replicated caches; logits and the following decode steps must equal a
single rank's (parallel/cp.py; the reference has no multi-rank long-prompt path)."""
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

LIM = dict(max_slots=2, max_ctx=128, prefill_chunk=32, max_decode_rows=8)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompt():
    g = torch.Generator().manual_seed(4)
    return torch.randint(0, 4096, (70,), generator=g).tolist()


def _worker(rank, world, port, q, balanced):
    os.environ["GRIMOIRE_CP_BALANCED"] = "1" if balanced else "0"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from grimoire_b200.parallel.cp import ContextParallel

        cfg = tiny_dense()
        model = DenseModel.from_state_dict(cfg, random_state_dict(cfg, seed=0), "cpu")
        cp = ContextParallel(dist.group.WORLD, "cpu")
        cp.attach(model, max_rows=32)
        eng = Engine(model, EngineLimits(**LIM))
        s = eng.open()
        lg = eng.prefill(s, _prompt()).float().clone()
        eng.release(s)
        out = eng.generate(_prompt(), 8)
        q.put((rank, lg, out, dict(cp.stats), cp.layout(32)[1] is not None))
    finally:
        dist.destroy_process_group()


def test_balanced_layout_gives_every_rank_the_same_causal_work():
    from grimoire_b200.parallel.cp import ContextParallel

    M, W = 4096, 8
    work, seen = [], []
    for r in range(W):
        cp = ContextParallel.__new__(ContextParallel)
        cp.world, cp.rank, cp.balanced, cp._layouts, cp.device = W, r, True, {}, torch.device("cpu")
        segs, perm = cp.layout(M)
        a, b = cp.local_rows(M)
        assert [int(x) for x in perm[a:b]] == [g0 + i for g0, n in segs for i in range(n)]
        work.append(sum((g0 + i + 1) for g0, n in segs for i in range(n)))          # keys seen by the rank's query rows
        seen += perm[a:b].tolist()
        rows = torch.tensor([g0 for g0, _ in segs] + [segs[1][0] + 5])
        owner, local = cp.owner_index(rows, M)
        assert owner.tolist() == [r, r, r] and local.tolist() == [0, segs[0][1], segs[0][1] + 5]
    assert sorted(seen) == list(range(M))
    assert max(work) - min(work) <= 0.001 * max(work)


@pytest.mark.parametrize("balanced", [True, False])
def test_cp2_prefill_logits_and_tokens_equal_single_rank(balanced):
    cfg = tiny_dense()
    eng = Engine(DenseModel.from_state_dict(cfg, random_state_dict(cfg, seed=0), "cpu"), EngineLimits(**LIM))
    s = eng.open()
    want = eng.prefill(s, _prompt()).float().clone()
    eng.release(s)
    single = eng.generate(_prompt(), 8)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, balanced)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, lg, out, stats, used in res:
        assert used == balanced
        assert torch.allclose(lg, want, atol=1e-4), (rank, float((lg - want).abs().max()))
        assert out == single
        assert stats["chunks"] >= 3 and stats["exchanges"] == stats["chunks"] * cfg.num_hidden_layers
