"""Tensor-parallel partitioning on CPU ranks (gloo, world 2): the host-side logic of the split --
head / FFN sharding, per-shard quantisation, the all-reduce call sites -- must reproduce the
single-rank tokens (tier T4 of the reference's strategy: distributed tests without a cluster,
tools/test_parallel_e2e.cpp)."""
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


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _prompt():
    g = torch.Generator().manual_seed(1)
    return torch.randint(0, 4096, (16,), generator=g).tolist()


def _worker(rank, world, port, q, split_head=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from grimoire_b200.parallel.tp import TensorParallel

        cfg = tiny_dense()
        sd = random_state_dict(cfg, seed=0)
        model = DenseModel.from_state_dict(cfg, sd, "cpu", tp_rank=rank, tp_world=world)
        tp = TensorParallel(dist.group.WORLD, "cpu")
        tp.attach(model, max_rows=64)
        extra = None
        if split_head:
            assert tp.split_head(model)
            v0, vn = model.head_split
            assert model.lm_head.N == vn and v0 == rank * vn
        eng = Engine(model, EngineLimits(max_slots=2, max_ctx=128, prefill_chunk=64, max_decode_rows=8))
        out = eng.generate(_prompt(), 12)
        if split_head:
            # whole logits rows on demand: the gathered row equals the single-rank row
            _, trace = eng.generate(_prompt(), 3, collect_logits=True)
            extra = (tp.stats["head_pick"], [t.clone() for t in trace])
        q.put((rank, out, tp.stats["nccl_allreduce"], extra))
    finally:
        dist.destroy_process_group()


def test_tp2_tokens_equal_single_rank():
    cfg = tiny_dense()
    sd = random_state_dict(cfg, seed=0)
    single = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), EngineLimits(max_slots=2, max_ctx=128, prefill_chunk=64,
                                                                            max_decode_rows=8)).generate(_prompt(), 12)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, out, n_ar, _ in res:
        assert out == single, (rank, out, single)
        assert n_ar == 2 * cfg.num_hidden_layers * 12      # 2 per layer per forward (1 prefill + 11 decode steps)


def test_tp2_vocabulary_split_head_picks_the_same_tokens():
    """Every rank keeps half of the lm_head rows; greedy steps exchange (value, index) candidates (tp_head_pick,
    src/grimoire.cpp:5381-5449) and must emit the single-rank tokens; whole logits rows are gathered on demand."""
    cfg = tiny_dense()
    sd = random_state_dict(cfg, seed=0)
    eng1 = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), EngineLimits(max_slots=2, max_ctx=128, prefill_chunk=64, max_decode_rows=8))
    single = eng1.generate(_prompt(), 12)
    _, trace1 = eng1.generate(_prompt(), 3, collect_logits=True)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, True)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, out, _, (picks, trace) in res:
        assert out == single, (rank, out, single)
        assert picks >= 11                                   # the decode steps went through the candidate exchange
        for a, b in zip(trace, trace1):
            assert torch.allclose(a, b, atol=1e-4), rank


def test_head_pick_rule_ties_and_empty_rows():
    """One process, world 1 emulation of the rule: highest value, lowest index on a tie, INT_MAX when a row has no
    finite candidate."""
    from grimoire_b200.parallel.tp import pick_candidates

    vals = torch.tensor([[1.0, 3.0, 3.0], [float("-inf")] * 3, [2.0, 2.0, 1.0]])
    idx = torch.tensor([[7, 9, 4], [0x7fffffff] * 3, [5, 3, 1]])
    assert pick_candidates(vals, idx).tolist() == [4, 0x7fffffff, 3]


def test_tp_rejects_indivisible_heads():
    cfg = tiny_dense()
    with pytest.raises(ValueError):
        DenseModel(cfg, "cpu", tp_rank=0, tp_world=3)
