"""Scheduler: policy core (C++) and the engine-driving thread, on CPU.  Identity claims follow the
reference's device gates (tools/test_scheduler.cpp, test_batch_decode.cpp): concurrent == alone,
prompts of different lengths, cancellation frees the slot."""
import ctypes
import threading

import pytest
import torch

from grimoire_b200 import _native
from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.models.dense import DenseModel
from grimoire_b200.models.synthetic import random_state_dict
from grimoire_b200.sched.scheduler import PLAN_ADMIT, PLAN_STEP, PLAN_WAIT, Scheduler, _Plan


def _core(width=4, hold=8.0, hold_long=100.0, depths=(3, 2), interleave=64, chunk=256):
    lib = _native.host()
    lib.grm_sched_new.restype = ctypes.c_void_p
    d = (ctypes.c_int * len(depths))(*depths)
    h = ctypes.c_void_p(lib.grm_sched_new(width, 4096, interleave, chunk, 32768, 1000, ctypes.c_double(hold),
                                          ctypes.c_double(hold_long), d, len(depths), 32))
    return lib, h


def _plan(lib, h, now):
    p = _Plan()
    lib.grm_sched_plan(h, ctypes.c_double(now), ctypes.byref(p))
    return p


def test_core_hold_then_batched_admission_then_interleave():
    lib, h = _core()
    assert lib.grm_sched_submit(h, ctypes.c_int64(1), 100, 10, 0, ctypes.c_double(0.0)) == 0
    p = _plan(lib, h, 1.0)
    assert p.kind == PLAN_WAIT and 6.9 < p.wait_ms <= 7.0          # waits for a burst
    lib.grm_sched_submit(h, ctypes.c_int64(2), 300, 10, 0, ctypes.c_double(2.0))
    p = _plan(lib, h, 11.0)                                         # hold expired: both admitted together
    assert p.kind == PLAN_ADMIT and p.n_admit == 2
    assert (p.admit_from[0], p.admit_to[0]) == (0, 100) and (p.admit_from[1], p.admit_to[1]) == (0, 256)
    lib.grm_sched_on_prefilled(h, ctypes.c_int64(1), 100)
    lib.grm_sched_on_prefilled(h, ctypes.c_int64(2), 256)
    p = _plan(lib, h, 12.0)
    # job 1 decodes; job 2's remaining 44 prompt tokens are read between steps in interleave chunks
    assert p.kind == (PLAN_ADMIT | PLAN_STEP) and p.n_live == 1 and p.live_job[0] == 1
    assert (p.admit_from[0], p.admit_to[0]) == (256, 300) and p.draft_depth == 3
    lib.grm_sched_on_prefilled(h, ctypes.c_int64(2), 300)
    p = _plan(lib, h, 13.0)
    assert p.kind == PLAN_STEP and p.n_live == 2 and p.draft_depth == 2     # depth table by live count
    # long prompts use the long hold; an over-long prompt is refused
    assert lib.grm_sched_submit(h, ctypes.c_int64(3), 5000, 10, 0, ctypes.c_double(13.0)) == -1
    lib.grm_sched_delete(h)


def test_core_cancel_and_retire_free_slots():
    lib, h = _core(width=1, hold=0.0)
    lib.grm_sched_submit(h, ctypes.c_int64(1), 10, 2, 0, ctypes.c_double(0.0))
    lib.grm_sched_submit(h, ctypes.c_int64(2), 10, 2, 0, ctypes.c_double(0.0))
    p = _plan(lib, h, 1.0)
    assert p.n_admit == 1 and p.admit_job[0] == 1                 # one slot: job 2 queues
    lib.grm_sched_on_prefilled(h, ctypes.c_int64(1), 10)
    lib.grm_sched_on_tokens(h, ctypes.c_int64(1), 2, 0)          # budget exhausted -> DONE
    lib.grm_sched_cancel(h, ctypes.c_int64(2))
    p = _plan(lib, h, 2.0)
    retired = sorted((p.retired_job[i], p.retired_slot[i]) for i in range(p.n_retired))
    assert retired == [(1, 0), (2, -1)] and p.kind == 0
    lib.grm_sched_delete(h)


@pytest.fixture(scope="module")
def engine():
    cfg = tiny_dense()
    sd = random_state_dict(cfg, seed=3)
    return Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), EngineLimits(max_slots=4, max_ctx=256, prefill_chunk=64, max_decode_rows=16))


def _prompt(n, seed):
    return torch.randint(0, 4096, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _prompts():
    g = torch.Generator().manual_seed(7)
    return [torch.randint(0, 4096, (n,), generator=g).tolist() for n in (5, 23, 70)]


def test_concurrent_requests_equal_alone(engine):
    prompts = _prompts()
    alone = [engine.generate(p, 10) for p in prompts]
    s = Scheduler(engine, width=3, interleave_chunk=32, prefill_chunk=64, hold_ms=20.0)
    res = [None] * 3
    def work(i):
        res[i] = s.generate(prompts[i], 10)
    ts = [threading.Thread(target=work, args=(i,)) for i in range(3)]
    [t.start() for t in ts]
    [t.join(timeout=120) for t in ts]
    s.shutdown()
    for i in range(3):
        out, why, job = res[i]
        assert out == alone[i], (i, out, alone[i])
        assert why == "length"
    assert s.metrics["steps"] > 0 and s.metrics["rows"] > s.metrics["steps"]     # batched rows really ran
    assert engine.kv.pages_used() == 0


def test_cancel_releases_slot_and_copy_drafts_keep_tokens(engine):
    prompts = _prompts()
    s = Scheduler(engine, width=2, hold_ms=0.0, depths=(4, 2), copy_drafts=True)
    seen = []
    out, why, _ = s.generate(prompts[1], 50, on_token=lambda t: (seen.append(t), len(seen) < 4)[1])
    assert why == "cancelled" and len(out) == 4
    # repetitive prompt: copy drafts fire, tokens still equal plain greedy
    rep = (prompts[0] * 6)[:40]
    plain = engine.generate(rep, 12)
    out2, why2, job = s.generate(rep, 12)
    s.shutdown()
    assert out2 == plain and why2 == "length"
    assert engine.kv.pages_used() == 0


def test_overlong_prompt_is_a_value_error(engine):
    s = Scheduler(engine, width=1, hold_ms=0.0)
    with pytest.raises(ValueError):
        s.generate(list(range(300)), 4)
    s.shutdown()


def test_short_prompts_admitted_together_run_one_pass(engine):
    """Prompts that arrive together share ONE M-row prefill (admit_batch, grimoire.cpp:12071) and still produce the
    tokens they produce alone."""
    import threading

    prompts = [_prompt(n, seed) for n, seed in ((9, 31), (17, 32), (5, 33))]
    alone = [engine.generate(p, 6) for p in prompts]
    sched = Scheduler(engine, width=4, hold_ms=200.0, hold_long_ms=400.0, use_graph=False)
    res = [None] * len(prompts)

    def run(i):
        res[i] = sched.generate(prompts[i], 6)[0]

    ts = [threading.Thread(target=run, args=(i,)) for i in range(len(prompts))]
    [t.start() for t in ts]
    [t.join(120) for t in ts]
    batches = sched.metrics.get("admit_batches", 0)
    sched.shutdown()
    assert res == alone
    assert batches >= 1 and engine.counters.get("prefill_batches", 0) >= 1


def test_prefill_batch_logits_equal_single_prefill(engine):
    import torch

    prompts = [_prompt(12, 41), _prompt(7, 42)]
    single = []
    for p in prompts:
        s = engine.open()
        single.append(engine.prefill(s, p).clone())
        engine.release(s)
    seqs = [engine.open(), engine.open()]
    got = engine.prefill_batch(seqs, prompts)
    for a, b in zip(single, got):
        assert int(a.argmax()) == int(b.argmax()) and torch.allclose(a, b, atol=5e-3)
    nxt = engine.decode_rows([int(g.argmax()) for g in got], seqs, [s.length for s in seqs], use_graph=False)
    assert len(nxt) == 2
    [engine.release(s) for s in seqs]
