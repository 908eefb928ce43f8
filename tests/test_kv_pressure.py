"""KV page pool under pressure: cached prefix entries give their pages back to a live decode that crosses a page border,
and a request that cannot get a page fails alone (the reference's pooled KV refuses per request, ensure_kv / admit_kv
grimoire.cpp:12036-12070)."""
import pytest
import torch

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.engine.kv import OutOfPages
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.models.dense import DenseModel
from grimoire_b200.sched.scheduler import Scheduler


def _prompt(n, seed):
    return torch.randint(0, 4096, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.fixture()
def engine():
    model = DenseModel.random(tiny_dense(), "cpu", seed=3)
    # 8 pages in total = 128 tokens for everybody
    eng = Engine(model, EngineLimits(max_slots=4, max_ctx=128, prefill_chunk=64, max_decode_rows=8, kv_pages=8))
    eng.enable_prefix_cache()
    return eng


def test_decode_across_a_page_border_evicts_cached_prefixes(engine):
    eng = engine
    # fill the pool with cached conversations: 3 entries x 2 pages
    for seed in (1, 2, 3):
        s = eng.open()
        eng.prefill(s, _prompt(32, seed))
        eng.release(s, cache=True)
    assert eng.kv.pages_free() == 2 and len(eng.prefix_cache.entries) == 3
    s = eng.open()
    lg = eng.prefill(s, _prompt(32, 9))                 # takes the last two free pages
    assert eng.kv.pages_free() == 0
    tok = int(lg.argmax())
    # position 32 starts a new page: only an eviction can provide it
    nxt = eng.decode_rows([tok], [s], [s.length], use_graph=False)
    assert len(nxt) == 1 and len(eng.prefix_cache.entries) == 2 and len(s.pages) == 3
    eng.release(s)


def test_build_step_graph_path_also_reclaims(engine):
    eng = engine
    for seed in (1, 2, 3, 4):
        s = eng.open()
        eng.prefill(s, _prompt(32, seed))
        eng.release(s, cache=True)
    assert eng.kv.pages_free() == 0
    s = eng.open()
    eng.prefix_cache.make_room(1)
    eng.prefill(s, _prompt(10, 11))
    eng.kv.ensure(s, s.length + 40)                     # the step-graph builder maps pages ahead the same way
    assert len(s.pages) == 4 and len(eng.prefix_cache.entries) < 4
    eng.release(s)


def test_only_the_request_that_runs_out_fails(engine):
    eng = engine
    eng.prefix_cache = None
    eng.kv.reclaim = None
    sched = Scheduler(eng, width=4, hold_ms=0.0, hold_long_ms=0.0, use_graph=False)
    import threading

    res = {}

    def run(name, prompt, n):
        try:
            res[name] = sched.generate(prompt, n)[0]
        except Exception as e:  # noqa: BLE001
            res[name] = e

    # a: 60 + 40 tokens = 7 pages; b: 14 + 30 tokens needs 3 pages: together 10 > 8
    ta = threading.Thread(target=run, args=("a", _prompt(60, 5), 40))
    tb = threading.Thread(target=run, args=("b", _prompt(14, 6), 30))
    ta.start(); tb.start(); ta.join(120); tb.join(120)
    sched.shutdown()
    outcomes = [res["a"], res["b"]]
    failed = [o for o in outcomes if isinstance(o, Exception)]
    done = [o for o in outcomes if not isinstance(o, Exception)]
    assert len(failed) == 1 and isinstance(failed[0], OutOfPages), outcomes
    assert len(done) == 1 and len(done[0]) in (30, 40)
    assert eng.kv.pages_used() == 0
