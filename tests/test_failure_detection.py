"""Failure detection without faulting a GPU: failures are made on the host (a rank that raises, a
rank that never joins, a corrupted control header, a silent heartbeat); on the GPU the only failure
exercised is a bounded device-side wait running out on a flag nothing sets."""
import ctypes
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from grimoire_b200.parallel import control as C
from grimoire_b200.parallel.health import Heartbeat, RankLost


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class _FakeKv:
    def __init__(self):
        self.slots = {}


class _FailingEngine:
    """Engine stand-in whose prefill raises (a worker-side fault made on the host)."""

    def __init__(self):
        self.kv = _FakeKv()

    def open(self, slot=None):
        self.kv.slots[slot] = object()

    def prefill(self, seq, tokens, want_logits=True):
        raise RuntimeError("injected worker failure")


def _rank_raises(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    ch = C.ControlChannel(dist.group.WORLD)
    if rank == 0:
        try:
            ch.send(C.OPEN, 0)
            ch.send(C.PREFILL, 0, 0, [1, 2, 3])
            # the worker is gone now: a later message must fail within the group timeout, not hang
            for _ in range(4):
                ch.send(C.STEP, 1, 0, [5, 0, 3])
            q.put(("root", "no error"))
        except C.WorkerLost as e:
            q.put(("root", "WorkerLost"))
    else:
        try:
            C.worker_loop(_FailingEngine(), ch)
            q.put(("worker", "returned"))
        except RuntimeError as e:
            q.put(("worker", str(e)))
    # no destroy_process_group: the peer is gone and a collective teardown could block
    q.close(); q.join_thread()
    os._exit(0)


def test_worker_exception_unblocks_root_with_worker_lost():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_raises, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        got = dict(q.get(timeout=90) for _ in procs)
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.kill()
    assert got["worker"] == "injected worker failure"
    assert got["root"] == "WorkerLost"


def _rank_alone(port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        q.put("joined")
    except Exception as e:          # the rendezvous gives up: the launcher reports it instead of hanging
        q.put(type(e).__name__)
    q.close(); q.join_thread()
    os._exit(0)


def test_rank_that_never_joins_times_out():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_rank_alone, args=(_free_port(), q))
    p.start()
    try:
        res = q.get(timeout=90)
    finally:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    assert res != "joined"


def test_corrupted_header_is_rejected_before_allocation(monkeypatch):
    ch = C.ControlChannel.__new__(C.ControlChannel)
    ch.group, ch.src, ch.rank, ch.is_root = None, 0, 1, False
    for bad in ([99, 0, 0, 0], [C.STEP, 1, 0, C.MAX_PAYLOAD + 1], [C.STEP, 1, 0, -4]):
        def fake_broadcast(t, src=0, group=None, _bad=bad):
            assert t.numel() == C.HEADER, "payload buffer allocated from an unvalidated length"
            t.copy_(torch.tensor(_bad, dtype=torch.int64))
        monkeypatch.setattr(dist, "broadcast", fake_broadcast)
        with pytest.raises(C.WorkerLost):
            ch.recv()

    def closed(t, src=0, group=None):
        raise RuntimeError("Connection closed by peer")
    monkeypatch.setattr(dist, "broadcast", closed)
    with pytest.raises(C.WorkerLost):
        ch.recv()
    with pytest.raises(C.WorkerLost):
        ch.send(C.STEP, 1, 0, [1, 2, 3])


def test_heartbeat_flags_a_silent_rank():
    store = dist.HashStore()
    now = [0.0]
    a = Heartbeat(store, 0, 3, stale_after=2.0, clock=lambda: now[0])
    b = Heartbeat(store, 1, 3, stale_after=2.0, clock=lambda: now[0])
    c = Heartbeat(store, 2, 3, stale_after=2.0, clock=lambda: now[0])
    assert a.stale() == []
    for t in (1.0, 2.0, 3.0, 4.0):
        now[0] = t
        b.beat()                     # rank 1 keeps beating, rank 2 went silent after its first beat
        dead = a.stale()
    assert dead == [2]
    with pytest.raises(RankLost) as ei:
        a.check()
    assert ei.value.ranks == [2]
    c.beat()                         # it comes back: no longer stale
    assert a.stale() == []


def test_heartbeat_thread_beats():
    store = dist.HashStore()
    hb = Heartbeat(store, 0, 1, interval=0.02).start()
    import time
    v0 = int(store.get("grm/hb/0"))
    time.sleep(0.2)
    hb.stop()
    assert int(store.get("grm/hb/0")) > v0


@pytest.mark.gpu
def test_bounded_device_wait_reports_timeout_and_context_survives():
    """ep_plan waits for per-source dispatch flags; nothing sets them here, so the wait runs out after
    a short limit, the kernel records GRM_ERR_FLAG_TIMEOUT, publishes zero tiles and returns."""
    from grimoire_b200 import _native
    from grimoire_b200.ops.core import status_read

    dev = torch.device("cuda")
    status_read(clear=True)
    W, E_loc, max_tiles = 2, 4, 64
    z = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
    flags, groups, state = z(8), z(W * E_loc * 2), z(16)
    te, r0, nr, src, nt = z(max_tiles), z(max_tiles), z(max_tiles), z(max_tiles), torch.full((1,), 7, dtype=torch.int32, device=dev)
    code = _native.cuda().grm_ep_plan(_native.ptr(flags), _native.ptr(groups), _native.ptr(te), _native.ptr(r0), _native.ptr(nr),
                                      _native.ptr(src), _native.ptr(nt), _native.ptr(state), ctypes.c_int(E_loc), ctypes.c_int(W),
                                      ctypes.c_int(max_tiles), ctypes.c_uint(2000), _native.stream_ptr())
    assert code == 0
    torch.cuda.synchronize()
    st = status_read(clear=True)
    assert st[0] == 2 and (st[1] >> 16) == 0x5          # FLAG_TIMEOUT raised by the plan kernel
    assert int(nt) == 0
    # the context is still usable and the status block is clean again
    x = torch.arange(8, device=dev).float()
    assert float((x * 2).sum()) == 56.0
    assert status_read()[0] == 0
