"""Per-rank entry of ``grimoire multi TP|PP|EP|CP``: rank 0 runs the HTTP server and the scheduler over a
``ControlledEngine``; every other rank runs ``worker_loop`` (grimoire_server.cpp:251-264: non
front-end ranks run grimoire_pp_worker_loop)."""
from __future__ import annotations

import argparse
import signal
import sys
import threading

from .. import config as cfgmod


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="grimoire_b200.parallel.launch")
    cfgmod.add_engine_flags(ap)
    ap.add_argument("--mode", choices=["TP", "PP", "EP", "CP", "UP"], default="TP")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--host", default="0.0.0.0")
    ns = ap.parse_args(argv)
    import os

    import torch.distributed as dist

    from ..api import Grimoire
    from .bootstrap import init_parallel
    from .control import ControlChannel, ControlledEngine, worker_loop

    world = int(os.environ.get("WORLD_SIZE", "1"))
    lay = init_parallel(tp_world=world if ns.mode == "TP" else 1, pp_world=world if ns.mode == "PP" else 1,
                        ep_world=world if ns.mode == "EP" else 1, cp_world=world if ns.mode in ("CP", "UP") else 1)
    ec = cfgmod.from_args(ns)
    ec.tp_rank, ec.tp_world, ec.pp_rank, ec.pp_world = lay.tp_rank, lay.tp_world, lay.pp_rank, lay.pp_world
    ec.ep_rank, ec.ep_world = lay.ep_rank, lay.ep_world
    tp = pp = None
    if lay.tp_world > 1:
        from .tp import TensorParallel

        tp = TensorParallel(lay.tp_group, lay.device, fused=bool(ec.tp_fused))
    if lay.pp_world > 1:
        from .pp import PipelineParallel

        pp = PipelineParallel(lay.pp_group, lay.device)
    g = Grimoire.load(ec, device=str(lay.device), tp=tp, pp=pp, ep_group=lay.ep_group,
                      up_group=lay.cp_group if ns.mode == "UP" else None)
    if lay.cp_world > 1 and ns.mode == "CP":
        # whole-model replicas: prompt chunks split by rows, caches replicated, decode steps replicated
        from .cp import ContextParallel

        ContextParallel(lay.cp_group, lay.device).attach(g.model, max_rows=ec.prefill_chunk)
    if (ec.copy_drafts or g.drafter is not None) and getattr(g.model, "supports_verify_rows", True):
        g.engine.enable_speculation()            # on every rank: verify blocks and single rows on the same kernels
    ch = ControlChannel(lay.control_group)
    if not lay.is_front_end:
        served = worker_loop(g.engine, ch)
        print(f"[rank{lay.rank}] worker loop ended after {served} calls", flush=True)
        dist.destroy_process_group()
        return 0
    from ..server import make_server

    g.engine = ControlledEngine(g.engine, ch)
    srv = make_server(g, ec.host, ns.port)

    def stop(signum, frame):
        srv.app.stopping.set()
        threading.Thread(target=srv.shutdown, daemon=True).start()

    signal.signal(signal.SIGTERM, stop)
    signal.signal(signal.SIGINT, stop)
    print(f"[rank0] listening on {ec.host}:{ns.port} ({ns.mode}{world})", flush=True)
    try:
        srv.serve_forever()
    finally:
        g.close()
        g.engine.shutdown()
        srv.server_close()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
