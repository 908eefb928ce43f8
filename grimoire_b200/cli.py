"""Command line: ``generate`` (default), ``serve``, ``multi TP|PP|EP|CP|DP``, ``quantize``, ``inspect``.

Flags of the single-prompt CLI follow tools/grimoire_main.cpp:66-167 (``-m --proj --ctx -p -n
--prefill-only --prefix-cache-test --score-ids/--score-out --ppl ...``); no ``-p`` prints the load
report and the micro-benchmarks.  ``multi`` is the launcher of docker-entrypoint.sh:32-119: one
server process per GPU with the rank variables set, started back to front, TERM forwarded.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time

from . import config as cfgmod


def _generate(argv) -> int:
    ap = argparse.ArgumentParser(prog="grimoire")
    cfgmod.add_engine_flags(ap)
    ap.add_argument("-p", "--prompt", default=None)
    ap.add_argument("-n", type=int, default=128, dest="n_tokens")
    ap.add_argument("--prefill-only", type=int, default=0, metavar="N")
    ap.add_argument("--prefix-cache-test", type=int, default=0, metavar="N")
    ap.add_argument("--score-ids", default="", help="file with space separated token ids")
    ap.add_argument("--score-out", default="", help="where the fp32 logits go (torch .pt)")
    ap.add_argument("--ppl", default="", metavar="FILE")
    ap.add_argument("--ppl-ctx", type=int, default=512)
    ap.add_argument("--ppl-chunks", type=int, default=0)
    ap.add_argument("--ppl-kld-base", default="", help="a llama-perplexity --kl-divergence-base file, or baseline logits (.pt)")
    ap.add_argument("--ppl-dump", default="", metavar="FILE", help="per-token TSV: target and best log-probabilities, eight candidates")
    ap.add_argument("--ppl-selfcheck", action="store_true", help="compare the last scored decode logits with a batched prefill")
    ap.add_argument("--spec-depth", type=int, default=0)
    ns = ap.parse_args(argv)
    if not ns.model:
        ap.error("-m/--model is required (a HF directory, or synthetic:<preset>)")
    ec = cfgmod.from_args(ns)
    from .api import Grimoire

    g = Grimoire.load(ec)
    tok = g.tokenizer
    try:
        if ns.score_ids:
            import torch

            ids = [int(t) for t in open(ns.score_ids).read().split()]
            lg = g.score_ids(ids)
            if ns.score_out:
                torch.save(lg, ns.score_out)
            print(json.dumps({"positions": len(ids), "argmax": lg.argmax(-1).tolist()[:16]}))
            return 0
        if ns.ppl:
            text = open(ns.ppl).read()
            ids = tok.with_bos(tok.encode(text)) if tok else [int(t) for t in text.split()]      # BOS first when the tokenizer asks for it
            llama_base = bool(ns.ppl_kld_base) and open(ns.ppl_kld_base, "rb").read(8) == b"_logits_"
            res = g.perplexity(ids, ns.ppl_ctx, ns.ppl_chunks, dump=ns.ppl_dump, selfcheck=ns.ppl_selfcheck,
                               kld_base=ns.ppl_kld_base if llama_base else "")
            if ns.ppl_kld_base and not llama_base:
                # a torch file of baseline logits (--score-out of another run): distances over the first window
                import torch

                from .utils.kld import kld_stats

                res["kld"] = kld_stats(torch.load(ns.ppl_kld_base), g.score_ids(ids[: ns.ppl_ctx]))
            report = res.pop("kld_report", "")
            print(json.dumps(res))
            if report:
                print(report)
            return 0
        if ns.prefill_only:
            print(json.dumps({"pp": ns.prefill_only, "tok_s": round(g.bench_prefill(ns.prefill_only), 1)}))
            return 0
        if ns.prefix_cache_test:
            import torch

            ids = torch.randint(0, g.model.cfg.vocab_size, (ns.prefix_cache_test,), generator=torch.Generator().manual_seed(0)).tolist()
            times = []
            for _ in range(2):
                s = g.engine.open()
                t0 = time.perf_counter()
                n = g.engine.prefix_reuse(s, ids)
                g.engine.prefill(s, ids[n:])
                times.append(time.perf_counter() - t0)
                g.engine.release(s, cache=True)
            print(json.dumps({"tokens": len(ids), "first_s": round(times[0], 4), "repeat_s": round(times[1], 4)}))
            return 0
        if ns.prompt is None:
            rep = {"weights_gb": round(g.model.weight_bytes() / 1e9, 3), "kv_pages": g.engine.kv.num_pages}
            rep["pp512_tok_s"] = round(g.bench_prefill(min(512, ec.ctx - 16)), 1)
            rep["tg64_tok_s"] = round(g.bench_decode(64, min(128, ec.ctx // 2)), 1)
            print(json.dumps(rep))
            return 0
        ids = tok.encode_chat([{"role": "user", "content": ns.prompt}]) if tok else [int(t) for t in ns.prompt.split()]
        from .engine.generation import SpecStats

        st = SpecStats()
        t0 = time.perf_counter()
        pieces = []

        def emit(t):
            if tok:
                sys.stdout.write(tok.decode([t]))
                sys.stdout.flush()
            else:
                pieces.append(t)
            return True

        out, why = g.generate(ids, ns.n_tokens, tok.eos() if tok else None, tok.eos2() if tok else None, emit, ns.spec_depth, st)
        dt = time.perf_counter() - t0
        if not tok:
            print(" ".join(str(t) for t in pieces))
        print(f"\n[{len(out)} tokens, {len(out) / dt:.1f} tok/s incl. prompt, finish={why}]", file=sys.stderr)
        if ec.spec_stats and st.rounds:
            print(st.line(), file=sys.stderr)
        return 0
    finally:
        g.close()


def _multi(argv) -> int:
    ap = argparse.ArgumentParser(prog="grimoire multi")
    ap.add_argument("mode", choices=["TP", "PP", "EP", "CP", "UP", "DP", "tp", "pp", "ep", "cp", "up", "dp"])
    ap.add_argument("--gpus", type=int, default=0, help="ranks to start (default: all visible GPUs)")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--master-port", type=int, default=29555)
    ns, rest = ap.parse_known_args(argv)
    import torch

    n = ns.gpus or max(1, torch.cuda.device_count())
    mode = ns.mode.upper()
    if mode == "DP":
        from .parallel.dp import run_replicas

        return run_replicas(n, ns.port, rest)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(ns.master_port), "-m", "grimoire_b200.parallel.launch", "--mode", mode, "--port", str(ns.port), *rest]
    proc = subprocess.Popen(cmd)
    for sig in (signal.SIGTERM, signal.SIGINT):
        signal.signal(sig, lambda s, f: proc.send_signal(signal.SIGTERM))
    return proc.wait()


def _quantize(argv) -> int:
    from .formats.artifact import quantize_cli

    return quantize_cli(argv)


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "serve":
        from .server import serve

        return serve(argv[1:])
    if argv and argv[0] == "multi":
        return _multi(argv[1:])
    if argv and argv[0] == "quantize":
        return _quantize(argv[1:])
    if argv and argv[0] == "inspect":
        from .formats.artifact import inspect_cli

        return inspect_cli(argv[1:])
    if argv and argv[0] == "generate":
        argv = argv[1:]
    return _generate(argv)


if __name__ == "__main__":
    sys.exit(main())
