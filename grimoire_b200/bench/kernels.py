"""Per-kernel micro-benchmarks on the 27B projection / attention shapes.

    python -m grimoire_b200.bench.kernels smallm  --rows 1        # int4 small-M (decode GEMV family)
    python -m grimoire_b200.bench.kernels mx      --rows 1        # MXFP4 small-M
    python -m grimoire_b200.bench.kernels gemm    --rows 4096     # tcgen05 GEMM on the prefill shapes
    python -m grimoire_b200.bench.kernels attn    --ctx 4096      # paged int8 decode attention
    python -m grimoire_b200.bench.kernels prefill --rows 4096     # flash prefill attention

Timing: CUDA events around a CUDA-graph replay of the iterations, after warm-up, synchronised on both sides.  Every case
cycles through enough operand copies that the bytes touched between two uses of the same copy
exceed the 126 MB L2, so DRAM figures are cold-cache.  Fractions are quoted against the measured
copy bandwidth / cuBLAS bf16 throughput in MEASURED_PEAKS.json at the repository root when present,
else against 6650 GB/s and 1590 TFLOP/s ("of fallback").  The same commands with a small
``--iters`` are the ones profiled under ncu.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import _native
from ..formats.w4_tile_layout import W4Tiled
from ..ops import core as K
from ..ops.linear import W4Linear, gemm_bf16
from ..ops.workspace import Workspace

L2_BYTES = 126e6
SHAPES = [("qkv", 7168, 5120, False, "bf16"), ("o", 5120, 5120, False, "add_f32"), ("gate_up", 34816, 5120, True, "swiglu"),
          ("down", 5120, 17408, False, "add_f32")]


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "of measured"
    except Exception:
        return 6650.0, 1590.0, "of fallback"


def timed(fn, iters: int, warmup: int = 5) -> float:
    """Mean microseconds per call of ``fn(i)``.  The ``iters`` calls are captured into one CUDA graph and
    the replay is timed, so the figure is device time back to back without host launch gaps (the way
    the engine runs these kernels in its decode graph)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for i in range(iters):
                fn(i)
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / iters


def _synthetic_w4(N: int, K_: int, swiglu: bool, dev) -> W4Linear:
    lin = W4Linear.__new__(W4Linear)
    lin.name = f"mb{N}x{K_}"
    lin.N, lin.K, lin.group, lin.swiglu = N, K_, 128, swiglu
    lin.device, lin.ws, lin.Np, lin.w_ref = torch.device(dev), Workspace(dev), N, None
    w = torch.randint(-2 ** 31, 2 ** 31 - 1, (N // 32, K_ // 64, 2, 32, 4), dtype=torch.int32, device=dev)
    sz = torch.full((N // 16, K_ // 128, 16), (0x4308 << 16) | 0x1C00, dtype=torch.int32, device=dev)   # zero 8, scale 2^-8
    lin.tiled = W4Tiled(w, sz, N, K_, 128)
    lin.out_features = N // 2 if swiglu else N
    return lin


def bench_smallm(args) -> None:
    hbm, _, tag = peaks()
    dev = "cuda"
    for name, N, K_, sw, epi in SHAPES:
        if args.only and name != args.only:
            continue
        one = _synthetic_w4(N, K_, sw, dev)
        copies = max(2, int(L2_BYTES * 2 // one.tiled.nbytes()) + 1)
        lins = [one] + [_synthetic_w4(N, K_, sw, dev) for _ in range(copies - 1)]
        x = torch.randn(args.rows, K_, device=dev).bfloat16()
        out = torch.zeros(args.rows, N // 2 if sw else N, dtype=torch.float32 if epi == "add_f32" else torch.bfloat16, device=dev)
        us = timed(lambda i: lins[i % copies](x, out, epi), args.iters)
        gbs = one.tiled.nbytes() / 1e9 / (us * 1e-6)
        print(f"smallm_w4 {name:8s} M={args.rows:2d} N={N:6d} K={K_:6d} copies={copies:2d}  {us:8.2f} us  {gbs:7.0f} GB/s  "
              f"{gbs / hbm:.3f} {tag} copy bandwidth", flush=True)


def bench_tc(args) -> None:
    """Single-row int4 projections as a tensor-core weight stream (gemv_w4_tc.cu), same shapes and byte count."""
    from ..formats.w4_rowblock import STAGE_BYTES, W4RowBlock

    hbm, _, tag = peaks()
    dev = "cuda"
    for name, N, K_, sw, epi in SHAPES:
        if args.only and name != args.only:
            continue
        nbytes = (N // 128) * (K_ // 128) * STAGE_BYTES
        copies = max(2, int(L2_BYTES * 2 // nbytes) + 1)
        lins = []
        for _ in range(copies):
            lin = _synthetic_w4(32, 64, sw, dev)
            lin.N, lin.K, lin.Np, lin.out_features = N, K_, N, N // 2 if sw else N
            data = torch.randint(0, 256, (N // 128, K_ // 128, STAGE_BYTES), dtype=torch.uint8, device=dev)
            szw = torch.tensor([0x00, 0x1C, 0x08, 0x43], dtype=torch.uint8, device=dev).repeat(128)     # scale 2^-8, zero 8
            data[:, :, 8192:] = szw
            lin.rb = W4RowBlock(data, N, K_, N)
            lins.append(lin)
        x = torch.randn(1, K_, device=dev).bfloat16()
        out = torch.zeros(1, N // 2 if sw else N, dtype=torch.float32 if epi == "add_f32" else torch.bfloat16, device=dev)
        us = timed(lambda i: lins[i % copies]._tc_row(x, None, None, out, epi, 0.0, 0.0), args.iters)
        gbs = nbytes / 1e9 / (us * 1e-6)
        print(f"gemv_w4_tc {name:8s} M= 1 N={N:6d} K={K_:6d} copies={copies:2d}  {us:8.2f} us  {gbs:7.0f} GB/s  "
              f"{gbs / hbm:.3f} {tag} copy bandwidth", flush=True)


def bench_mx(args) -> None:
    """MXFP4 small-M kernel on the same shapes (bytes = packed e2m1 + e8m0 scales)."""
    from ..formats.codecs import Fmt
    from ..formats.quantize import QuantWeight
    from ..ops.linear import MXLinear

    hbm, _, tag = peaks()
    dev = "cuda"
    for name, N, K_, sw, epi in SHAPES:
        if args.only and name != args.only:
            continue
        nbytes = N * K_ // 2 + N * K_ // 32
        copies = max(2, int(L2_BYTES * 2 // nbytes) + 1)
        lins = []
        for _ in range(copies):
            qw = QuantWeight(Fmt.MXFP4, N, K_, torch.randint(0, 256, (N, K_ // 2), dtype=torch.uint8),
                             scales=torch.full((N, K_ // 32), 120, dtype=torch.uint8), group=32)
            lins.append(MXLinear(qw, dev, name, swiglu=sw))
        x = torch.randn(args.rows, K_, device=dev).bfloat16()
        out = torch.zeros(args.rows, N // 2 if sw else N, dtype=torch.float32 if epi == "add_f32" else torch.bfloat16, device=dev)
        us = timed(lambda i: lins[i % copies](x, out, epi), args.iters)
        gbs = nbytes / 1e9 / (us * 1e-6)
        print(f"smallm_mx {name:8s} M={args.rows:2d} N={N:6d} K={K_:6d} copies={copies:2d}  {us:8.2f} us  {gbs:7.0f} GB/s  "
              f"{gbs / hbm:.3f} {tag} copy bandwidth", flush=True)


def bench_rowq(args) -> None:
    """Byte-per-weight small-M kernel (int8 with a scale per row unless --fmt names another format)."""
    from ..formats.codecs import PROJ_NAMES, Fmt
    from ..formats.quantize import QuantWeight
    from ..ops.linear import RowQLinear

    hbm, _, tag = peaks()
    dev = "cuda"
    fmt = PROJ_NAMES[args.fmt]
    for name, N, K_, sw, epi in SHAPES:
        if args.only and name != args.only:
            continue
        width = 2 if fmt == Fmt.BF16 else 1
        nbytes = N * K_ * width + (N * K_ // 32 if fmt == Fmt.MXFP8 else 4 * N)
        copies = max(2, int(L2_BYTES * 2 // nbytes) + 1)
        lins = []
        for _ in range(copies):
            pay = torch.randint(0, 120, (N, K_ * width), dtype=torch.uint8)
            sc = None if fmt == Fmt.BF16 else (torch.full((N, K_ // 32), 120, dtype=torch.uint8) if fmt == Fmt.MXFP8
                                              else torch.full((N,), 1e-3))
            lins.append(RowQLinear(QuantWeight(fmt, N, K_, pay, scales=sc, group=32), dev, name, swiglu=sw))
        x = torch.randn(args.rows, K_, device=dev).bfloat16()
        out = torch.zeros(args.rows, N // 2 if sw else N, dtype=torch.float32 if epi == "add_f32" else torch.bfloat16, device=dev)
        for lin in lins:                          # every copy once outside the capture (resident bf16 forms are made here)
            lin(x, out, epi)
        us = timed(lambda i: lins[i % copies](x, out, epi), args.iters)
        gbs = nbytes / 1e9 / (us * 1e-6)
        print(f"smallm_rowq {args.fmt:8s} {name:8s} M={args.rows:2d} N={N:6d} K={K_:6d} copies={copies:2d}  {us:8.2f} us  {gbs:7.0f} GB/s  "
              f"{gbs / hbm:.3f} {tag} copy bandwidth", flush=True)


def bench_gguf(args) -> None:
    """Projections over raw GGUF blocks (--fmt q4_0 / q8_0 / q4_k / q5_k / q6_k / iq4_nl / iq4_xs) at the 27B shapes."""
    from ..ops.linear import GgufLinear

    hbm, _, tag = peaks()
    dev = "cuda"
    t, bb, bw = {"q4_0": (2, 18, 32), "q8_0": (8, 34, 32), "q4_k": (12, 144, 256), "q5_k": (13, 176, 256), "q6_k": (14, 210, 256),
                 "iq4_nl": (20, 18, 32), "iq4_xs": (23, 136, 256)}[args.fmt]
    for name, N, K_, sw, epi in SHAPES:
        if args.only and name != args.only:
            continue
        row_bytes = K_ // bw * bb
        nbytes = N * row_bytes
        copies = max(2, int(L2_BYTES * 2 // nbytes) + 1)
        lins = []
        for _ in range(copies):
            raw = torch.randint(0, 64, (N, row_bytes), dtype=torch.uint8, device=dev)     # small bytes: fp16 scales stay finite
            parts = [(raw[: N // 2], t), (raw[N // 2:], t)] if sw else [(raw, t)]
            lins.append(GgufLinear(parts, K_, dev, name, swiglu=sw))
        x = torch.randn(args.rows, K_, device=dev).bfloat16()
        out = torch.zeros(args.rows, N // 2 if sw else N, dtype=torch.float32 if epi == "add_f32" else torch.bfloat16, device=dev)
        for lin in lins:
            lin(x, out, epi)
        us = timed(lambda i: lins[i % copies](x, out, epi), args.iters)
        gbs = nbytes / 1e9 / (us * 1e-6)
        print(f"gemv_gguf {args.fmt:7s} {name:8s} M={args.rows:2d} N={N:6d} K={K_:6d} copies={copies:2d}  {us:8.2f} us  {gbs:7.0f} GB/s  "
              f"{gbs / hbm:.3f} {tag} copy bandwidth", flush=True)


def bench_gemm(args) -> None:
    _, tf, tag = peaks()
    dev = "cuda"
    M = args.rows
    for name, N, K_, sw, epi in SHAPES:
        if args.only and name != args.only:
            continue
        nbytes = (M * K_ + N * K_) * 2
        copies = max(2, int(L2_BYTES * 2 // nbytes) + 1)
        A = [torch.randn(M, K_, device=dev).bfloat16() for _ in range(copies)]
        B = [(torch.randn(N, K_, device=dev) * 0.02).bfloat16() for _ in range(copies)]
        out = torch.zeros(M, N // 2 if sw else N, dtype=torch.float32 if epi == "add_f32" else torch.bfloat16, device=dev)
        us = timed(lambda i: gemm_bf16(A[i % copies], B[i % copies], out, epi), args.iters)
        tfl = 2.0 * M * N * K_ / (us * 1e-6) / 1e12
        print(f"gemm_tcgen05 {name:8s} M={M} N={N:6d} K={K_:6d} epi={epi:8s} {us:9.2f} us  {tfl:7.1f} TFLOP/s  "
              f"{tfl / tf:.3f} {tag} cuBLAS bf16 burst", flush=True)


def _paged_kv(ctx: int, slots: int, geom, dev):
    from ..engine.kv import KvPool

    pool = KvPool(1, geom.Hkv, geom.D, slots * ((ctx + 31) // 16) + 1, slots, ctx + 16, dev)
    seqs = [pool.open_slot() for _ in range(slots)]
    for s in seqs:
        pool.ensure(s, ctx + 1)
        s.length = ctx
    lay = pool.layers[0]
    lay.k.random_(-127, 127)
    lay.v.random_(-127, 127)
    lay.ks.fill_(0.01)
    lay.vs.fill_(0.01)
    return pool, seqs


def bench_attn(args) -> None:
    hbm, _, tag = peaks()
    dev = "cuda"
    geom = K.AttnGeom(Hq=40, Hkv=8, D=128, rot=128, scale=128 ** -0.5)
    M = args.rows
    slots = max(M, int(L2_BYTES * 2 // (args.ctx * geom.Hkv * geom.D * 2)) + 1)
    pool, seqs = _paged_kv(args.ctx, slots, geom, dev)
    ws = Workspace(dev)
    q = torch.randn(M, geom.Hq * geom.D, device=dev).bfloat16()
    out = torch.zeros_like(q)
    pos = torch.full((M,), args.ctx - 1, dtype=torch.int32, device=dev)
    row_seq = [torch.tensor([(i * M + r) % slots for r in range(M)], dtype=torch.int32, device=dev) for i in range(slots)]
    splits = args.splits or K.decode_splits(args.ctx, M, geom.Hkv)
    us = timed(lambda i: K.paged_decode_attn(q, row_seq[i % slots], pos, pool.table, pool.layers[0], geom, out, splits, ws), args.iters)
    nbytes = M * args.ctx * geom.Hkv * (geom.D + 4) * 2
    gbs = nbytes / 1e9 / (us * 1e-6)
    print(f"paged_decode_attn rows={M} ctx={args.ctx} splits={splits}  {us:8.2f} us  {gbs:7.0f} GB/s  {gbs / hbm:.3f} {tag} copy bandwidth",
          flush=True)


def bench_vattn(args) -> None:
    """A verify block of ``--rows`` consecutive positions at the end of a ``--ctx``-token context: the one-pass verify
    kernel (attn_verify.cu) against the per-row decode kernel on the same rows, and one row alone."""
    hbm, _, tag = peaks()
    dev = "cuda"
    geom = K.AttnGeom(Hq=40, Hkv=8, D=128, rot=128, scale=128 ** -0.5)
    R = args.rows
    slots = int(L2_BYTES * 2 // (args.ctx * geom.Hkv * geom.D * 2)) + 1
    pool, seqs = _paged_kv(args.ctx, slots, geom, dev)
    ws = Workspace(dev)
    q = torch.randn(R, geom.Hq * geom.D, device=dev).bfloat16()
    out = torch.zeros_like(q)
    pos = torch.arange(args.ctx - R, args.ctx, dtype=torch.int32, device=dev)
    per = K.verify_rows_per_group(geom)
    row_seq, blocks = [], []
    for i in range(slots):
        row_seq.append(torch.full((R,), i, dtype=torch.int32, device=dev))
        groups = K.verify_groups([i] * R, list(range(args.ctx - R, args.ctx)), per)
        blocks.append(torch.tensor(groups, dtype=torch.int32).t().contiguous().to(dev))
    ngroups = blocks[0].shape[1]
    s_rows = K.decode_splits(args.ctx, R, geom.Hkv)
    s_blk = K.decode_splits(args.ctx, ngroups, geom.Hkv)
    s_one = K.decode_splits(args.ctx, 1, geom.Hkv)
    us_rows = timed(lambda i: K.paged_decode_attn(q, row_seq[i % slots], pos, pool.table, pool.layers[0], geom, out, s_rows, ws), args.iters)
    us_blk = timed(lambda i: K.paged_verify_attn(q, blocks[i % slots], ngroups, pool.table, pool.layers[0], geom, out, s_blk, ws), args.iters)
    us_one = timed(lambda i: K.paged_decode_attn(q[:1], row_seq[i % slots][:1], pos[-1:], pool.table, pool.layers[0], geom, out[:1], s_one, ws),
                   args.iters)
    nbytes = args.ctx * geom.Hkv * (geom.D + 4) * 2
    print(f"verify block rows={R} ctx={args.ctx}: one pass per group of {per} rows ({ngroups} groups, splits {s_blk}) {us_blk:8.2f} us "
          f"({ngroups * nbytes / 1e9 / (us_blk * 1e-6):6.0f} GB/s, {ngroups * nbytes / 1e9 / (us_blk * 1e-6) / hbm:.3f} {tag} copy bandwidth) | "
          f"row by row (splits {s_rows}) {us_rows:8.2f} us | one row {us_one:8.2f} us | block / one row = {us_blk / us_one:.2f}", flush=True)


def bench_prefill(args) -> None:
    _, tf, tag = peaks()
    dev = "cuda"
    geom = K.AttnGeom(Hq=40, Hkv=8, D=128, rot=128, scale=128 ** -0.5)
    T = args.rows
    q = torch.randn(T, geom.Hq * geom.D, device=dev).bfloat16()
    k = torch.randn(T, geom.Hkv * geom.D, device=dev).bfloat16()
    v = torch.randn(T, geom.Hkv * geom.D, device=dev).bfloat16()
    out = torch.zeros_like(q)
    us = timed(lambda i: K.flash_prefill(q, k, v, geom, out, 0), args.iters)
    tfl = 4.0 * geom.Hq * geom.D * T * T / 2 / (us * 1e-6) / 1e12        # causal: half the score matrix
    print(f"flash_prefill T={T} Hq=40 Hkv=8 D=128 causal  {us:9.2f} us  {tfl:7.1f} TFLOP/s  {tfl / tf:.3f} {tag} cuBLAS bf16 burst", flush=True)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["smallm", "tc", "mx", "rowq", "gguf", "gemm", "attn", "vattn", "prefill"])
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--splits", type=int, default=0, help="attn: split-KV factor (0 = the engine's heuristic)")
    ap.add_argument("--fmt", default="int8", help="rowq: int8 / bf16 / fp8_e4m3 / fp8_e5m2 / mxfp8; gguf: q4_0 / q8_0 / q4_k / q5_k / q6_k / iq4_nl / iq4_xs")
    ap.add_argument("--only", default="", help="one of qkv / o / gate_up / down")
    args = ap.parse_args(argv)
    {"smallm": bench_smallm, "tc": bench_tc, "mx": bench_mx, "rowq": bench_rowq, "gguf": bench_gguf, "gemm": bench_gemm, "attn": bench_attn, "vattn": bench_vattn, "prefill": bench_prefill}[args.what](args)
    print(f"launches={_native.launch_count}", flush=True)


if __name__ == "__main__":
    main()
