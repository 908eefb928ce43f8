"""Fused compute+collective paths against their NCCL compositions, with roofline fractions.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29521 \
        -m grimoire_b200.bench.fused

Per rank of a W-way group, on the 27B shapes (hidden 5120, FFN 17408, int4 g128 weights):

* **tp_prefill**: the MLP block of a 4096-row prefill chunk under tensor + sequence parallelism:
  all-gather -> column-parallel gate|up GEMM (SwiGLU epilogue) -> row-parallel down GEMM -> reduce-scatter
  -> residual add + RMSNorm on the token shard.  Fused: the down GEMM's epilogue pushes partial tiles to
  the row owners, ``rs_reduce_norm_ag`` reduces / normalises / pushes the rows to every rank and the next
  GEMM's producer waits per m-tile.  Baseline: the same GEMM kernels with NCCL reduce-scatter and
  all-gather between them.
* **tp_decode**: row-parallel down projection of 1 and 8 decode rows + all-reduce: one kernel with the
  all-reduce in its epilogue against GEMV + NCCL all-reduce.
* **ep_moe**: one MoE layer of the hybrid model (512 experts x FFN 512, top-10 + shared, fp8 block weights)
  for 4096 and 1 rows: fused dispatch / grouped GEMM with peer-push / combine against the all-reduce
  composition.

Timing: CUDA events on the launching stream around ``iters`` back-to-back iterations after warm-up, with a
barrier + synchronise on both sides, maximum over ranks.  Roofline of a fused path = the slower of its
FLOPs at the measured dense bf16 GEMM rate and its bytes that must cross NVLink at 770 GB/s per
direction per GPU (measured peer-copy rate); the fraction is roofline time / measured time.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..models.config import hybrid_moe_80b
from ..ops import core as K
from ..ops.linear import gemm_bf16, w4_dequant_into
from ..parallel.tp import TensorParallel
from .kernels import _synthetic_w4, peaks

NVLINK_GBS = 770.0


def _timed(fn, iters: int, dev, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def _timed_graph(fn, iters: int, dev) -> float:
    """ms per call of ``fn`` replayed from a CUDA graph of ``iters`` calls (no host launch cost between the calls; every
    rank replays the same graph at the same time), max over ranks."""
    fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fn()
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.graph(g, stream=side):
            for _ in range(iters):
                fn()
    torch.cuda.synchronize()
    dist.barrier()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


class _Cfg:
    hidden_size = 5120


class _Model:
    cfg = _Cfg()
    tp = None


def bench_tp_prefill(dev, W: int, rank: int, iters: int) -> dict:
    _, tflops, _ = peaks()
    M, H, I = 4096, 5120, 17408
    Il = I // W
    gate_up = _synthetic_w4(2 * Il, H, True, dev)
    down = _synthetic_w4(H, Il, False, dev)
    norm_w = torch.ones(H, device=dev)
    tp = TensorParallel(dist.group.WORLD, dev, fused=True)
    tp.attach(_Model(), max_rows=64)
    tp.sp_setup(M, H)
    R = M // W
    hs = tp.sp_hs[:R]
    hs.normal_()
    act = torch.zeros(M, Il, dtype=torch.bfloat16, device=dev)
    state = {"first": True}

    def fused():
        x_full, agc, age = tp.sp_reduce_norm_allgather(hs, norm_w, 1e-6, 0.0, reduce=not state["first"], M=M)
        state["first"] = False
        tp.sp_gemm_allgathered(gate_up, x_full, agc, age, act, "swiglu")
        tp.sp_gemm_reduce_scatter(down, act, M, H)

    ms_fused = _timed(fused, iters, dev)
    tp.check()
    # NCCL composition with the same GEMM kernels
    x_shard = torch.zeros(R, H, dtype=torch.bfloat16, device=dev)
    x_all = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
    part = torch.zeros(M, H, dtype=torch.bfloat16, device=dev)
    red = torch.zeros(R, H, dtype=torch.bfloat16, device=dev)
    h2 = torch.randn(R, H, device=dev)

    def nccl():
        K.add_rmsnorm(h2, norm_w, x_shard, 1e-6, 0.0, delta=red)
        dist.all_gather_into_tensor(x_all, x_shard)
        gemm_bf16(x_all, w4_dequant_into(gate_up), act, "swiglu")
        gemm_bf16(act, w4_dequant_into(down), part, "bf16")
        dist.reduce_scatter_tensor(red, part)

    ms_nccl = _timed(nccl, iters, dev)
    flops = 2.0 * M * (2 * Il) * H + 2.0 * M * H * Il
    t_compute = flops / (tflops * 1e12) * 1e3
    wire = 2.0 * (W - 1) / W * M * H * 2            # reduce-scatter + all-gather, bf16, per direction per GPU
    t_wire = wire / (NVLINK_GBS * 1e9) * 1e3
    roof = max(t_compute, t_wire)
    return {"path": "tp_prefill_mlp_block", "rows": M, "ms_fused": round(ms_fused, 3), "ms_nccl": round(ms_nccl, 3),
            "roofline_ms": round(roof, 3), "roofline_bound": "compute" if t_compute >= t_wire else "nvlink",
            "fraction_of_roofline": round(roof / ms_fused, 3), "speedup_vs_nccl": round(ms_nccl / ms_fused, 3)}


def bench_tp_decode(dev, W: int, rank: int, iters: int) -> list:
    hbm, _, _ = peaks()
    H, I = 5120, 17408
    Il = I // W
    down = _synthetic_w4(H, Il, False, dev)
    out = []
    for M in (1, 8):
        tp = TensorParallel(dist.group.WORLD, dev, fused=True)
        tp.attach(_Model(), max_rows=64)
        x = torch.randn(M, Il, device=dev).bfloat16()
        h = torch.zeros(M, H, device=dev)
        ms_fused = _timed_graph(lambda: tp.row_parallel_add(down, x, h), max(iters, 20), dev)
        ms_local = _timed_graph(lambda: down(x, h, "add_f32"), max(iters, 20), dev)     # the product alone, no exchange
        tp.check()
        tpn = TensorParallel(dist.group.WORLD, dev, fused=False)
        tpn.attach(_Model(), max_rows=64)
        ms_nccl = _timed(lambda: tpn.row_parallel_add(down, x, h), iters, dev)
        t_mem = down.tiled.nbytes() / (hbm * 1e9) * 1e3
        t_wire = (W - 1) * M * H * 4 / (NVLINK_GBS * 1e9) * 1e3
        roof = max(t_mem, t_wire)
        out.append({"path": "tp_decode_down_allreduce", "rows": M, "us_fused": round(ms_fused * 1e3, 2), "us_product_only": round(ms_local * 1e3, 2),
                    "us_nccl": round(ms_nccl * 1e3, 2), "roofline_us": round(roof * 1e3, 2), "roofline_bound": "hbm" if t_mem >= t_wire else "nvlink",
                    "fraction_of_roofline": round(roof / ms_fused, 3), "speedup_vs_nccl": round(ms_nccl / ms_fused, 3)})
    return out


def bench_ep(dev, W: int, rank: int, iters: int) -> list:
    from ..models.hybrid import HybridBuffers, HybridModel

    _, tflops, _ = peaks()
    hbm = peaks()[0]
    cfg = hybrid_moe_80b(1)
    model = HybridModel.random(cfg, dev, seed=0, max_slots=2, ep_rank=rank, ep_world=W)
    ep = model.attach_ep(dist.group.WORLD, max_rows=4096, fused=True)
    L = model.layers[0]
    H, E, k, I = cfg.hidden_size, cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size
    out = []
    for M in (4096, 1):
        buf = HybridBuffers(model, M, 1)
        x = torch.randn(M, H, device=dev).bfloat16()
        buf.x[:M].copy_(x)
        h = buf.h[:M]

        def run():
            model._moe(L, buf.x[:M], h, buf, M, decode=M <= 8)

        ep.fused = True
        ms_fused = _timed(run, iters, dev)
        ep.check()
        ep.fused = False
        ms_nccl = _timed(run, max(2, iters // 2), dev)
        ep.fused = True
        flops = 2.0 * M * (k + 1) * 3 * H * I / W
        t_compute = flops / (tflops * 1e12) * 1e3
        pairs_remote = M / W * k * (W - 1) / W                     # (row, expert) pairs leaving this rank
        wire = max(pairs_remote * H * 2, pairs_remote * H * 4) + (W - 1) / W * M * H * 4     # dispatch bf16 | return fp32, + row all-gather
        t_wire = wire / (NVLINK_GBS * 1e9) * 1e3
        t_mem = min(E // W, M * k) * 3 * H * I / (hbm * 1e9) * 1e3     # expert weights that must be read at least once
        roof = max(t_compute, t_wire, t_mem)
        bound = "compute" if roof == t_compute else ("nvlink" if roof == t_wire else "hbm")
        out.append({"path": "ep_moe_layer", "rows": M, "ms_fused": round(ms_fused, 3), "ms_allreduce_composition": round(ms_nccl, 3),
                    "roofline_ms": round(roof, 4), "roofline_bound": bound, "fraction_of_roofline": round(roof / ms_fused, 3),
                    "speedup_vs_composition": round(ms_nccl / ms_fused, 3)})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="", help="tp_prefill | tp_decode | ep")
    ns = ap.parse_args(argv)
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        print(json.dumps({"error": "launch with torchrun on 2 or more GPUs"}))
        return 0
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    res = []
    if ns.only in ("", "tp_prefill"):
        res.append(bench_tp_prefill(dev, world, rank, ns.iters))
    if ns.only in ("", "tp_decode"):
        res += bench_tp_decode(dev, world, rank, max(ns.iters, 50))
    if ns.only in ("", "ep"):
        res += bench_ep(dev, world, rank, ns.iters)
    if rank == 0:
        hbm, tf, tag = peaks()
        print(json.dumps({"n_gpus": world, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "nvlink_gbs": NVLINK_GBS, "source": tag},
                          "device_status": list(K.status_read()), "results": res}), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
