"""Process-group layout for TP x PP (x DP) on one node: one process per GPU under torchrun.

rank = (dp * pp_world + pp) * tp_world + tp.  TP groups share a pipeline stage, PP groups share a
TP index, and a gloo group over the same ranks carries the control protocol (CPU only).  The
reference wires ranks by environment variables and Unix sockets (docker-entrypoint.sh:32-119,
pp_connect grimoire.cpp:4501-4614); the layout and the "start every rank, front end on rank 0"
contract are the same.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class ParallelLayout:
    rank: int
    world: int
    tp_rank: int
    tp_world: int
    pp_rank: int
    pp_world: int
    tp_group: Optional[object] = None
    pp_group: Optional[object] = None
    ep_rank: int = 0
    ep_world: int = 1
    ep_group: Optional[object] = None
    cp_world: int = 1
    cp_group: Optional[object] = None
    control_group: Optional[object] = None
    device: Optional[torch.device] = None

    @property
    def is_front_end(self) -> bool:
        return self.rank == 0


def init_parallel(tp_world: int = 1, pp_world: int = 1, backend: Optional[str] = None, ep_world: int = 1, cp_world: int = 1) -> ParallelLayout:
    """``ep_world`` > 1 (expert parallelism of the hybrid MoE family) uses every rank as one expert shard; ``cp_world`` > 1
    (context parallelism: prompt chunks split by rows) uses every rank as a whole-model replica.  Neither combines with
    tensor or pipeline stages."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if ep_world > 1 and (tp_world != 1 or pp_world != 1 or ep_world != world):
        raise ValueError(f"expert parallel {ep_world} must span the whole world ({world}) without tp / pp")
    if cp_world > 1 and (tp_world != 1 or pp_world != 1 or ep_world != 1 or cp_world != world):
        raise ValueError(f"context parallel {cp_world} must span the whole world ({world}) without tp / pp / ep")
    if ep_world == 1 and cp_world == 1 and tp_world * pp_world != world:
        raise ValueError(f"tp {tp_world} x pp {pp_world} != world size {world}")
    cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if cuda else "gloo")
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if not dist.is_initialized():
        if backend == "nccl":
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group(backend)
    tp_rank, pp_rank = (rank % tp_world, rank // tp_world) if ep_world == 1 and cp_world == 1 else (0, 0)
    lay = ParallelLayout(rank, world, tp_rank, tp_world, pp_rank, pp_world, device=dev)
    # every rank must create every group, in the same order
    for p in range(pp_world):
        ranks = [p * tp_world + t for t in range(tp_world)]
        g = dist.new_group(ranks) if tp_world > 1 else None
        if p == pp_rank:
            lay.tp_group = g
    for t in range(tp_world):
        ranks = [p * tp_world + t for p in range(pp_world)]
        g = dist.new_group(ranks) if pp_world > 1 else None
        if t == tp_rank:
            lay.pp_group = g
    if ep_world > 1:
        lay.ep_rank, lay.ep_world, lay.ep_group = rank, ep_world, dist.new_group(list(range(world)))
    if cp_world > 1:
        lay.cp_world, lay.cp_group = cp_world, dist.new_group(list(range(world)))
    lay.control_group = dist.new_group(list(range(world)), backend="gloo") if world > 1 else None
    return lay
