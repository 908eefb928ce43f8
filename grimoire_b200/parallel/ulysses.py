"""Ulysses-style head / sequence exchange for attention over whole-model replicas.

Every rank holds the whole model but only ``Hkv / R`` KV heads of the cache (``R`` times the context fits in the same
memory; the replicated-cache context parallelism of parallel/cp.py trades that for no exchange in decode).  Attention always
runs head-parallel: rank r owns q heads [r Hq/R, (r+1) Hq/R) and their KV heads.

* prompt chunk of M rows, M divisible by R: rank r projects rows [r M/R, (r+1) M/R) only; one all-to-all turns
  "my rows x all heads" into "all rows x my heads" (q | k | v packed per destination), attention runs over the chunk and the
  cached past of the local heads, a second all-to-all brings "my rows x all heads" of the attention output back; o_proj and
  the MLP run on the local rows -- 1/R of the projection FLOPs and 1/R of the attention per rank, two exchanges per layer;
* decode rows (and chunks that do not divide): every rank runs the projections of all rows (replicated), attends with its
  own heads, and an all-gather assembles the attention output.

The exchanges are ``torch.distributed`` collectives (NCCL all-to-all over NVSwitch on GPUs, gloo on CPU ranks); there is no
fused kernel form.  The reference has no counterpart (its long prompts are single-rank, include/b70/generation.hpp:202-213).
"""
from __future__ import annotations

import dataclasses

import torch
import torch.distributed as dist


class UlyssesParallel:
    def __init__(self, group, device):
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.stats = {"split_chunks": 0, "replicated_passes": 0, "all_to_all": 0, "all_gather": 0}
        self._buf: dict = {}

    def attach(self, model) -> None:
        """Must run before the engine is built: the KV pool is sized from the model's (now local) head geometry."""
        if getattr(model, "tp_world", 1) != 1 or getattr(model, "pp_world", 1) != 1 or getattr(model, "cp", None) is not None:
            raise ValueError("the head / sequence exchange runs over whole model replicas")
        g = model.geom
        if g.Hq % self.world or g.Hkv % self.world:
            raise ValueError(f"{self.world} ranks do not divide {g.Hq} q / {g.Hkv} kv heads")
        if g.q_gated:
            raise ValueError("gated attention is not built for the head / sequence exchange")
        self.full = g
        self.Hq_l, self.Hkv_l, self.D = g.Hq // self.world, g.Hkv // self.world, g.D
        model.geom = dataclasses.replace(g, Hq=self.Hq_l, Hkv=self.Hkv_l)
        model.Hq, model.Hkv = self.Hq_l, self.Hkv_l
        model.up = self

    # ---- staging ----
    def scratch(self, name: str, rows: int, cols: int, dtype=torch.bfloat16) -> torch.Tensor:
        t = self._buf.get(name)
        if t is None or t.shape[0] < rows or t.shape[1] != cols or t.dtype != dtype:
            t = torch.zeros(max(rows, 16), cols, dtype=dtype, device=self.device)
            self._buf[name] = t
        return t[:rows]

    def head_columns(self, qkv_full: torch.Tensor, r: int) -> torch.Tensor:
        """[rows][q_l + 2 kv_l]: the q | k | v columns of rank r's heads out of a full-head projection row."""
        D, f = self.D, self.full
        q0, k0, v0 = 0, f.Hq * D, (f.Hq + f.Hkv) * D
        ql, kl = self.Hq_l * D, self.Hkv_l * D
        return torch.cat([qkv_full[:, q0 + r * ql: q0 + (r + 1) * ql], qkv_full[:, k0 + r * kl: k0 + (r + 1) * kl],
                          qkv_full[:, v0 + r * kl: v0 + (r + 1) * kl]], dim=1)

    # ---- exchanges ----
    def rows_to_heads(self, qkv_loc: torch.Tensor, M: int) -> torch.Tensor:
        """qkv_loc [M / R][all heads] of this rank's rows -> [M][local heads] of every row (rows in chunk order)."""
        n = M // self.world
        send = torch.stack([self.head_columns(qkv_loc, r) for r in range(self.world)]).contiguous()       # [R][n][w]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        self.stats["all_to_all"] += 1
        return recv.reshape(M, send.shape[2])

    def heads_to_rows(self, attn_h: torch.Tensor, M: int) -> torch.Tensor:
        """attn_h [M][local q heads] -> [M / R][all q heads] of this rank's rows."""
        n, ql = M // self.world, self.Hq_l * self.D
        send = attn_h.reshape(self.world, n, ql).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)
        self.stats["all_to_all"] += 1
        return recv.permute(1, 0, 2).reshape(n, self.world * ql)                                          # head blocks in rank order

    def gather_heads(self, attn_h: torch.Tensor) -> torch.Tensor:
        """attn_h [rows][local q heads] on every rank -> [rows][all q heads] on every rank."""
        parts = [torch.empty_like(attn_h) for _ in range(self.world)]
        dist.all_gather(parts, attn_h.contiguous(), group=self.group)
        self.stats["all_gather"] += 1
        return torch.cat(parts, dim=1)

    def split_ready(self, M: int) -> bool:
        return M % self.world == 0 and M >= self.world

    def local_rows(self, M: int) -> tuple[int, int]:
        n = M // self.world
        return self.rank * n, (self.rank + 1) * n
