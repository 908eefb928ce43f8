"""Hybrid linear-attention decoders (Qwen3-Next / Qwen3.5 family): repeating 3 Gated DeltaNet
layers + 1 gated full-attention layer, every FFN a top-k MoE with one shared expert.  The same class
serves the family's neighbours: the 27B hybrid with a dense SwiGLU FFN (int4 projections), and
Qwen3-MoE-style decoders (plain attention in every layer, routed experts without a shared expert).

Layer math and conventions follow the reference engine's forward() for this family
(grimoire.cpp:15105-15202 DeltaNet mixer, :15207-15351 gated attention, :15364-15453 MoE) and the
numerics it pins with tests: zero-centred (1+w) norms except the DeltaNet output norm, q|gate split
of q_proj with ``attn * sigmoid(gate)`` before o_proj, per-head q/k RMSNorm before partial RoPE,
conv(k=4)+SiLU over packed q|k|v, L2-normalised q/k, ``o = (S q)/sqrt(Dk)``, ``rms_norm(o)*silu(z)``,
router softmax over all experts -> top-k -> renormalise, shared expert scaled by sigmoid(x.w_gate).
Weights are block-scaled fp8 (e4m3, 1x128 scales); the tiny a/b gate projections and the router
stay bf16.  Per-slot recurrent state (DeltaNet ``S`` + conv ring) lives beside the paged KV cache.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from ..formats.codecs import Fmt
from ..formats.quantize import QuantWeight, quantize
from ..formats.w4_tile_layout import interleave_gate_up_q
from ..ops import core as K
from ..ops import hybrid as Hb
from ..ops import ref
from ..ops.linear import BF16Linear, W4Linear
from ..ops.workspace import Workspace
from ..utils import trace
from .config import ModelConfig
from .dense import DenseModel, RowBatch

# expert-parallel decode of <= 8 rows through replicated routing + the all-reducing combine kernel (0: dispatch chain)
EP_DECODE_LL = os.environ.get("GRIMOIRE_EP_DECODE_LL", "1") != "0"


@dataclass
class MoEBlock:
    router: BF16Linear            # [E + 1][H]: expert logits, last row = shared-expert gate
    gate_up: torch.Tensor         # uint8 [E][2I][H]
    gate_up_scale: torch.Tensor   # fp32  [E][2I][H/128]
    down: torch.Tensor            # uint8 [E][H][I]
    down_scale: torch.Tensor      # fp32  [E][H][I/128]
    shared_gu: Optional[Hb.FP8BlockLinear]      # None: no shared expert (Qwen3-MoE)
    shared_down: Optional[Hb.FP8BlockLinear]


@dataclass
class HybridLayer:
    kind: str                     # "gdn" | "attn"
    in_norm: torch.Tensor
    post_norm: torch.Tensor
    moe: Optional[MoEBlock]       # None: dense FFN (ffn_gu / ffn_down)
    cx: Optional[object] = None   # ops.cpu_experts.CpuExperts: this layer's experts that live in host memory
    ffn_gu: Optional[object] = None
    ffn_down: Optional[object] = None
    # K2-Horizon: separate attention gate projection (softplus), routed value projection, router selection bias
    gate_proj: Optional[object] = None
    mova: Optional[object] = None
    router_bias: Optional[torch.Tensor] = None
    # gdn
    in_qkv: Optional[Hb.FP8BlockLinear] = None
    in_z: Optional[Hb.FP8BlockLinear] = None
    in_ab: Optional[BF16Linear] = None
    conv_w: Optional[torch.Tensor] = None
    A_log: Optional[torch.Tensor] = None
    dt_bias: Optional[torch.Tensor] = None
    gdn_norm: Optional[torch.Tensor] = None
    out_proj: Optional[Hb.FP8BlockLinear] = None
    # attention
    qkv: Optional[Hb.FP8BlockLinear] = None
    o: Optional[Hb.FP8BlockLinear] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    kv_index: int = -1
    state_index: int = -1


class HybridBuffers:
    def __init__(self, m: "HybridModel", max_rows: int, max_logit_rows: int, dense_kv_tokens: int = 0):
        cfg, dev = m.cfg, m.device
        H, g = cfg.hidden_size, m.geom
        bf, f32 = torch.bfloat16, torch.float32
        mk = lambda *s, dt: torch.zeros(*s, dtype=dt, device=dev)
        k = cfg.num_experts_per_tok
        self.h, self.x = mk(max_rows, H, dt=f32), mk(max_rows, H, dt=bf)
        self.qkv = mk(max_rows, cfg.q_size + 2 * cfg.kv_size, dt=bf)
        self.q, self.gate, self.attn = (mk(max_rows, g.Hq * g.D, dt=bf) for _ in range(3))
        self.gdn_qkv, self.gdn_conv = mk(max_rows, m.gdn_channels, dt=bf), mk(max_rows, m.gdn_channels, dt=bf)
        self.gdn_z, self.gdn_o = mk(max_rows, m.Hv * m.Dv, dt=bf), mk(max_rows, m.Hv * m.Dv, dt=bf)
        self.gdn_ab = mk(max_rows, 2 * m.Hv, dt=f32)
        # row pitch padded to 16 bytes so the GEMM epilogue can use 128-bit stores
        self.router = mk(max_rows, (cfg.num_experts + 1 + 3) // 4 * 4, dt=f32)
        self.ids, self.wts = mk(max_rows, k, dt=torch.int32), mk(max_rows, k + 1, dt=f32)
        self.act = mk(max_rows * k, cfg.moe_intermediate_size, dt=bf)
        self.y = mk(max_rows * (k + 1), H, dt=f32)
        self.act_s = mk(max_rows, max(cfg.shared_expert_intermediate_size, 0 if cfg.is_moe else cfg.intermediate_size), dt=bf)
        # dense-FFN layers inside an MoE model (mlp-only / off-step layers) get their own activation rows
        mixed = cfg.is_moe and not all(cfg.layer_is_sparse(i) for i in range(cfg.num_hidden_layers))
        self.act_d = mk(max_rows, cfg.intermediate_size, dt=bf) if mixed else self.act_s
        self.pos = mk(max_rows, k + 1, dt=torch.int32)
        self.xf, self.logits = mk(max_logit_rows, H, dt=bf), mk(max_logit_rows, cfg.vocab_size, dt=f32)
        self.next_ids = mk(max_logit_rows, dt=torch.int32)
        self.dense_k = mk(dense_kv_tokens, g.Hkv * g.D, dt=bf) if dense_kv_tokens else None
        self.dense_v = mk(dense_kv_tokens, g.Hkv * g.D, dt=bf) if dense_kv_tokens else None
        # static tables of the decode path: one run / one expert tile per row (graph friendly)
        ar = torch.arange(max_rows * k, dtype=torch.int32, device=dev)
        self.run_start = torch.arange(max_rows, dtype=torch.int32, device=dev)
        self.run_len = torch.ones(max_rows, dtype=torch.int32, device=dev)
        self.tile_row0, self.tile_rows, self.tile_src = ar, torch.ones_like(ar), (ar // k).to(torch.int32)
        self.max_rows, self.max_logit_rows = max_rows, max_logit_rows
        self._k = k
        self._decode_pos: dict[int, torch.Tensor] = {}

    def decode_pos(self, M: int) -> torch.Tensor:
        t = self._decode_pos.get(M)
        if t is None:
            k, dev = self._k, self.pos.device
            t = torch.empty(M, k + 1, dtype=torch.int32, device=dev)
            t[:, :k] = torch.arange(M * k, dtype=torch.int32, device=dev).reshape(M, k)
            t[:, k] = torch.arange(M * k, M * (k + 1), dtype=torch.int32, device=dev)
            self._decode_pos[M] = t
        return t


class _DictSource:
    """A state dict behind the tensor-resolver interface ``from_checkpoint`` reads (synthetic weights, tests)."""

    def __init__(self, cfg: ModelConfig, sd: dict):
        self.cfg, self.sd = cfg, sd
        self.prefix = "model.language_model." if any(k.startswith("model.language_model.") for k in sd) else "model."

    def linear(self, name: str):
        return self.sd.get(name + ".weight")

    def plain(self, name: str):
        return self.sd.get(name)

    tensor = plain

    def embedding(self):
        return self.sd[self.prefix + "embed_tokens.weight"]


class _AgnesSource:
    """An Agnes checkpoint seen through the hybrid family's names (src/qwen35_loader.cpp:1148-1165, :1264-1290): its two
    attention submodules are ``delta_attn`` / ``global_attn``, and every mlp carries a second, narrow SwiGLU
    (``mlp.parallel_ffn.{gate,up,down}_proj``) on the same normed input whose result lands in the same residual.  Two
    SwiGLUs summed are one SwiGLU over the concatenated intermediate, so the fold is a load-time concatenation:
    gate' = [gate ; pgate] and up' = [up ; pup] by rows, down' = [down | pdown] by columns."""

    def __init__(self, src, cfg: ModelConfig):
        self.src, self.cfg, self.prefix = src, cfg, src.prefix

    def _name(self, name: str) -> str:
        return name.replace(".linear_attn.", ".delta_attn.").replace(".self_attn.", ".global_attn.")

    def plain(self, name: str):
        return self.src.plain(self._name(name))

    def tensor(self, name: str):
        return self.src.tensor(self._name(name))

    def embedding(self):
        return self.src.embedding()

    def linear(self, name: str):
        dense = lambda t: t.dequant() if hasattr(t, "dequant") else t.float()
        for role in ("gate_proj", "up_proj", "down_proj"):
            if name.endswith(".mlp." + role) and self.cfg.parallel_ffn_intermediate_size > 0:
                main = self.src.linear(name)
                par = self.src.linear(name[: -len(role)] + "parallel_ffn." + role)
                if main is None:
                    return None
                if par is None:
                    raise KeyError(f"parallel_ffn_intermediate_size is {self.cfg.parallel_ffn_intermediate_size} but the checkpoint has no "
                                   f"{name[: -len(role)]}parallel_ffn.{role}")
                return torch.cat([dense(main), dense(par)], dim=1 if role == "down_proj" else 0)
        return self.src.linear(self._name(name))


class HybridModel:
    def __init__(self, cfg: ModelConfig, device, workspace: Optional[Workspace] = None, max_slots: int = 8, proj: Optional[str] = None):
        self.cfg, self.device = cfg, torch.device(device)
        self.ws = workspace or Workspace(device)
        self.tp_rank, self.tp_world, self.pp_rank, self.pp_world = 0, 1, 0, 1
        self.tp = self.pp = None
        self.ep = None                   # parallel.ep.ExpertParallel when the experts are sharded over ranks
        self.expert_perm = None          # per layer: physical -> logical expert (set_expert_placement), None = identity
        self._local_moe = None           # single-GPU instance of the same chain for prompt chunks
        self._hits = None                # [layers][experts] int64 routing counts on the device (record_expert_hits)
        rt = os.environ.get("GRIMOIRE_ROUTE_TRACE", "")
        self._route_trace = open(rt, "ab") if rt and cfg.is_moe else None
        self._trace_decode = False
        if self._route_trace is not None:
            self.graph_safe = False      # the trace reads the routes on the host every layer
        self.vram_experts = 0            # > 0: experts per layer kept on the device, the rest computed on the host
        self.heat = None                 # expert_placement.ExpertHeat while the RAM tier swaps experts at run time
        self.swaps_per_step, self.swaps_done = 0, 0
        self._cur_layer = 0
        self.ep_rank, self.ep_world = 0, 1
        self.supports_verify_rows = True       # verify blocks: rows run as one recurrent run, rejected rows are undone by replay
        self._vtrace = None                    # per-layer conv inputs / gate inputs of the verify step in flight
        self.Hq, self.Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        self.Hk, self.Hv, self.Dk, self.Dv = cfg.linear_num_key_heads, cfg.linear_num_value_heads, cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.gdn_channels = 2 * self.Hk * self.Dk + self.Hv * self.Dv
        self.geom = K.AttnGeom(self.Hq, self.Hkv, cfg.head_dim, cfg.rot_dim, cfg.softmax_scale or ref.softmax_scale(cfg.head_dim),
                               bool(cfg.attn_output_gate), cfg.sliding_window, cfg.rms_norm_eps, cfg.norm_offset)
        # projections outside the experts: block fp8 beside fp8 experts, int4 g128 for the dense-FFN hybrid, unless told
        self.proj = proj if proj in ("int4", "fp8") else ("fp8" if cfg.is_moe or cfg.quant == "fp8_block" else "int4")
        self.inv_freq = ref.rope_inv_freq(cfg.rot_dim, cfg.rope_theta).to(self.device)
        self.layers: list[HybridLayer] = []          # all layers, in order
        self.kv_layer_count = cfg.num_attention_layers()
        self.max_slots = max_slots
        n_gdn = cfg.num_hidden_layers - self.kv_layer_count
        self.state = torch.zeros(n_gdn, max_slots, self.Hv, self.Dv, self.Dk, dtype=torch.float32, device=self.device)
        self.ring = torch.zeros(n_gdn, max_slots, self.gdn_channels, 3, dtype=torch.float32, device=self.device)
        self.ring_tmp = torch.zeros(max_slots, self.gdn_channels, 3, dtype=torch.float32, device=self.device)
        self.embed = self.final_norm = self.lm_head = None

    def reset_slot(self, slot: int) -> None:
        """A fresh conversation starts from a zero recurrent state (grimoire.cpp:10436-10451)."""
        self.state[:, slot].zero_()
        self.ring[:, slot].zero_()

    def snapshot_slot(self, slot: int):
        """Recurrent state of one conversation (prefix-cache entries of this family carry it: the reference snapshots
        conv tails + DeltaNet matrices with the KV, snapshot_recurrent grimoire.cpp:12364-12406)."""
        return self.state[:, slot].clone(), self.ring[:, slot].clone()

    def load_slot(self, slot: int, snap) -> None:
        self.state[:, slot].copy_(snap[0])
        self.ring[:, slot].copy_(snap[1])

    # ------------------------------------------------------------------------------------------
    # speculative verify blocks over recurrent layers
    # ------------------------------------------------------------------------------------------
    def begin_verify(self, slots: torch.Tensor, rows: int):
        """Call before a decode step that contains verify blocks (several consecutive rows of one conversation).  The
        recurrent layers run a block as one run, so after the step their state has consumed every row, including drafts
        that will be rejected.  This records what is needed to undo that: a snapshot of the state of ``slots`` and, per
        DeltaNet layer, the conv inputs and gate inputs of every row (the reference's verify kernels leave the state
        untouched and save k / v / a / beta per row instead, src/deltanet.cpp:368-460; its replay is :461-628)."""
        n_gdn = self.state.shape[0]
        tr = self._vtrace_buf if getattr(self, "_vtrace_buf", None) is not None and self._vtrace_buf["pre"].shape[1] >= rows else None
        if tr is None:
            tr = {"pre": torch.zeros(n_gdn, rows, self.gdn_channels, dtype=torch.bfloat16, device=self.device),
                  "ab": torch.zeros(n_gdn, rows, 2 * self.Hv, dtype=torch.float32, device=self.device)}
            self._vtrace_buf = tr
        self._vtrace = tr
        return {"snap": self.save_recurrent(slots), "slots": [int(v) for v in slots.tolist()], "trace": tr}

    def end_verify(self) -> None:
        self._vtrace = None

    def commit_verify(self, handle, slot: int, row0: int, keep: int, rows: int, pos0: int, buf: "HybridBuffers") -> None:
        """Make the recurrent state of ``slot`` the state after the first ``keep`` of the ``rows`` rows of its verify block
        (rows row0.. of the step, first position pos0): nothing to do when every row was accepted; otherwise the
        snapshot comes back and the kept rows are replayed through conv + delta rule from the recorded inputs."""
        if keep >= rows:
            return
        idx, st, rg = handle["snap"]
        j = handle["slots"].index(slot)
        self.state[:, slot].copy_(st[:, j])
        self.ring[:, slot].copy_(rg[:, j])
        if keep <= 0:
            return
        dev = self.device
        tr = handle["trace"]
        row_seq = torch.full((keep,), slot, dtype=torch.int32, device=dev)
        row_pos = torch.arange(pos0, pos0 + keep, dtype=torch.int32, device=dev)
        run_slot = torch.tensor([slot], dtype=torch.int32, device=dev)
        run_start = torch.zeros(1, dtype=torch.int32, device=dev)
        run_len = torch.tensor([keep], dtype=torch.int32, device=dev)
        touched = torch.tensor([slot], dtype=torch.long, device=dev)
        conv, z, o = buf.gdn_conv[:keep], buf.gdn_z[:keep], buf.gdn_o[:keep]
        for L in self.layers:
            if L.kind != "gdn":
                continue
            si = L.state_index
            pre = tr["pre"][si, row0: row0 + keep]
            Hb.conv4_silu(pre, L.conv_w, self.ring[si], self.ring_tmp, row_seq, row_pos, conv, touched)
            Hb.gdn_runs(conv, tr["ab"][si, row0: row0 + keep], z, L.A_log, L.dt_bias, L.gdn_norm, self.cfg.rms_norm_eps, self.state[si],
                        run_slot, run_start, run_len, o, self.Hk, self.Hv, self.Dk, self.Dv)

    def attach_ep(self, group, max_rows: int, fused=None):
        """Shard the MoE layers over ``group`` (the model must have been built with the matching
        ep_rank / ep_world expert slice)."""
        from ..parallel.ep import ExpertParallel

        cfg = self.cfg
        self.ep = ExpertParallel(group, self.device, cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size,
                                 cfg.moe_intermediate_size, max_rows, fused=fused)
        if (self.ep.rank, self.ep.world) != (self.ep_rank, self.ep_world):
            raise ValueError("expert slice of the model does not match the expert-parallel group")
        return self.ep

    def save_recurrent(self, slots: torch.Tensor):
        """Copy of the recurrent state of ``slots`` (conv tails + delta-rule matrices).  Used around
        executions whose effect must not persist (graph warm-up runs) and for speculative rollback
        (the reference keeps a per-slot state checkpoint for the same purpose, grimoire.cpp:10452-10500)."""
        idx = slots.long()
        return idx, self.state.index_select(1, idx), self.ring.index_select(1, idx)

    def restore_recurrent(self, saved) -> None:
        idx, st, rg = saved
        self.state.index_copy_(1, idx, st)
        self.ring.index_copy_(1, idx, rg)

    # ------------------------------------------------------------------------------------------
    @staticmethod
    def random(cfg: ModelConfig, device, seed: int = 0, std: float = 0.02, max_slots: int = 8, gen_device=None,
               ep_rank: int = 0, ep_world: int = 1) -> "HybridModel":
        """Random-init weights.  ``gen_device`` picks where the numbers are drawn (draw on "cpu" to get
        the same model on a GPU and on the CPU path).  With ``ep_world`` > 1 the rank keeps experts
        [ep_rank * E/W, (ep_rank + 1) * E/W) of every layer (same values as the unsharded model)."""
        if cfg.is_k2:
            # the K2 layer mix (dense and sparse layers, routed value experts) is built from named tensors
            from .synthetic import random_hybrid_state_dict

            return HybridModel.from_checkpoint(_DictSource(cfg, random_hybrid_state_dict(cfg, seed)), device, max_slots=max_slots)
        m = HybridModel(cfg, device, max_slots=max_slots)
        m.ep_rank, m.ep_world = ep_rank, ep_world
        if cfg.num_experts % ep_world or (not cfg.is_moe and ep_world > 1):
            raise ValueError("experts do not split evenly over the expert-parallel ranks")
        e0, e1 = ep_rank * (cfg.num_experts // ep_world), (ep_rank + 1) * (cfg.num_experts // ep_world)
        dev = m.device
        gdev = torch.device(gen_device or dev)
        g = torch.Generator(device=gdev)
        H, D = cfg.hidden_size, cfg.head_dim
        E, I, Is = cfg.num_experts, cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size

        def rnd(*shape, tag, scale=std):
            g.manual_seed(seed * 1000003 + tag)
            return (torch.randn(*shape, generator=g, device=gdev, dtype=torch.float32) * scale).to(dev)

        fp8 = m._lin
        nw = (lambda n: torch.zeros(n, device=dev)) if cfg.norm_zero_centered else (lambda n: torch.ones(n, device=dev))
        kv_i = st_i = 0
        for i in range(cfg.num_hidden_layers):
            t = i * 64
            moe, ffn = None, {}
            if not cfg.is_moe:
                Id = cfg.intermediate_size
                ffn = dict(ffn_gu=m._lin_gate_up(rnd(Id, H, tag=t + 25), rnd(Id, H, tag=t + 26), f"L{i}.gate_up"),
                           ffn_down=fp8(rnd(H, Id, tag=t + 27), f"L{i}.down"))
            else:
                gu = rnd(E, 2 * I, H, tag=t + 20)
                dn = rnd(E, H, I, tag=t + 21)
                gq = [quantize(gu[e], Fmt.FP8_BLOCK) for e in range(E)] if E <= 64 else None
                if gq is not None:
                    dq = [quantize(dn[e], Fmt.FP8_BLOCK) for e in range(E)]
                    gu8, gus = torch.stack([q.payload for q in gq]), torch.stack([q.scales for q in gq])
                    dn8, dns = torch.stack([q.payload for q in dq]), torch.stack([q.scales for q in dq])
                else:   # many experts: quantize as one [E*N][K] matrix (1x128 blocks never cross rows)
                    q1 = quantize(gu.reshape(E * 2 * I, H), Fmt.FP8_BLOCK)
                    q2 = quantize(dn.reshape(E * H, I), Fmt.FP8_BLOCK)
                    gu8, gus = q1.payload.reshape(E, 2 * I, H), q1.scales.reshape(E, 2 * I, H // 128)
                    dn8, dns = q2.payload.reshape(E, H, I), q2.scales.reshape(E, H, I // 128)
                del gu, dn
                gu8, gus, dn8, dns = gu8[e0:e1], gus[e0:e1], dn8[e0:e1], dns[e0:e1]
                router = rnd(E + 1, H, tag=t + 22, scale=0.5)
                if not Is:
                    router[E].zero_()
                moe = MoEBlock(BF16Linear(router, dev, f"L{i}.router"), gu8.contiguous(), gus.float().contiguous(),
                               dn8.contiguous(), dns.float().contiguous(),
                               Hb.FP8BlockLinear(rnd(2 * Is, H, tag=t + 23), dev, f"L{i}.shared_gu") if Is else None,
                               Hb.FP8BlockLinear(rnd(H, Is, tag=t + 24), dev, f"L{i}.shared_down") if Is else None)
            if cfg.is_attention_layer(i):
                L = HybridLayer("attn", nw(H), nw(H), moe, qkv=fp8(rnd(cfg.q_size + 2 * cfg.kv_size, H, tag=t + 1), f"L{i}.qkv"),
                                o=fp8(rnd(H, m.Hq * D, tag=t + 2), f"L{i}.o"), q_norm=nw(D) if cfg.qk_norm else None,
                                k_norm=nw(D) if cfg.qk_norm else None, kv_index=kv_i, **ffn)
                kv_i += 1
            else:
                L = HybridLayer("gdn", nw(H), nw(H), moe, in_qkv=fp8(rnd(m.gdn_channels, H, tag=t + 3), f"L{i}.in_qkv"),
                                in_z=fp8(rnd(m.Hv * m.Dv, H, tag=t + 4), f"L{i}.in_z"),
                                in_ab=BF16Linear(rnd(2 * m.Hv, H, tag=t + 5, scale=0.2), dev, f"L{i}.in_ab"),
                                conv_w=rnd(m.gdn_channels, 4, tag=t + 6, scale=0.4), A_log=rnd(m.Hv, tag=t + 7, scale=0.5),
                                dt_bias=rnd(m.Hv, tag=t + 8, scale=0.5), gdn_norm=torch.ones(m.Dv, device=dev),
                                out_proj=fp8(rnd(H, m.Hv * m.Dv, tag=t + 9), f"L{i}.out_proj"), state_index=st_i, **ffn)
                st_i += 1
            m.layers.append(L)
        m.embed = rnd(cfg.vocab_size, H, tag=900001).bfloat16()
        m.final_norm = nw(H)
        m.lm_head = fp8(rnd(cfg.vocab_size, H, tag=900002), "lm_head")
        return m

    # ------------------------------------------------------------------------------------------
    # checkpoints
    # ------------------------------------------------------------------------------------------
    def _lin(self, w, name: str):
        """Runtime projection outside the experts: int4 g128 (W4Linear) or block-scaled fp8, by the model's format."""
        if self.proj == "int4":
            if not (isinstance(w, QuantWeight) and w.fmt == Fmt.INT4):
                w = quantize(w.dequant() if hasattr(w, "dequant") else w.float(), Fmt.INT4, group=self.cfg.quant_group)
            return W4Linear(w, self.device, name, workspace=self.ws)
        return Hb.FP8BlockLinear(w, self.device, name)

    def _lin_gate_up(self, g, u, name: str):
        """(gate, up) of a SwiGLU FFN as one projection with the swiglu epilogue."""
        dense = lambda t: t.dequant() if hasattr(t, "dequant") else t.float()
        if self.proj == "int4":
            q = lambda t: t if isinstance(t, QuantWeight) and t.fmt == Fmt.INT4 else quantize(dense(t), Fmt.INT4, group=self.cfg.quant_group)
            return W4Linear(interleave_gate_up_q(q(g), q(u)), self.device, name, swiglu=True, workspace=self.ws)
        return Hb.FP8BlockLinear(torch.cat([dense(g), dense(u)], dim=0), self.device, name)

    def set_expert_placement(self, heat_file: str) -> bool:
        """Balanced expert ownership from a routing-heat file (models/expert_placement.py: the hit counts a serving run
        saved): per layer the hottest experts are dealt onto the least-loaded rank, so that the ranks of an expert-parallel
        group see even traffic instead of whatever the checkpoint's expert order gives.  Must be called before the layers
        are added; every rank must use the same file.  Returns False (identity placement) when the file does not match
        the model.  Reference: the heat / hit-file manager of the tiered-MoE path (src/moe_tier.cpp)."""
        from .expert_placement import ExpertHeat, balanced_placement

        cfg = self.cfg
        heat = ExpertHeat(cfg.num_hidden_layers, cfg.num_experts)
        if self.layers or not heat.load(heat_file):
            return False
        self.expert_perm = [balanced_placement(heat.h[l], self.ep_world) for l in range(cfg.num_hidden_layers)]
        return True

    def _add_layer(self, i: int, w: dict) -> None:
        """One layer from logical fp32 tensors (``[out][in]``; stored block-fp8 QuantWeights are used as they are).
        K2-Horizon layers add attn_gate (the softplus gate projection), router_bias, and on sparse layers v_router, v_router_bias,
        v_experts [Ev][kv][H] instead of v.
        Keys: in_norm, post_norm; for an MoE FFN router [E][H], gate_up [E][2I][H], down [E][H][I] and, with a shared
        expert, shared_gate [1][H], shared_gate_proj, shared_up_proj, shared_down_proj; for a dense FFN ffn_gate, ffn_up,
        ffn_down; then either q, k, v, o, q_norm, k_norm or in_qkv, in_z, in_a, in_b, conv [C][4],
        A_log, dt_bias, gdn_norm, out_proj."""
        cfg, dev = self.cfg, self.device
        E = cfg.num_experts
        e0, e1 = self.ep_rank * (E // self.ep_world), (self.ep_rank + 1) * (E // self.ep_world)
        f32 = lambda t: None if t is None else t.to(device=dev, dtype=torch.float32).contiguous()
        dense = lambda t: t.dequant() if hasattr(t, "dequant") else t.float()
        perm = self.expert_perm[i] if self.expert_perm is not None and cfg.is_moe else None
        if perm is not None:
            # Placement: physical expert j of this layer is logical expert perm[j].  The experts' weights and the router's
            # rows are permuted together, so routing yields physical ids and nothing downstream changes; rank r owns
            # physical experts [r E / W, (r + 1) E / W), i.e. the logical set the placement gave it.
            idx = torch.as_tensor(perm, dtype=torch.long)
            w = dict(w)
            w["gate_up"], w["down"] = w["gate_up"][idx], w["down"][idx]
            w["router"] = dense(w["router"])[idx]
        fp8 = self._lin

        def experts(t3):
            n, k = t3.shape[1], t3.shape[2]
            q = quantize(t3[e0:e1].reshape((e1 - e0) * n, k).float(), Fmt.FP8_BLOCK)
            return q.payload.reshape(e1 - e0, n, k).to(dev).contiguous(), q.scales.reshape(e1 - e0, n, k // 128).float().to(dev).contiguous()

        moe, ffn = None, {}
        if not cfg.layer_is_sparse(i):
            ffn = dict(ffn_gu=self._lin_gate_up(w["ffn_gate"], w["ffn_up"], f"L{i}.gate_up"), ffn_down=fp8(w["ffn_down"], f"L{i}.down"))
        else:
            gu8, gus = experts(w["gate_up"])
            dn8, dns = experts(w["down"])
            nres = self.vram_experts
            if 0 < nres < E:
                # RAM tier: physical experts [nres, E) stay in host memory (the placement put the hottest first)
                from ..ops.cpu_experts import CpuExperts
                from ..utils.host_budget import host_available_ram

                need_b = sum(t[nres:].numel() * t.element_size() for t in (gu8, gus, dn8, dns))
                if need_b + (1 << 30) > host_available_ram():
                    raise MemoryError(f"layer {i}: {need_b >> 20} MiB of host-resident experts do not fit the RAM this process may take")
                ffn["cx"] = CpuExperts(nres, gu8[nres:], gus[nres:], dn8[nres:], dns[nres:], pin=self.device.type == "cuda")
                gu8, gus, dn8, dns = (t[:nres].contiguous() for t in (gu8, gus, dn8, dns))
            sg = w.get("shared_gate")
            router = torch.cat([dense(w["router"]), dense(sg) if sg is not None else torch.zeros(1, cfg.hidden_size)], dim=0)
            shared = w.get("shared_gate_proj") is not None
            if shared and sg is None and not cfg.is_k2:          # K2's shared experts are ungated
                raise KeyError(f"layer {i}: a shared expert without its gate (mlp.shared_expert_gate)")
            if w.get("router_bias") is not None:
                ffn["router_bias"] = f32(w["router_bias"])
            moe = MoEBlock(BF16Linear(router, dev, f"L{i}.router"), gu8, gus, dn8, dns,
                           Hb.FP8BlockLinear(torch.cat([dense(w["shared_gate_proj"]), dense(w["shared_up_proj"])], dim=0), dev,
                                             f"L{i}.shared_gu") if shared else None,
                           Hb.FP8BlockLinear(w["shared_down_proj"], dev, f"L{i}.shared_down") if shared else None)
        if cfg.is_attention_layer(i):
            if w.get("v_experts") is not None:
                # K2 sparse layer: q | k from one projection, v from the routed bank of value experts
                from ..ops.k2 import MovaValue

                qkv = torch.cat([dense(w["q"]), dense(w["k"])], dim=0)
                ffn["mova"] = MovaValue(dense(w["v_router"]), w.get("v_router_bias"), w["v_experts"].float(), cfg.mova_top_k, dev)
            else:
                qkv = torch.cat([dense(w["q"]), dense(w["k"]), dense(w["v"])], dim=0)
            if w.get("attn_gate") is not None:
                ffn["gate_proj"] = fp8(w["attn_gate"], f"L{i}.attn_gate")
            L = HybridLayer("attn", f32(w["in_norm"]), f32(w["post_norm"]), moe, qkv=fp8(qkv, f"L{i}.qkv"), o=fp8(w["o"], f"L{i}.o"),
                            q_norm=f32(w.get("q_norm")), k_norm=f32(w.get("k_norm")),
                            kv_index=sum(1 for l in self.layers if l.kind == "attn"), **ffn)
        else:
            ab = torch.cat([dense(w["in_a"]), dense(w["in_b"])], dim=0)
            L = HybridLayer("gdn", f32(w["in_norm"]), f32(w["post_norm"]), moe, in_qkv=fp8(w["in_qkv"], f"L{i}.in_qkv"),
                            in_z=fp8(w["in_z"], f"L{i}.in_z"), in_ab=BF16Linear(ab, dev, f"L{i}.in_ab"),
                            conv_w=f32(w["conv"].reshape(self.gdn_channels, -1)), A_log=f32(w["A_log"]), dt_bias=f32(w["dt_bias"]),
                            gdn_norm=f32(w["gdn_norm"]), out_proj=fp8(w["out_proj"], f"L{i}.out_proj"),
                            state_index=sum(1 for l in self.layers if l.kind == "gdn"), **ffn)
        self.layers.append(L)

    @staticmethod
    def from_checkpoint(path, device, max_slots: int = 8, ep_rank: int = 0, ep_world: int = 1, expert_heat: str = "",
                        expert_perm=None, proj: Optional[str] = None, model_cls=None, vram_experts: int = 0) -> "HybridModel":
        """Load a HF directory of the hybrid family.  Tensor names follow the reference's resolver
        (src/qwen35_loader.cpp:1149-1169 ``linear_attn.{in_proj_qkv,in_proj_z,in_proj_a,in_proj_b,conv1d,A_log,dt_bias,norm,
        out_proj}``, :1320-1380 ``mlp.gate``, ``mlp.shared_expert*``, per-expert ``mlp.experts.N.*`` or the fused
        ``mlp.experts.gate_up_proj`` [E][2I][H] / ``mlp.experts.down_proj`` [E][H][I]; a dense FFN under ``mlp.gate_proj`` /
        ``up_proj`` / ``down_proj``).  Experts are served as block-scaled fp8; the other projections as block-scaled fp8 beside
        an MoE FFN and int4 g128 beside a dense one (``proj`` "int4" / "fp8" overrides); the a / b gates and the router stay
        bf16 (keep_qwen_bf16, :129-159)."""
        from ..formats.checkpoint import Checkpoint

        ck = Checkpoint(path) if isinstance(path, (str, bytes)) or hasattr(path, "__fspath__") else path    # or any tensor resolver
        cfg = ck.cfg
        if cfg.is_agnes and not isinstance(ck, _AgnesSource):
            ck = _AgnesSource(ck, cfg)
        if (cfg.is_moe and cfg.num_experts % ep_world) or (not cfg.is_moe and ep_world > 1):
            raise ValueError("from_checkpoint: the experts do not split over the expert-parallel ranks")
        m = (model_cls or HybridModel)(cfg, device, max_slots=max_slots, proj=proj)      # a family built on these blocks passes its class
        m.ep_rank, m.ep_world = ep_rank, ep_world
        if vram_experts and cfg.is_moe and vram_experts < cfg.num_experts:
            # RAM tier (one GPU): ``vram_experts`` experts per layer on the device -- the hottest of the heat file when there
            # is one, the first ones otherwise -- and the rest in host memory behind the CPU pool
            if ep_world > 1 or cfg.is_k2:
                raise ValueError("host-resident experts are served on one GPU with the softmax router")
            m.vram_experts = int(vram_experts)
            m.graph_safe = False                                  # the routes come back to the host every layer
            if expert_perm is None and expert_heat:
                from .expert_placement import ExpertHeat

                heat = ExpertHeat(cfg.num_hidden_layers, cfg.num_experts)
                if heat.load(expert_heat):
                    expert_perm = [sorted(range(cfg.num_experts), key=lambda e, l=l: (-float(heat.h[l][e]), e)) for l in range(cfg.num_hidden_layers)]
        if expert_perm is not None:
            m.expert_perm = [list(p) for p in expert_perm]       # explicit placement (per layer: physical -> logical expert)
        elif expert_heat:
            m.set_expert_placement(expert_heat)
        E = cfg.num_experts

        def need(v, name):
            if v is None:
                raise KeyError(f"checkpoint has no tensor for {name}")
            return v

        for i in range(cfg.num_hidden_layers):
            p = f"{ck.prefix}layers.{i}."
            lin = lambda k: need(ck.linear(p + k), p + k)
            w = {"in_norm": need(ck.plain(p + "input_layernorm.weight"), p + "input_layernorm"),
                 "post_norm": need(ck.plain(p + "post_attention_layernorm.weight"), p + "post_attention_layernorm")}
            dq = lambda t: t.dequant() if hasattr(t, "dequant") else t.float()
            if not cfg.layer_is_sparse(i):
                w.update(ffn_gate=lin("mlp.gate_proj"), ffn_up=lin("mlp.up_proj"), ffn_down=lin("mlp.down_proj"))
            else:
                w["router"] = lin("mlp.gate")
                if cfg.is_k2:
                    w["router_bias"] = ck.plain(p + "mlp.gate.bias")
                    if cfg.shared_expert_intermediate_size:
                        w.update(shared_gate_proj=lin("mlp.shared_experts.gate_proj"), shared_up_proj=lin("mlp.shared_experts.up_proj"),
                                 shared_down_proj=lin("mlp.shared_experts.down_proj"))
                elif cfg.shared_expert_intermediate_size:
                    w.update(shared_gate=ck.linear(p + "mlp.shared_expert_gate"), shared_gate_proj=lin("mlp.shared_expert.gate_proj"),
                             shared_up_proj=lin("mlp.shared_expert.up_proj"), shared_down_proj=lin("mlp.shared_expert.down_proj"))
                fused_gu, fused_dn = ck.tensor(p + "mlp.experts.gate_up_proj"), ck.tensor(p + "mlp.experts.down_proj")
                if fused_gu is not None and fused_dn is not None:
                    w["gate_up"], w["down"] = fused_gu.float(), fused_dn.float()
                else:
                    gu, dn = [], []
                    for e in range(E):
                        x = f"mlp.experts.{e}."
                        gu.append(torch.cat([dq(lin(x + "gate_proj")), dq(lin(x + "up_proj"))], dim=0))
                        dn.append(dq(lin(x + "down_proj")))
                    w["gate_up"], w["down"] = torch.stack(gu), torch.stack(dn)
            if cfg.is_attention_layer(i):
                a = "self_attn."
                w.update(q=lin(a + "q_proj"), k=lin(a + "k_proj"), o=lin(a + "o_proj"),
                         q_norm=ck.plain(p + a + "q_norm.weight"), k_norm=ck.plain(p + a + "k_norm.weight"))
                if cfg.attn_gate_proj:
                    w["attn_gate"] = lin(a + "gate_proj")
                if cfg.mova_experts and cfg.layer_is_sparse(i):
                    w.update(v_router=lin(a + "v_router"), v_router_bias=ck.plain(p + a + "v_router.bias"),
                             v_experts=torch.stack([dq(lin(a + f"v_experts.{e}")) for e in range(cfg.mova_experts)]))
                else:
                    w["v"] = lin(a + "v_proj")
            else:
                a = "linear_attn."
                w.update(in_qkv=lin(a + "in_proj_qkv"), in_z=lin(a + "in_proj_z"), in_a=lin(a + "in_proj_a"), in_b=lin(a + "in_proj_b"),
                         conv=need(ck.plain(p + a + "conv1d.weight"), p + a + "conv1d"), A_log=need(ck.plain(p + a + "A_log"), "A_log"),
                         dt_bias=need(ck.plain(p + a + "dt_bias"), "dt_bias"), gdn_norm=need(ck.plain(p + a + "norm.weight"), "norm"),
                         out_proj=lin(a + "out_proj"))
            m._add_layer(i, w)
        m.embed = ck.embedding().to(device=m.device, dtype=torch.bfloat16).contiguous()
        m.final_norm = need(ck.plain(ck.prefix + "norm.weight"), "norm.weight").to(m.device)
        head = ck.linear("lm_head")
        m.lm_head = m._lin(head if head is not None else ck.embedding(), "lm_head")
        return m

    def weight_bytes(self) -> int:
        n = self.lm_head.nbytes()
        for L in self.layers:
            moe = L.moe
            if moe is not None:
                n += moe.gate_up.numel() + moe.down.numel() + 4 * (moe.gate_up_scale.numel() + moe.down_scale.numel())
            if L.mova is not None:
                n += L.mova.w.numel() + 4 * L.mova.scale.numel()
            for lin in (L.in_qkv, L.in_z, L.out_proj, L.qkv, L.o, L.ffn_gu, L.ffn_down, L.gate_proj, moe and moe.shared_gu, moe and moe.shared_down):
                if lin is not None:
                    n += lin.nbytes()
        return n

    def make_buffers(self, max_rows: int, max_logit_rows: int, dense_kv_tokens: int = 0) -> HybridBuffers:
        return HybridBuffers(self, max_rows, max_logit_rows, dense_kv_tokens)

    # ------------------------------------------------------------------------------------------
    def _moe(self, L: HybridLayer, x, h, buf: HybridBuffers, M: int, decode: bool) -> None:
        cfg, moe = self.cfg, L.moe
        E, k, H = cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size
        lg = buf.router[:M, : cfg.num_experts + 1]
        moe.router(x, lg, "f32")
        if cfg.router_sigmoid:
            self._moe_k2(L, x, h, buf, M, decode, lg)
            return self._credit(ids=buf.ids[:M])
        if self.ep is None and not decode and x.is_cuda and M > 64 and L.cx is None and self._route_trace is None:
            # a prompt chunk on one GPU: group the rows by expert on the device (the expert-parallel chain with
            # this GPU as its only rank) instead of sorting on the host, which would stall the stream every layer
            if self._local_moe is None or self._local_moe.max_rows < buf.max_rows:
                from ..parallel.ep import ExpertParallel

                self._local_moe = ExpertParallel(None, self.device, E, k, H, cfg.moe_intermediate_size, buf.max_rows, fused=True)
            self._local_moe.moe_fused(moe, x, h, lg, buf.ids, buf.wts, buf.act_s, M, cfg.norm_topk_prob)
            return self._credit(counts=self._local_moe.counts)
        if self.ep is not None and self.ep.fused and decode and M <= self.ep.ll_rows and EP_DECODE_LL:
            # a few decode rows: every rank runs the chosen experts it owns on the replicated rows and the combine
            # kernel all-reduces the weighted sums (no dispatch / return traffic, one exchange per layer)
            ep = self.ep
            ids, wts = buf.ids[:M], buf.wts[:M]
            Hb.moe_route(lg, E, k, cfg.norm_topk_prob, ids, wts, shared_gate=True)
            te, nr, pos = ep.decode_tiles(ids, M)
            act, y = buf.act[: M * k], buf.y[: M * (k + 1)]
            r0, src = buf.tile_row0[: M * k], buf.tile_src[: M * k]
            Hb.grouped_gemm_fp8(x, src, te, r0, nr, moe.gate_up, moe.gate_up_scale, act, "swiglu", small=True)
            Hb.grouped_gemm_fp8(act, None, te, r0, nr, moe.down, moe.down_scale, y, "f32", small=True)
            if moe.shared_gu is None:
                y[M * k: M * (k + 1)].zero_()
            elif ep.rank == 0:
                moe.shared_gu(x, buf.act_s[:M], "swiglu")
                moe.shared_down(buf.act_s[:M], y[M * k: M * (k + 1)], "f32")
            ep.combine_allreduce(h, y, pos, wts, M)
            return self._credit(ids=ids) if ep.rank == 0 else None      # every rank routed the same rows: one of them counts
        if self.ep is not None:
            if self.ep.fused:
                self.ep.moe_fused(moe, x, h, lg, buf.ids, buf.wts, buf.act_s, M, cfg.norm_topk_prob)
                return self._credit(counts=self.ep.counts)          # this rank's share of the rows
            self.ep.moe_allreduce(moe, x, h, lg, M, cfg.norm_topk_prob, ids_out=buf.ids[:M])
            return self._credit(ids=buf.ids[:M]) if self.ep.rank == 0 else None
        ids, wts = buf.ids[:M], buf.wts[:M]
        Hb.moe_route(lg, E, k, cfg.norm_topk_prob, ids, wts, shared_gate=True)
        self._credit(ids=ids)
        host_part = None
        if L.cx is not None:
            # routes to host experts: the CPU pool computes them from host copies of the rows while the device runs the
            # resident ones; on the device they become expert 0 with weight 0
            ids_h, wts_h, x_h = (t.to("cpu", copy=True) for t in (ids, wts, x))       # copies even when the model itself runs on the CPU path
            if self.heat is not None:
                perm = self.expert_perm[self._cur_layer]
                self.heat.credit(self._cur_layer, [perm[j] for j in ids_h.reshape(-1).tolist()])
            away = ids >= L.cx.first
            wts[:, :k].masked_fill_(away, 0.0)
            ids.masked_fill_(away, 0)
            host_part = L.cx.run(x_h, ids_h, wts_h)
        act, y, pos = buf.act[: M * k], buf.y[: M * (k + 1)], buf.pos[:M]
        if decode:
            te, r0, nr, src = ids.reshape(-1), buf.tile_row0[: M * k], buf.tile_rows[: M * k], buf.tile_src[: M * k]
            pos = buf.decode_pos(M)          # static for a row count: slot j of row m is grouped row m*k + j, shared at M*k + m
        else:
            flat = ids.reshape(-1).long()
            order = torch.sort(flat, stable=True).indices
            counts = torch.bincount(flat, minlength=E).cpu()
            src = (order // k).to(torch.int32)
            inv = torch.empty_like(order)
            inv[order] = torch.arange(order.numel(), device=order.device)
            pos[:, :k] = inv.reshape(M, k).to(torch.int32)
            tiles_per = (counts + 15) // 16
            starts = torch.cumsum(counts, 0) - counts
            te = torch.repeat_interleave(torch.arange(E), tiles_per)
            within = torch.arange(int(tiles_per.sum())) - torch.repeat_interleave(torch.cumsum(tiles_per, 0) - tiles_per, tiles_per)
            r0c = starts[te] + within * 16
            nrc = torch.minimum(torch.full_like(r0c, 16), counts[te] - within * 16)
            te, r0, nr = (t.to(torch.int32).to(x.device) for t in (te, r0c, nrc))
        Hb.grouped_gemm_fp8(x, src, te, r0, nr, moe.gate_up, moe.gate_up_scale, act, "swiglu", small=decode)
        Hb.grouped_gemm_fp8(act, None, te, r0, nr, moe.down, moe.down_scale, y, "f32", small=decode)
        # shared expert as slot k of the combine (a zero contribution when the model has none)
        if moe.shared_gu is None:
            y[M * k: M * (k + 1)].zero_()
        else:
            moe.shared_gu(x, buf.act_s[:M], "swiglu")
            moe.shared_down(buf.act_s[:M], y[M * k: M * (k + 1)], "f32")
        if not decode:
            pos[:, k] = torch.arange(M * k, M * (k + 1), dtype=torch.int32, device=x.device)
        Hb.moe_combine(h, y, pos, wts)
        if host_part is not None:
            h.add_(host_part.to(h.device, non_blocking=True))

    # ---- routing counts for the placement file ----
    def record_expert_hits(self, path: str, every: int = 256) -> None:
        """Count every routing decision on the device ([layer][expert]) and add the counts to the hit file ``path`` every
        ``every`` served tokens and at ``save_expert_hits`` (tm_save_hits, src/grimoire.cpp:14295-14320: each process adds
        what it counted since its last save).  The file is the one ``set_expert_placement`` reads at the next load."""
        cfg = self.cfg
        if not cfg.is_moe:
            return
        self._hits = torch.zeros(cfg.num_hidden_layers, cfg.num_experts, dtype=torch.int64, device=self.device)
        self._hits_saved = torch.zeros(cfg.num_hidden_layers, cfg.num_experts, dtype=torch.int64)
        self._hits_one = torch.ones(1, dtype=torch.int64, device=self.device)
        self._hits_path, self._hits_every, self._hits_tokens = path, max(1, int(every)), 0

    def _credit(self, ids=None, counts=None) -> None:
        if self._route_trace is not None and ids is not None:
            # diagnosis (GRIMOIRE_ROUTE_TRACE=<file>): int32 {layer, rows, top_k, kind (1 prompt rows, 2 decode rows)} then
            # rows x top_k int32 logical expert ids -- the order in which experts were asked for, which the counts cannot
            # give (route_trace, src/grimoire.cpp:14322-14338).  Costs a device-to-host read per layer.
            import struct

            h = ids.to("cpu", copy=True)
            if self.expert_perm is not None:
                perm = torch.tensor(self.expert_perm[self._cur_layer], dtype=torch.int32)
                h = perm[h.long()]
            M, k = h.shape
            self._route_trace.write(struct.pack("<4i", self._cur_layer, M, k, 2 if M <= 64 and self._trace_decode else 1))
            self._route_trace.write(h.to(torch.int32).contiguous().numpy().tobytes())
            self._route_trace.flush()
        if self._hits is None:
            return
        row = self._hits[self._cur_layer]
        if counts is not None:
            row.add_(counts[: row.numel()])
        else:
            flat = ids.reshape(-1).long()
            row.index_add_(0, flat, self._hits_one.expand(flat.numel()))

    # ---- RAM tier: experts change places between the device and the host as the traffic moves ----
    def enable_expert_swaps(self, swaps_per_step: int, params=None) -> None:
        """Keep a decayed heat per (layer, expert) from the routes the host sees and, at every step boundary, promote up to
        ``swaps_per_step`` hot host experts into the device slots of colder resident ones (hysteresis as in
        ``ExpertHeat.propose_swaps``; within a layer: every layer owns its device slots).  Reference: the heat engine of the
        tiered-MoE manager (include/b70/expert_heat.hpp:22-100; tm_heat_step, src/grimoire.cpp:14348)."""
        from .expert_placement import ExpertHeat

        cfg = self.cfg
        if not self.vram_experts:
            raise ValueError("expert swaps need host-resident experts (vram_experts)")
        if self.expert_perm is None:
            self.expert_perm = [list(range(cfg.num_experts)) for _ in range(cfg.num_hidden_layers)]
        self.heat = ExpertHeat(cfg.num_hidden_layers, cfg.num_experts, params)
        self.swaps_per_step = int(swaps_per_step)

    def swap_experts(self, layer: int, hot: int, cold: int) -> None:
        """Logical expert ``hot`` (in host memory) takes the device slot of logical expert ``cold``: weights, scales and
        router rows change places, and so do the two entries of the layer's placement."""
        L, perm = self.layers[layer], self.expert_perm[layer]
        j, hh = perm.index(cold), perm.index(hot)
        n = self.vram_experts
        if not (j < n <= hh) or L.cx is None:
            raise ValueError("swap_experts: hot must be host-resident and cold device-resident")
        moe, cx = L.moe, L.cx
        for dev_t, host_t in ((moe.gate_up, cx.gu), (moe.gate_up_scale, cx.gus), (moe.down, cx.dn), (moe.down_scale, cx.dns)):
            tmp = dev_t[j].to("cpu", copy=True)
            dev_t[j].copy_(host_t[hh - n])
            host_t[hh - n].copy_(tmp)
        rw = moe.router.w
        tmp = rw[j].clone()
        rw[j].copy_(rw[hh])
        rw[hh].copy_(tmp)
        perm[j], perm[hh] = hot, cold
        if self._hits is not None:                           # the routing counts are kept per physical slot: they move along
            for t in (self._hits[layer], self._hits_saved[layer]):
                a = t[j].clone()
                t[j] = t[hh]
                t[hh] = a
        self.swaps_done += 1

    def heat_step(self) -> int:
        """One step boundary of the heat engine; returns the number of swaps made."""
        if self.heat is None or self.swaps_per_step <= 0:
            return 0
        n, made = self.vram_experts, 0
        for l, L in enumerate(self.layers):
            if L.cx is None or made >= self.swaps_per_step:
                continue
            perm = self.expert_perm[l]
            where = {e: j for j, e in enumerate(perm)}
            for sw in self.heat.propose_swaps(lambda ll, e: where[e] < n, lambda ll, e: ll == l):
                if made >= self.swaps_per_step:
                    break
                self.swap_experts(l, sw.promote_expert, sw.demote_expert)
                made += 1
        return made

    def on_tokens(self, n: int) -> None:
        """Host-side step boundary (the engine calls it with the rows it committed)."""
        self.heat_step()
        if self._hits is None:
            return
        self._hits_tokens += n
        if self._hits_tokens >= self._hits_every:
            self.save_expert_hits()

    def save_expert_hits(self) -> None:
        """Add the counts since the last save to the hit file under an exclusive lock (several expert-parallel ranks write
        the same file).  Counts are kept per physical expert and land on the logical expert the placement maps it to."""
        if self._hits is None:
            return
        import fcntl
        import json
        import os

        from .expert_placement import ExpertHeat

        cfg = self.cfg
        now = self._hits.cpu()
        delta = now - self._hits_saved
        self._hits_saved, self._hits_tokens = now, 0
        if self.expert_perm is not None:
            logical = torch.zeros_like(delta)
            for l, perm in enumerate(self.expert_perm):
                logical[l, torch.tensor(perm, dtype=torch.long)] = delta[l]
            delta = logical
        if not int(delta.sum()):
            return
        with open(self._hits_path + ".lock", "w") as lock:
            fcntl.flock(lock, fcntl.LOCK_EX)
            heat = ExpertHeat(cfg.num_hidden_layers, cfg.num_experts)
            if os.path.exists(self._hits_path) and not heat.load(self._hits_path):
                return                                   # another model's file: left alone
            heat.hits = heat.hits + delta.numpy()
            heat.save(self._hits_path)

    def _moe_k2(self, L: HybridLayer, x, h, buf: HybridBuffers, M: int, decode: bool, lg) -> None:
        """K2 routing (sigmoid scores, selection-only bias, normalised and scaled weights) with an ungated shared expert, on the
        plain grouped-GEMM path of one GPU (rows grouped by expert on the host for prompt chunks)."""
        from ..ops import k2 as K2

        cfg, moe = self.cfg, L.moe
        E, k = cfg.num_experts, cfg.num_experts_per_tok
        if self.ep is not None:
            raise NotImplementedError("the K2 router is not built into the expert-parallel chain")
        ids, wts = buf.ids[:M], buf.wts[:M]
        K2.router_topk_bias(lg[:, :E], L.router_bias, k, ids, wts, True, cfg.norm_topk_prob, cfg.router_scale)
        wts[:, k] = 1.0
        act, y, pos = buf.act[: M * k], buf.y[: M * (k + 1)], buf.pos[:M]
        if decode:
            te, r0, nr, src = ids.reshape(-1), buf.tile_row0[: M * k], buf.tile_rows[: M * k], buf.tile_src[: M * k]
            pos = buf.decode_pos(M)
        else:
            flat = ids.reshape(-1).long()
            order = torch.sort(flat, stable=True).indices
            counts = torch.bincount(flat, minlength=E).cpu()
            src = (order // k).to(torch.int32)
            inv = torch.empty_like(order)
            inv[order] = torch.arange(order.numel(), device=order.device)
            pos[:, :k] = inv.reshape(M, k).to(torch.int32)
            tiles_per = (counts + 15) // 16
            starts = torch.cumsum(counts, 0) - counts
            te = torch.repeat_interleave(torch.arange(E), tiles_per)
            within = torch.arange(int(tiles_per.sum())) - torch.repeat_interleave(torch.cumsum(tiles_per, 0) - tiles_per, tiles_per)
            r0c = starts[te] + within * 16
            nrc = torch.minimum(torch.full_like(r0c, 16), counts[te] - within * 16)
            te, r0, nr = (t.to(torch.int32).to(x.device) for t in (te, r0c, nrc))
        Hb.grouped_gemm_fp8(x, src, te, r0, nr, moe.gate_up, moe.gate_up_scale, act, "swiglu", small=decode)
        Hb.grouped_gemm_fp8(act, None, te, r0, nr, moe.down, moe.down_scale, y, "f32", small=decode)
        if moe.shared_gu is None:
            y[M * k: M * (k + 1)].zero_()
        else:
            moe.shared_gu(x, buf.act_s[:M], "swiglu")
            moe.shared_down(buf.act_s[:M], y[M * k: M * (k + 1)], "f32")
        if not decode:
            pos[:, k] = torch.arange(M * k, M * (k + 1), dtype=torch.int32, device=x.device)
        Hb.moe_combine(h, y, pos, wts)

    def _norm(self, h, w, x) -> None:
        cfg = self.cfg
        if cfg.norm_groups > 1:
            from ..ops import k2 as K2

            K2.rmsnorm_grouped(h, w, x, cfg.norm_groups, cfg.rms_norm_eps)
        else:
            K.add_rmsnorm(h, w, x, cfg.rms_norm_eps, cfg.norm_offset)

    def forward(self, rb: RowBatch, buf: HybridBuffers, kv_layers, block_table) -> torch.Tensor:
        cfg, geom = self.cfg, self.geom
        M = rb.tokens.shape[0]
        eps, off = cfg.rms_norm_eps, cfg.norm_offset
        h, x = buf.h[:M], buf.x[:M]
        K.embed(rb.tokens, self.embed, h)
        prefill = rb.mode == "prefill"
        T = rb.q_pos0 + M
        if prefill:
            run_slot = torch.tensor([rb.seq_slot], dtype=torch.int32, device=self.device)
            run_start = torch.zeros(1, dtype=torch.int32, device=self.device)
            run_len = torch.tensor([M], dtype=torch.int32, device=self.device)
            touched = torch.tensor([rb.seq_slot], dtype=torch.long, device=self.device)
        elif rb.runs is not None:
            run_slot, run_start, run_len = rb.runs
            touched = run_slot.long()
        else:
            run_slot, run_start, run_len = rb.row_seq, buf.run_start[:M], buf.run_len[:M]
            touched = rb.row_seq.long()
        tr = self._vtrace
        tl = trace.timeline.on
        for li, L in enumerate(self.layers):
            if tl: trace.mark("gdn: norm + in projections" if L.kind == "gdn" else "attn: norm + qkv")
            if L.kind == "gdn":
                self._norm(h, L.in_norm, x)
                si = L.state_index
                L.in_qkv(x, buf.gdn_qkv[:M], "bf16")
                L.in_z(x, buf.gdn_z[:M], "bf16")
                L.in_ab(x, buf.gdn_ab[:M], "f32")
                if tl: trace.mark("gdn: conv + recurrence")
                if tr is not None:
                    tr["pre"][si, :M].copy_(buf.gdn_qkv[:M])
                    tr["ab"][si, :M].copy_(buf.gdn_ab[:M])
                Hb.conv4_silu(buf.gdn_qkv[:M], L.conv_w, self.ring[si], self.ring_tmp, rb.row_seq, rb.row_pos, buf.gdn_conv[:M], touched)
                Hb.gdn_runs(buf.gdn_conv[:M], buf.gdn_ab[:M], buf.gdn_z[:M], L.A_log, L.dt_bias, L.gdn_norm, eps, self.state[si],
                            run_slot, run_start, run_len, buf.gdn_o[:M], self.Hk, self.Hv, self.Dk, self.Dv, chunked=prefill and M >= 32)
                if tl: trace.mark("gdn: out_proj")
                L.out_proj(buf.gdn_o[:M], h, "add_f32")
            else:
                kvl = kv_layers[L.kv_index]
                qkv, q, attn = buf.qkv[:M], buf.q[:M], buf.attn[:M]
                gate = buf.gate[:M] if geom.q_gated else None
                if L.mova is not None or L.gate_proj is not None or cfg.norm_groups > 1:
                    # K2: the normed input feeds q | k, the routed value projection and the gate projection
                    self._norm(h, L.in_norm, x)
                    if L.mova is not None:
                        nqk = L.qkv.N
                        L.qkv(x, qkv[:, :nqk], "bf16")
                        L.mova(x, qkv[:, nqk:])
                    else:
                        L.qkv(x, qkv, "bf16")
                    if L.gate_proj is not None:
                        L.gate_proj(x, buf.gate[:M], "bf16")
                else:
                    DenseModel._norm_linear(L.qkv, h, L.in_norm, x, qkv, "bf16", eps, off)   # norm inside the one-row GEMV when it can
                if tl: trace.mark("attn: rope + attention")
                if prefill:
                    if rb.q_pos0 > 0:
                        K.gather_kv_dense(kvl, block_table[rb.seq_slot], rb.q_pos0, buf.dense_k, buf.dense_v)
                    K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, gate,
                                   buf.dense_k[rb.q_pos0: T], buf.dense_v[rb.q_pos0: T])
                    K.flash_prefill(q, buf.dense_k, buf.dense_v, geom, attn, rb.q_pos0, gate)
                else:
                    K.rope_kvwrite(qkv, rb.row_pos, rb.row_seq, block_table, self.inv_freq, geom, q, kvl, L.q_norm, L.k_norm, gate)
                    K.paged_decode_attn(q, rb.row_seq, rb.row_pos, block_table, kvl, geom, attn, rb.splits, self.ws, gate)
                if L.gate_proj is not None:
                    from ..ops import k2 as K2

                    K2.softplus_gate(attn, buf.gate[:M], attn)
                if tl: trace.mark("attn: o_proj")
                L.o(attn, h, "add_f32")
            if tl: trace.mark("ffn")
            if L.moe is None:
                act = buf.act_d[:M]
                if cfg.norm_groups > 1:
                    self._norm(h, L.post_norm, x)
                    L.ffn_gu(x, act, "swiglu")
                else:
                    DenseModel._norm_linear(L.ffn_gu, h, L.post_norm, x, act, "swiglu", eps, off)
                L.ffn_down(act, h, "add_f32")
            else:
                self._norm(h, L.post_norm, x)
                self._cur_layer, self._trace_decode = li, not prefill
                self._moe(L, x, h, buf, M, decode=not prefill)
        if tl: trace.mark("head")
        if rb.logits_rows is None:
            hsel, n = h, M
        else:
            n = rb.logits_rows.shape[0]
            hsel = h.index_select(0, rb.logits_rows) if n != M else h
        xf, logits = buf.xf[:n], buf.logits[:n]
        self._norm(hsel, self.final_norm, xf)
        self.lm_head(xf, logits, "f32")
        if tl: trace.mark("end")
        return logits
