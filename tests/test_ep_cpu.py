"""Expert parallelism on CPU ranks (gloo, world 2): expert slicing, row shards and the all-reduce
composition must reproduce the single-rank hybrid model's logits."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.models.config import FULL_ATTN, LINEAR_ATTN, ModelConfig
from grimoire_b200.models.hybrid import HybridModel

LIM = dict(max_slots=2, max_ctx=128, prefill_chunk=32, max_decode_rows=4)


def _cfg():
    lt = [LINEAR_ATTN, FULL_ATTN]
    return ModelConfig(model_type="qwen3_next", hidden_size=256, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                       head_dim=128, vocab_size=512, intermediate_size=0, partial_rotary_factor=0.5, attn_output_gate=True, qk_norm=True,
                       norm_zero_centered=True, layer_types=lt, linear_num_key_heads=1, linear_num_value_heads=2,
                       linear_key_head_dim=128, linear_value_head_dim=128, num_experts=8, num_experts_per_tok=3,
                       moe_intermediate_size=128, shared_expert_intermediate_size=128, quant="fp8_block")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(eng):
    prompt = torch.randint(0, 512, (37,), generator=torch.Generator().manual_seed(3)).tolist()
    s = eng.open()
    lg = eng.prefill(s, prompt).float().cpu().clone()
    toks, l2 = eng.decode_rows([int(lg.argmax())], [s], [s.length], return_logits=True)
    return lg, l2[0].float().cpu().clone(), toks


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model = HybridModel.random(_cfg(), "cpu", seed=4, max_slots=2, ep_rank=rank, ep_world=world)
        ep = model.attach_ep(dist.group.WORLD, max_rows=32)
        lg, l2, toks = _run(Engine(model, EngineLimits(**LIM)))
        q.put((rank, lg.numpy(), l2.numpy(), toks, ep.stats["allreduce_layers"], model.layers[0].moe.gate_up.shape[0]))
    finally:
        dist.destroy_process_group()


def test_ep2_cpu_logits_equal_single_rank():
    lg0, l20, toks0 = _run(Engine(HybridModel.random(_cfg(), "cpu", seed=4, max_slots=2), EngineLimits(**LIM)))
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = sorted((q.get(timeout=240) for _ in procs), key=lambda r: r[0])
        for p in procs:
            p.join(timeout=60)
    finally:
        for p in procs:
            if p.is_alive():
                p.kill()
    for rank, lg, l2, toks, n_ar, e_loc in res:
        assert e_loc == 4 and n_ar > 0
        assert toks == toks0
        assert float((torch.from_numpy(lg) - lg0).abs().max()) < 2e-3 * max(1.0, float(lg0.abs().max()))
        assert float((torch.from_numpy(l2) - l20).abs().max()) < 2e-3 * max(1.0, float(l20.abs().max()))
    assert (res[0][1] == res[1][1]).all()          # both ranks hold the same logits
