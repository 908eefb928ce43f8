"""End-to-end identities on a small dense model on the GPU (tier T3 of the reference's test
strategy: batched == sequential, graph == eager, chunked == one-shot, GPU == CPU oracle path)."""
import pytest
import torch

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.models.config import small_dense, tiny_dense
from grimoire_b200.models.dense import DenseModel
from grimoire_b200.models.synthetic import random_state_dict
from grimoire_b200.ops import core as K

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def setup():
    cfg = small_dense(layers=3)
    sd = random_state_dict(cfg, seed=0)
    gpu = Engine(DenseModel.from_state_dict(cfg, sd, "cuda"), EngineLimits(max_slots=4, max_ctx=512, prefill_chunk=128, max_decode_rows=16))
    cpu = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), EngineLimits(max_slots=4, max_ctx=512, prefill_chunk=128, max_decode_rows=16))
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (150,), generator=g).tolist()
    return cfg, gpu, cpu, prompt


def test_gpu_matches_cpu_path(setup):
    cfg, gpu, cpu, prompt = setup
    og, tg = gpu.generate(prompt, 12, collect_logits=True, use_graph=False)
    # teacher-force the CPU path with the GPU's tokens
    s = cpu.open()
    lg = cpu.prefill(s, prompt)
    worst = float((lg - tg[0]).abs().max())
    for i in range(11):
        pos = s.length
        _, l2 = cpu.decode_rows([og[i]], [s], [pos], return_logits=True)
        cpu.commit_rows([s], [og[i]], [pos])
        worst = max(worst, float((l2[0] - tg[i + 1]).abs().max()))
    cpu.release(s)
    scale = float(tg[0].abs().max())
    assert worst < 0.05 * max(scale, 1.0), (worst, scale)
    assert K.status_read()[0] == 0


def test_graph_replay_equals_eager(setup):
    cfg, gpu, cpu, prompt = setup
    a = gpu.generate(prompt, 16, use_graph=False)
    b = gpu.generate(prompt, 16, use_graph=True)
    assert a == b
    assert gpu.counters["graph_replays"] > 0


def test_batched_decode_is_bit_identical_to_solo(setup, monkeypatch):
    """With every batch width on the tensor-core small-M kernel (GRIMOIRE_GEMV_W4=0) a conversation's logits do not
    depend on who shares its step; with the single-row CUDA-core GEMV (the default) they agree to rounding and pick
    the same token."""
    from grimoire_b200.ops import linear

    cfg, gpu, cpu, prompt = setup
    for gemv in (False, True):
        monkeypatch.setattr(linear, "GEMV_W4", gemv)
        sa, sb = gpu.open(), gpu.open()
        la, lb = gpu.prefill(sa, prompt), gpu.prefill(sb, prompt[:61])
        ta, tb = int(la.argmax()), int(lb.argmax())
        both, lg = gpu.decode_rows([ta, tb], [sa, sb], [sa.length, sb.length], use_graph=False, return_logits=True)
        lg = lg.clone()
        solo, l1 = gpu.decode_rows([tb], [sb], [sb.length], use_graph=False, return_logits=True)
        assert both[1] == solo[0]
        if gemv:
            assert float((lg[1] - l1[0]).abs().max()) < 0.02 * max(1.0, float(l1[0].abs().max()))
        else:
            assert torch.equal(lg[1], l1[0])
        gpu.release(sa), gpu.release(sb)
        assert gpu.kv.pages_used() == 0


def test_tiny_model_on_gpu_matches_cpu(setup):
    cfg = tiny_dense()
    sd = random_state_dict(cfg, seed=0)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 4096, (16,), generator=g).tolist()
    lim = EngineLimits(max_slots=2, max_ctx=128, prefill_chunk=64, max_decode_rows=8)
    a = Engine(DenseModel.from_state_dict(cfg, sd, "cuda"), lim).generate(prompt, 32)
    b = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), lim).generate(prompt, 32)
    assert a == b
