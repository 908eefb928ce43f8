"""MXFP4 projections: the hand-written small-M kernel and the dequantise-once GEMM path against the
fp32 dequantised oracle; the dense model with MXFP4 weights on the CPU path and on the GPU."""
import dataclasses

import pytest
import torch

from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.formats.w4_tile_layout import interleave_gate_up_q
from grimoire_b200.ops.linear import MXLinear


def _ref(x, qw, epi, swiglu):
    y = x.float() @ qw.dequant().t()
    if swiglu:
        I = qw.N // 2
        y3 = y.reshape(x.shape[0], I // 16, 2, 16)
        y = torch.nn.functional.silu(y3[:, :, 0]) * y3[:, :, 1]
        return y.reshape(x.shape[0], I)
    return y


def test_mxlinear_cpu_matches_dequant():
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 128, generator=g) * 0.05
    qw = quantize(w, Fmt.MXFP4)
    lin = MXLinear(qw, "cpu")
    x = torch.randn(3, 128, generator=g).bfloat16()
    out = torch.zeros(3, 64)
    lin(x, out, "f32")
    assert torch.allclose(out, _ref(x, qw, "f32", False), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 3, 8, 17, 64, 100])
@pytest.mark.parametrize("N,K", [(512, 1024), (48, 160), (5120, 2048)])
def test_mxlinear_gpu_matches_dequant(M, N, K):
    g = torch.Generator().manual_seed(M * 7 + N)
    w = torch.randn(N, K, generator=g) * 0.05
    qw = quantize(w, Fmt.MXFP4)
    lin = MXLinear(qw, "cuda")
    x = torch.randn(M, K, generator=g).bfloat16()
    ref = _ref(x, qw, "f32", False)
    tol = 2e-2 * float(ref.abs().max()) if M > 64 else 2e-3 * float(ref.abs().max())    # M > 64 rounds the weights to bf16
    for epi, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        out = torch.zeros(M, N, dtype=dt, device="cuda")
        lin(x.cuda(), out, epi)
        t = tol if dt == torch.float32 else tol + 8e-3 * float(ref.abs().max())
        assert float((out.float().cpu() - ref).abs().max()) < t, (epi, M, N, K)
    base = torch.randn(M, N, generator=g)
    out = base.clone().cuda()
    lin(x.cuda(), out, "add_f32")
    assert float((out.cpu() - base - ref).abs().max()) < tol


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 5, 8, 40, 96])
def test_mxlinear_gpu_swiglu(M):
    g = torch.Generator().manual_seed(M)
    I, K = 256, 512
    wg, wu = torch.randn(I, K, generator=g) * 0.05, torch.randn(I, K, generator=g) * 0.05
    qw = interleave_gate_up_q(quantize(wg, Fmt.MXFP4), quantize(wu, Fmt.MXFP4))
    lin = MXLinear(qw, "cuda", swiglu=True)
    x = torch.randn(M, K, generator=g).bfloat16()
    ref = _ref(x, qw, "swiglu", True)
    out = torch.zeros(M, I, dtype=torch.bfloat16, device="cuda")
    lin(x.cuda(), out, "swiglu")
    assert float((out.float().cpu() - ref).abs().max()) < (0.03 if M > 64 else 0.012) * max(1.0, float(ref.abs().max()))


def _mx_cfg():
    from grimoire_b200.models.config import tiny_dense
    return dataclasses.replace(tiny_dense(), quant="mxfp4")


def test_dense_model_mxfp4_cpu_generates():
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.dense import DenseModel
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = _mx_cfg()
    m = DenseModel.from_state_dict(cfg, random_state_dict(cfg, seed=0), "cpu")
    assert isinstance(m.layers[0].qkv, MXLinear) and isinstance(m.layers[0].gate_up, MXLinear)
    out = Engine(m, EngineLimits(max_slots=1, max_ctx=64, prefill_chunk=32, max_decode_rows=4)).generate(list(range(1, 17)), 8)
    assert len(out) == 8


@pytest.mark.gpu
def test_dense_model_mxfp4_gpu_matches_cpu():
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.dense import DenseModel
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = _mx_cfg()
    sd = random_state_dict(cfg, seed=0)
    lim = EngineLimits(max_slots=1, max_ctx=128, prefill_chunk=32, max_decode_rows=4)
    prompt = torch.randint(0, 4096, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    cpu, gpu = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), lim), Engine(DenseModel.from_state_dict(cfg, sd, "cuda"), lim)
    sc, sg = cpu.open(), gpu.open()
    lc, lg = cpu.prefill(sc, prompt).float(), gpu.prefill(sg, prompt).float().cpu()
    assert float((lc - lg).abs().max()) < 0.05 * max(1.0, float(lc.abs().max()))
    tok = int(lc.argmax())
    _, l2c = cpu.decode_rows([tok], [sc], [sc.length], return_logits=True)
    _, l2g = gpu.decode_rows([tok], [sg], [sg.length], use_graph=False, return_logits=True)
    assert float((l2c[0] - l2g[0].float().cpu()).abs().max()) < 0.05 * max(1.0, float(l2c.abs().max()))


def test_dense_model_fp8_block_cpu_and_api_proj(tmp_path):
    """--proj fp8: block-scaled e4m3 projections ([gate | up] SwiGLU halves) through the dense model."""
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import tiny_dense
    from grimoire_b200.models.dense import DenseModel
    from grimoire_b200.models.synthetic import random_state_dict
    from grimoire_b200.ops.hybrid import FP8BlockLinear

    cfg = dataclasses.replace(tiny_dense(), quant="fp8")
    sd = random_state_dict(cfg, seed=0)
    m = DenseModel.from_state_dict(cfg, sd, "cpu")
    assert isinstance(m.layers[0].qkv, FP8BlockLinear) and isinstance(m.layers[0].gate_up, FP8BlockLinear)
    lim = EngineLimits(max_slots=1, max_ctx=64, prefill_chunk=32, max_decode_rows=4)
    prompt = list(range(1, 17))
    out = Engine(m, lim).generate(prompt, 8)
    ref = Engine(DenseModel.from_state_dict(dataclasses.replace(cfg, quant="int4"), sd, "cpu"), lim)
    s1, s2 = Engine(m, lim).open(), ref.open()
    # fp8 (3 mantissa bits) and int4-g128 logits of the same weights agree to quantisation noise
    l8, l4 = Engine(m, lim).prefill(s1, prompt).float(), ref.prefill(s2, prompt).float()
    assert len(out) == 8 and float((l8 - l4).abs().max()) < 0.25 * max(1.0, float(l4.abs().max()))


@pytest.mark.gpu
def test_dense_model_fp8_gpu_matches_cpu():
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import tiny_dense
    from grimoire_b200.models.dense import DenseModel
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = dataclasses.replace(tiny_dense(), quant="fp8")
    sd = random_state_dict(cfg, seed=0)
    lim = EngineLimits(max_slots=1, max_ctx=256, prefill_chunk=128, max_decode_rows=4)
    prompt = torch.randint(0, 4096, (100,), generator=torch.Generator().manual_seed(1)).tolist()
    cpu, gpu = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), lim), Engine(DenseModel.from_state_dict(cfg, sd, "cuda"), lim)
    sc, sg = cpu.open(), gpu.open()
    lc, lg = cpu.prefill(sc, prompt).float(), gpu.prefill(sg, prompt).float().cpu()
    assert float((lc - lg).abs().max()) < 0.05 * max(1.0, float(lc.abs().max()))
    tok = int(lc.argmax())
    _, l2c = cpu.decode_rows([tok], [sc], [sc.length], return_logits=True)
    _, l2g = gpu.decode_rows([tok], [sg], [sg.length], use_graph=False, return_logits=True)
    assert float((l2c[0] - l2g[0].float().cpu()).abs().max()) < 0.05 * max(1.0, float(l2c.abs().max()))
