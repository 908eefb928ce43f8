"""--proj {bf16, int8, fp8_e4m3, fp8_e5m2, mxfp8}: the byte-per-weight projections (RowQLinear / smallm_rowq.cu)."""
import dataclasses

import pytest
import torch

from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.formats.w4_tile_layout import interleave_gate_up_q
from grimoire_b200.ops.linear import RowQLinear

FMTS = [Fmt.BF16, Fmt.INT8, Fmt.FP8_E4M3, Fmt.FP8_E5M2, Fmt.MXFP8]
PROJ = ["bf16", "int8", "fp8_e4m3", "fp8_e5m2", "mxfp8"]


def _ref(x, qw, swiglu):
    y = x.float() @ qw.dequant().float().t()
    if swiglu:
        I = qw.N // 2
        y3 = y.reshape(x.shape[0], I // 16, 2, 16)
        return (torch.nn.functional.silu(y3[:, :, 0]) * y3[:, :, 1]).reshape(x.shape[0], I)
    return y


@pytest.mark.parametrize("fmt", FMTS)
def test_rowq_cpu_matches_dequant(fmt):
    g = torch.Generator().manual_seed(0)
    qw = quantize(torch.randn(64, 128, generator=g) * 0.05, fmt)
    lin = RowQLinear(qw, "cpu")
    x = torch.randn(3, 128, generator=g).bfloat16()
    out = torch.zeros(3, 64)
    lin(x, out, "f32")
    assert torch.allclose(out, _ref(x, qw, False), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M", [1, 2, 3, 8, 17, 100])
@pytest.mark.parametrize("N,K", [(512, 1024), (48, 160), (1000, 2048)])
def test_rowq_gpu_matches_dequant(fmt, M, N, K):
    g = torch.Generator().manual_seed(M + N)
    qw = quantize(torch.randn(N, K, generator=g) * 0.05, fmt)
    lin = RowQLinear(qw, "cuda")
    x = torch.randn(M, K, generator=g).bfloat16()
    ref = _ref(x, qw, False)
    # from 4 rows the byte-per-weight formats may run the tcgen05 GEMM over a resident bf16 expansion of the weight
    tol = (0.03 if M >= 4 else 2e-3) * max(1.0, float(ref.abs().max()))
    out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    lin(x.cuda(), out, "f32")
    assert float((out.cpu() - ref).abs().max()) < tol
    h = torch.ones(M, N, dtype=torch.float32, device="cuda")
    lin(x.cuda(), h, "add_f32")
    assert float((h.cpu() - 1.0 - ref).abs().max()) < tol
    ob = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    lin(x.cuda(), ob, "bf16")
    assert float((ob.float().cpu() - ref).abs().max()) < tol + 0.01 * max(1.0, float(ref.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("M", [1, 5, 8, 40, 128])
def test_rowq_gpu_swiglu(fmt, M):
    g = torch.Generator().manual_seed(M)
    I, K = 256, 512
    wg, wu = torch.randn(I, K, generator=g) * 0.05, torch.randn(I, K, generator=g) * 0.05
    qw = interleave_gate_up_q(quantize(wg, fmt), quantize(wu, fmt))
    lin = RowQLinear(qw, "cuda", swiglu=True)
    x = torch.randn(M, K, generator=g).bfloat16()
    ref = _ref(x, qw, True)
    out = torch.zeros(M, I, dtype=torch.bfloat16, device="cuda")
    lin(x.cuda(), out, "swiglu")
    assert float((out.float().cpu() - ref).abs().max()) < (0.03 if M > 64 else 0.012) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("proj", PROJ)
def test_dense_model_rowq_cpu_generates(proj):
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import tiny_dense
    from grimoire_b200.models.dense import DenseModel
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = dataclasses.replace(tiny_dense(), quant=proj)
    sd = random_state_dict(cfg, seed=0)
    m = DenseModel.from_state_dict(cfg, sd, "cpu")
    assert isinstance(m.layers[0].qkv, RowQLinear) and isinstance(m.layers[0].gate_up, RowQLinear)
    lim = EngineLimits(max_slots=1, max_ctx=64, prefill_chunk=32, max_decode_rows=4)
    prompt = list(range(1, 17))
    assert len(Engine(m, lim).generate(prompt, 8)) == 8
    # logits agree with the int4-g128 model of the same weights to quantisation noise
    ref = Engine(DenseModel.from_state_dict(dataclasses.replace(cfg, quant="int4"), sd, "cpu"), lim)
    e = Engine(m, lim)
    l8, l4 = e.prefill(e.open(), prompt).float(), ref.prefill(ref.open(), prompt).float()
    assert float((l8 - l4).abs().max()) < 0.25 * max(1.0, float(l4.abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("proj", PROJ)
def test_dense_model_rowq_gpu_matches_cpu(proj):
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import tiny_dense
    from grimoire_b200.models.dense import DenseModel
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = dataclasses.replace(tiny_dense(), quant=proj)
    sd = random_state_dict(cfg, seed=0)
    lim = EngineLimits(max_slots=2, max_ctx=256, prefill_chunk=128, max_decode_rows=4)
    prompt = torch.randint(0, 4096, (100,), generator=torch.Generator().manual_seed(1)).tolist()
    cpu, gpu = Engine(DenseModel.from_state_dict(cfg, sd, "cpu"), lim), Engine(DenseModel.from_state_dict(cfg, sd, "cuda"), lim)
    sc, sg = cpu.open(), gpu.open()
    lc, lg = cpu.prefill(sc, prompt).float(), gpu.prefill(sg, prompt).float().cpu()
    assert float((lc - lg).abs().max()) < 0.05 * max(1.0, float(lc.abs().max()))
    tok = int(lc.argmax())
    _, l2c = cpu.decode_rows([tok], [sc], [sc.length], return_logits=True)
    _, l2g = gpu.decode_rows([tok], [sg], [sg.length], use_graph=False, return_logits=True)
    assert float((l2c[0] - l2g[0].float().cpu()).abs().max()) < 0.05 * max(1.0, float(l2c.abs().max()))
    # graph replay gives the eager tokens
    toks = gpu.generate(prompt[:32], 8)
    assert len(toks) == 8
