"""Projections over raw GGUF blocks (gemv_gguf.cu, ops/linear.py: GgufLinear) against the host block decoder
(csrc/host/gguf.cpp), which is itself checked bit for bit against golden vectors in tests/test_gguf.py.  The raw rows
are random bytes with sane fp16 scales: every byte pattern is a valid block of these types."""
import numpy as np
import pytest
import torch

from grimoire_b200.formats.gguf import dequantize

BLOCK = {2: (18, 32), 8: (34, 32), 12: (144, 256), 13: (176, 256), 14: (210, 256), 20: (18, 32), 23: (136, 256)}      # type -> (bytes, weights)


def _raw_rows(t: int, N: int, K: int, seed: int) -> torch.Tensor:
    bb, bw = BLOCK[t]
    g = torch.Generator().manual_seed(seed)
    nb = K // bw
    raw = torch.randint(0, 256, (N, nb, bb), dtype=torch.uint8, generator=g)
    h = lambda v: torch.tensor(np.frombuffer(np.float16(v).tobytes(), dtype=np.uint8).copy())
    d = torch.rand(N, nb, generator=g) * 0.02 + 0.005
    dbytes = torch.tensor(np.frombuffer(d.numpy().astype(np.float16).tobytes(), dtype=np.uint8).copy()).reshape(N, nb, 2)
    if t in (2, 8, 20, 23):
        raw[:, :, 0:2] = dbytes
    elif t in (12, 13):
        raw[:, :, 0:2] = dbytes
        raw[:, :, 2:4] = dbytes                       # dmin of the same size
    else:
        raw[:, :, 208:210] = dbytes
    return raw.reshape(N, nb * bb).contiguous()


def _oracle(t: int, raw: torch.Tensor, K: int) -> torch.Tensor:
    return dequantize(t, raw, raw.shape[0] * K).reshape(raw.shape[0], K)


@pytest.mark.gpu
@pytest.mark.parametrize("t", [2, 8, 12, 13, 14, 20, 23])
@pytest.mark.parametrize("M", [1, 3, 8, 13])
def test_gemv_over_raw_blocks_matches_host_decoder(t, M):
    from grimoire_b200.ops.linear import GgufLinear
    from grimoire_b200.ops.workspace import Workspace

    N, K = 44, 1024
    raw = _raw_rows(t, N, K, seed=10 * t + M)
    W = _oracle(t, raw, K)
    lin = GgufLinear([(raw, t)], K, "cuda", "t", workspace=Workspace("cuda"))
    x = (torch.randn(M, K, generator=torch.Generator().manual_seed(M)) * 0.5).bfloat16()
    ref = x.float() @ W.t()
    scale = max(1.0, float(ref.abs().max()))
    out = torch.zeros(M, N, dtype=torch.float32, device="cuda")
    lin(x.cuda(), out, "f32")
    assert float((out.cpu() - ref).abs().max()) < 2e-3 * scale
    ob = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    lin(x.cuda(), ob, "bf16")
    assert float((ob.float().cpu() - ref).abs().max()) < 2e-2 * scale
    h = torch.ones(M, N, dtype=torch.float32, device="cuda")
    lin(x.cuda(), h, "add_f32")
    assert float((h.cpu() - 1.0 - ref).abs().max()) < 2e-3 * scale


@pytest.mark.gpu
def test_gguf_linear_mixed_types_swiglu_and_tall_inputs():
    """q|k|v with a different block type for v (what K-quant mixes do), a (gate, up) pair with the SwiGLU product, and more
    than 64 rows through the bf16 expansion + tcgen05 GEMM."""
    from grimoire_b200.ops.linear import GgufLinear
    from grimoire_b200.ops.workspace import Workspace

    K = 512
    q, k, v = _raw_rows(12, 64, K, 1), _raw_rows(12, 32, K, 2), _raw_rows(14, 32, K, 3)
    lin = GgufLinear([(q, 12), (k, 12), (v, 14)], K, "cuda", "qkv", workspace=Workspace("cuda"))
    W = torch.cat([_oracle(12, q, K), _oracle(12, k, K), _oracle(14, v, K)])
    assert torch.equal(lin.dequant(), W)
    for M in (2, 100):
        x = (torch.randn(M, K, generator=torch.Generator().manual_seed(M)) * 0.5).bfloat16()
        ref = x.float() @ W.t()
        out = torch.zeros(M, 128, dtype=torch.bfloat16, device="cuda")
        lin(x.cuda(), out, "bf16")
        assert float((out.float().cpu() - ref).abs().max()) < 3e-2 * max(1.0, float(ref.abs().max())), M
    g, u = _raw_rows(8, 96, K, 4), _raw_rows(2, 96, K, 5)
    gu = GgufLinear([(g, 8), (u, 2)], K, "cuda", "gu", swiglu=True, workspace=Workspace("cuda"))
    for M in (1, 70):
        x = (torch.randn(M, K, generator=torch.Generator().manual_seed(7 + M)) * 0.5).bfloat16()
        ref = torch.nn.functional.silu(x.float() @ _oracle(8, g, K).t()) * (x.float() @ _oracle(2, u, K).t())
        out = torch.zeros(M, 96, dtype=torch.bfloat16, device="cuda")
        gu(x.cuda(), out, "swiglu")
        assert float((out.float().cpu() - ref).abs().max()) < 3e-2 * max(1.0, float(ref.abs().max())), M


def test_gguf_linear_cpu_path_uses_the_host_decoder():
    from grimoire_b200.ops.linear import GgufLinear

    K = 256
    raw = _raw_rows(12, 8, K, 9)
    lin = GgufLinear([(raw, 12)], K, "cpu", "t")
    x = torch.randn(2, K).bfloat16()
    out = torch.zeros(2, 8)
    lin(x, out, "f32")
    assert torch.allclose(out, x.float() @ _oracle(12, raw, K).t(), atol=1e-4)
