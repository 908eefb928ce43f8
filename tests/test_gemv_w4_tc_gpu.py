"""Single-row int4 projection as a tensor-core weight stream (gemv_w4_tc.cu, row-block layout of
formats/w4_rowblock.py) against the fp32 product with the dequantised weight; the layout round trip runs on CPU."""
import pytest
import torch

from grimoire_b200.formats import w4_rowblock as R
from grimoire_b200.formats import codecs as C
from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize

DEV = "cuda"


def test_rowblock_layout_round_trip_and_nibble_order():
    torch.manual_seed(1)
    qw = quantize(torch.randn(200, 384) * 0.05 + 0.01, Fmt.INT4, group=128)
    t = R.pack_rowblock(qw)
    assert t.data.shape == (2, 3, R.STAGE_BYTES) and t.N == 256 and t.rows == 200
    back = R.unpack_rowblock(t)
    q0, q1 = C.unpack_nibbles(qw.payload), C.unpack_nibbles(back.payload)
    assert torch.equal(q0, q1[:200]) and torch.equal(back.scales[:200], qw.scales.half()) and torch.equal(back.zeros[:200], qw.zeros)
    assert float(back.scales[200:].abs().max()) == 0.0                  # padding rows contribute nothing
    # word j of chunk i of row r: low nibbles = k0 .. k0 + 3, high nibbles = k0 + 4 .. k0 + 7, chunk at i ^ ((r >> 1) & 3)
    r, kg, i, j = 77, 2, 1, 2
    rec = t.data[0, kg]
    pos = i ^ ((r >> 1) & 3)
    word = rec[r * 64 + pos * 16 + 4 * j: r * 64 + pos * 16 + 4 * j + 4]
    k0 = 128 * kg + 32 * i + 8 * j
    assert [int(b) & 15 for b in word] == q0[r, k0:k0 + 4].tolist() and [int(b) >> 4 for b in word] == q0[r, k0 + 4:k0 + 8].tolist()
    with pytest.raises(ValueError):
        R.pack_rowblock(quantize(torch.randn(64, 256), Fmt.INT4, group=64))


def _lin(qw, swiglu=False):
    from grimoire_b200.ops import linear as L
    from grimoire_b200.ops.workspace import Workspace

    old = L.W4_TC
    L.W4_TC = True
    try:
        lin = L.W4Linear(qw, DEV, "t", swiglu=swiglu, workspace=Workspace(DEV))
    finally:
        L.W4_TC = old
    assert lin.rb is not None
    return lin


def _clean():
    from grimoire_b200.ops.core import status_read

    assert status_read()[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("epi", ["f32", "bf16", "add_f32"])
@pytest.mark.parametrize("N,K", [(256, 256), (1024, 1024), (200, 384), (5120, 17408), (7168, 5120), (34816, 1024)])
def test_tc_single_row_matches_dequant(N, K, epi):
    torch.manual_seed(N + K)
    qw = quantize(torch.randn(N, K) * 0.02 + 0.01, Fmt.INT4, group=128)
    lin = _lin(qw)
    x = torch.randn(1, K, device=DEV).bfloat16()
    want = x.float().cpu() @ qw.dequant().float().t()
    for rep in range(2):                                   # twice: the cross-CTA flags must be back at zero
        if epi == "add_f32":
            out = torch.ones(1, lin.Np, dtype=torch.float32, device=DEV)
            ref = want + 1.0
        else:
            out = torch.zeros(1, lin.Np, dtype=torch.float32 if epi == "f32" else torch.bfloat16, device=DEV)
            ref = want
        assert lin._tc_row(x, None, None, out, epi, 0.0, 0.0)
        tol = 2e-2 if epi == "bf16" else 2e-3
        got = out[:, :N].float().cpu()
        assert torch.allclose(got, ref, atol=tol * max(1.0, float(ref.abs().max())), rtol=tol), (rep, float((got - ref).abs().max()))
    _clean()


@pytest.mark.gpu
def test_tc_swiglu_and_fused_norm():
    from grimoire_b200.formats.w4_tile_layout import interleave_gate_up_q
    from grimoire_b200.ops import core as K_

    torch.manual_seed(3)
    I, K = 1536, 2048
    qg, qu = quantize(torch.randn(I, K) * 0.05, Fmt.INT4), quantize(torch.randn(I, K) * 0.05, Fmt.INT4)
    lin = _lin(interleave_gate_up_q(qg, qu), swiglu=True)
    x = torch.randn(1, K, device=DEV).bfloat16()
    xf = x.float().cpu()
    want = torch.nn.functional.silu(xf @ qg.dequant().float().t()) * (xf @ qu.dequant().float().t())
    out = torch.empty(1, I, dtype=torch.bfloat16, device=DEV)
    lin(x, out, "swiglu")                                  # the public call takes the stream for one row
    assert torch.allclose(out.float().cpu(), want, atol=0.012 * max(1.0, float(want.abs().max())), rtol=2e-2)
    # RMSNorm in the prologue == norm kernel, then the stream
    h = (torch.randn(1, K, device=DEV) * 3.0).contiguous()
    nw = (torch.rand(K, device=DEV) + 0.5).contiguous()
    xn = torch.empty(1, K, dtype=torch.bfloat16, device=DEV)
    for offset in (0.0, 1.0):
        K_.add_rmsnorm(h, nw, xn, 1e-6, offset)
        a = torch.empty(1, I, dtype=torch.bfloat16, device=DEV)
        b = torch.empty(1, I, dtype=torch.bfloat16, device=DEV)
        lin(xn, a, "swiglu")
        assert lin.fused_norm(h, nw, b, "swiglu", 1e-6, offset)
        assert torch.equal(a, b)
    _clean()


@pytest.mark.gpu
@pytest.mark.parametrize("xmax", [3.0e3, 2.0e-2])
def test_tc_outlier_and_tiny_activations(xmax):
    """Activations are quantised per 128-k group to 15 bits: a group with an outlier keeps 1/16256 of the outlier as its
    step, the other groups keep their own scale."""
    torch.manual_seed(11)
    N, K = 512, 5120
    qw = quantize(torch.randn(N, K) * 0.02 + 0.004, Fmt.INT4, group=128)
    lin = _lin(qw)
    x = torch.randn(1, K) * (xmax / 30 if xmax < 1 else 1.0)
    if xmax >= 1:
        x[0, 5] = xmax
        x[0, K // 2 + 3] = -0.8 * xmax
    x = x.to(DEV).bfloat16()
    want = x.float().cpu() @ qw.dequant().float().t()
    out = torch.empty(1, lin.Np, dtype=torch.float32, device=DEV)
    lin(x, out, "f32")
    got = out[:, :N].cpu()
    assert torch.isfinite(got).all()
    assert float((got - want).abs().max()) < 2e-3 * float(want.abs().max()) + 1e-6
    _clean()
