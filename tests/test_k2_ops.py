"""K2-Horizon operators: the host oracles (ref/k2_ref.py) against the properties the reference pins in
tests/test_k2_horizon.cpp and include/b70/k2_horizon.hpp, the CUDA kernels (csrc/kernels/k2_ops.cu) against the oracles, and
the MoVA routed value projection built from them."""
import math

import pytest
import torch

from grimoire_b200.ops import k2
from grimoire_b200.ref import k2_ref


def test_oracle_properties():
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(3, 64, generator=g) * 2, 1 + 0.1 * torch.randn(64, generator=g)
    y = k2_ref.rmsnorm_grouped(x, w, 2, 1e-6)
    # each half is normalised on its own: scaling one half leaves the other half's output untouched
    x2 = x.clone(); x2[:, 32:] *= 7
    y2 = k2_ref.rmsnorm_grouped(x2, w, 2, 1e-6)
    assert torch.allclose(y[:, :32], y2[:, :32]) and torch.allclose(y[:, 32:], y2[:, 32:], atol=1e-4)
    assert torch.allclose(k2_ref.rmsnorm_grouped(x, w, 1, 1e-6), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w)
    # softplus with beta = ln 2 is log2(1 + 2^x); linear above the threshold; gate 0 keeps attn (softplus(0) = 1)
    t = torch.tensor([-3.0, 0.0, 2.5, 40.0])
    assert torch.allclose(k2_ref.softplus(t[:3], k2_ref.K2_GATE_BETA), torch.log2(1 + 2 ** t[:3]), atol=1e-5)
    assert float(k2_ref.softplus(t[3:], k2_ref.K2_GATE_BETA)) == 40.0
    assert torch.allclose(k2_ref.softplus_gate(torch.ones(4), torch.zeros(4)), torch.ones(4), atol=1e-6)
    # the bias moves the selection, not the weights
    lg = torch.tensor([[2.0, 1.0, 0.0, -1.0]])
    ids, wts = k2_ref.router_topk(lg, torch.tensor([0.0, 0.0, 0.0, 5.0]), 2, True, False)
    assert ids.tolist() == [[3, 0]] and torch.allclose(wts, torch.sigmoid(torch.tensor([[-1.0, 2.0]])))
    ids, wts = k2_ref.router_topk(lg, None, 2, True, True, scaling=2.5)
    assert ids.tolist() == [[0, 1]] and abs(float(wts.sum()) - 2.5) < 1e-6
    ids, _ = k2_ref.router_topk(torch.zeros(1, 6), None, 3)
    assert ids.tolist() == [[0, 1, 2]]                                    # ties to the lower index
    assert [k2_ref.is_sparse_layer(i, [0, 1, 2], 100, 1) for i in range(5)] == [False, False, False, True, True]
    assert not k2_ref.is_sparse_layer(3, [], 0, 1) and [k2_ref.is_sparse_layer(i, [], 8, 2) for i in range(4)] == [False, True, False, True]


def test_mova_block_cpu_matches_oracle():
    g = torch.Generator().manual_seed(1)
    E, out, H, k = 8, 128, 256, 4
    rw, rb = torch.randn(E, H, generator=g) * 0.3, torch.randn(E, generator=g) * 0.2
    ex = torch.randn(E, out, H, generator=g) * 0.05
    mv = k2.MovaValue(rw, rb, ex, k, "cpu", scaling=1.0)
    x = (torch.randn(3, H, generator=g) * 0.5).bfloat16()
    got = torch.zeros(3, out, dtype=torch.bfloat16)
    mv(x, got)
    want = k2_ref.mova_value(x.float(), rw.bfloat16().float(), rb, mv.dequant(), k)
    assert torch.allclose(got.float(), want, atol=2e-2, rtol=2e-2), float((got.float() - want).abs().max())


@pytest.mark.gpu
def test_k2_kernels_match_oracles():
    from grimoire_b200.ops import core as K

    g = torch.Generator().manual_seed(2)
    h, w = torch.randn(5, 2560, generator=g) * 3, 1 + 0.1 * torch.randn(2560, generator=g)
    for groups in (1, 2, 4):
        out = torch.zeros(5, 2560, dtype=torch.bfloat16, device="cuda")
        k2.rmsnorm_grouped(h.cuda(), w.cuda(), out, groups, 1e-6)
        assert torch.allclose(out.float().cpu(), k2_ref.rmsnorm_grouped(h, w, groups, 1e-6), atol=2e-2, rtol=2e-2)
    a, gt = (torch.randn(7, 1024, generator=g)).bfloat16(), (torch.randn(7, 1024, generator=g) * 8).bfloat16()
    gt[0, :4] = torch.tensor([40.0, -40.0, 0.0, 29.0]).bfloat16()
    out = torch.zeros_like(a, device="cuda")
    k2.softplus_gate(a.cuda(), gt.cuda(), out)
    assert torch.allclose(out.float().cpu(), k2_ref.softplus_gate(a, gt), atol=2e-2, rtol=2e-2)
    for E, k, sig, norm, scal in ((100, 8, True, True, 2.5), (64, 4, True, True, 1.0), (16, 2, False, False, 1.0), (512, 10, True, False, 1.0)):
        lg, bias = torch.randn(9, E, generator=g) * 2, torch.randn(E, generator=g) * 0.5
        lg[0] = 0.0                                                      # all ties: lowest indices after the bias order
        ids, wts = torch.zeros(9, k, dtype=torch.int32, device="cuda"), torch.zeros(9, k, device="cuda")
        k2.router_topk_bias(lg.cuda(), bias.cuda(), k, ids, wts, sig, norm, scal)
        wi, ww = k2_ref.router_topk(lg, bias, k, sig, norm, scal)
        assert torch.equal(ids.cpu().long(), wi), (E, k)
        assert torch.allclose(wts.cpu(), ww, atol=1e-5, rtol=1e-4)
    E, out_w, H, k = 64, 256, 512, 4
    rw, rb = torch.randn(E, H, generator=g) * 0.3, torch.randn(E, generator=g) * 0.2
    ex = torch.randn(E, out_w, H, generator=g) * 0.05
    mv = k2.MovaValue(rw, rb, ex, k, "cuda")
    for M in (1, 5):
        x = (torch.randn(M, H, generator=g) * 0.5).bfloat16()
        got = torch.zeros(M, out_w, dtype=torch.bfloat16, device="cuda")
        mv(x.cuda(), got)
        want = k2_ref.mova_value(x.float(), rw.bfloat16().float(), rb, mv.dequant(), k)
        assert torch.allclose(got.float().cpu(), want, atol=3e-2, rtol=3e-2), (M, float((got.float().cpu() - want).abs().max()))
    assert K.status_read()[0] == 0
