"""sm_100a kernels against plain PyTorch fp32 references of the same op (tier T5 of the reference's
test strategy: kernel-vs-host-reference on device).  Shapes exercise every tail path: M in
{1,2,7,8,9,16,17,33,64}, N / K not multiples of the tile, ragged pages."""
import math

import pytest
import torch

from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.formats.w4_tile_layout import interleave_gate_up_q
from grimoire_b200.ops import core as K
from grimoire_b200.ops import ref
from grimoire_b200.ops.linear import BF16Linear, W4Linear, gemm_bf16
from grimoire_b200.ops.workspace import Workspace

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _assert_clean():
    code, detail, n = K.status_read()
    assert code == 0, f"device status: code={code} detail={detail:#x} count={n}"


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("N,Kd,group", [(256, 512, 128), (96, 1024, 64), (2048, 2048, 128)])
def test_smallm_w4_matches_fp32(M, N, Kd, group):
    torch.manual_seed(M * 131 + N)
    w = torch.randn(N, Kd) * 0.02
    qw = quantize(w, Fmt.INT4, group=group)
    lin = W4Linear(qw, DEV, "t", workspace=Workspace(DEV))
    x = (torch.randn(M, Kd) * 0.5).to(DEV).bfloat16()
    want = ref.linear_dequant(x.cpu(), qw.dequant())
    out32 = torch.empty(M, lin.Np, dtype=torch.float32, device=DEV)
    lin(x, out32, "f32")
    got = out32[:, :N].cpu()
    assert torch.allclose(got, want, atol=2e-3, rtol=1e-3), float((got - want).abs().max())
    out16 = torch.empty(M, lin.Np, dtype=torch.bfloat16, device=DEV)
    lin(x, out16, "bf16")
    assert torch.allclose(out16[:, :N].float().cpu(), want, atol=2e-2, rtol=2e-2)
    h = torch.ones(M, lin.Np, dtype=torch.float32, device=DEV)
    lin(x, h, "add_f32")
    assert torch.allclose(h[:, :N].cpu(), want + 1.0, atol=2e-3, rtol=1e-3)
    _assert_clean()


def test_smallm_w4_rows_are_batch_invariant():
    """Row r of a batch is bit-identical to the same row inside any other batch of 2..64 rows (the tensor-core kernel);
    a single row runs on the CUDA-core GEMV, whose fp16 group sums differ from the batch result by rounding only."""
    torch.manual_seed(0)
    qw = quantize(torch.randn(1024, 1024) * 0.02, Fmt.INT4)
    lin = W4Linear(qw, DEV, "t", workspace=Workspace(DEV))
    x = torch.randn(13, 1024, device=DEV).bfloat16()
    full = torch.empty(13, 1024, dtype=torch.float32, device=DEV)
    lin(x, full, "f32")
    for r in (0, 5, 11):
        two = torch.empty(2, 1024, dtype=torch.float32, device=DEV)
        lin(x[r: r + 2], two, "f32")
        assert torch.equal(two[0], full[r]) and torch.equal(two[1], full[r + 1])
        one = torch.empty(1, 1024, dtype=torch.float32, device=DEV)
        lin(x[r: r + 1], one, "f32")
        assert torch.allclose(one[0], full[r], atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("epi", ["f32", "bf16", "add_f32"])
@pytest.mark.parametrize("N,K,group", [(1024, 1024, 128), (96, 192, 64), (5120, 17408, 128), (512, 2048, 256)])
def test_gemv_w4_single_row_matches_dequant(N, K, group, epi):
    """gemv_w4.cu against the fp32 product with the dequantised weight (asymmetric zero points included)."""
    torch.manual_seed(N + K)
    qw = quantize(torch.randn(N, K) * 0.02 + 0.01, Fmt.INT4, group=group)
    lin = W4Linear(qw, DEV, "t", workspace=Workspace(DEV))
    x = torch.randn(1, K, device=DEV).bfloat16()
    want = (x.float().cpu() @ qw.dequant().float().t())
    if epi == "add_f32":
        out = torch.ones(1, lin.Np, dtype=torch.float32, device=DEV)
        want = want + 1.0
    else:
        out = torch.empty(1, lin.Np, dtype=torch.float32 if epi == "f32" else torch.bfloat16, device=DEV)
    lin(x, out, epi)
    tol = 2e-2 if epi == "bf16" else 3e-3
    assert torch.allclose(out[:, :N].float().cpu(), want, atol=tol * max(1.0, float(want.abs().max())), rtol=tol)
    _assert_clean()


@pytest.mark.parametrize("offset", [0.0, 1.0])
def test_gemv_w4_fused_norm_equals_norm_then_gemv(offset):
    """RMSNorm in the GEMV prologue gives the unfused pair's result (same bf16 rounding of the normalised row)."""
    torch.manual_seed(5)
    H, N = 2048, 1024
    qw = quantize(torch.randn(N, H) * 0.02, Fmt.INT4)
    lin = W4Linear(qw, DEV, "t", workspace=Workspace(DEV))
    h = (torch.randn(1, H, device=DEV) * 3.0).contiguous()
    nw = (torch.rand(H, device=DEV) + 0.5).contiguous()
    x = torch.empty(1, H, dtype=torch.bfloat16, device=DEV)
    K.add_rmsnorm(h, nw, x, 1e-6, offset)
    want = torch.empty(1, lin.Np, dtype=torch.float32, device=DEV)
    lin(x, want, "f32")
    got = torch.empty(1, lin.Np, dtype=torch.float32, device=DEV)
    assert lin.fused_norm(h, nw, got, "f32", 1e-6, offset)
    assert torch.allclose(got, want, atol=2e-3 * max(1.0, float(want.abs().max())), rtol=1e-3)
    _assert_clean()


def test_gemv_w4_single_row_swiglu():
    from grimoire_b200.formats.w4_tile_layout import interleave_gate_up_q
    torch.manual_seed(3)
    I, K = 512, 1024
    qg, qu = quantize(torch.randn(I, K) * 0.05, Fmt.INT4), quantize(torch.randn(I, K) * 0.05, Fmt.INT4)
    lin = W4Linear(interleave_gate_up_q(qg, qu), DEV, "gu", swiglu=True, workspace=Workspace(DEV))
    x = torch.randn(1, K, device=DEV).bfloat16()
    xf = x.float().cpu()
    want = torch.nn.functional.silu(xf @ qg.dequant().float().t()) * (xf @ qu.dequant().float().t())
    out = torch.empty(1, I, dtype=torch.bfloat16, device=DEV)
    lin(x, out, "swiglu")
    assert torch.allclose(out.float().cpu(), want, atol=0.012 * max(1.0, float(want.abs().max())), rtol=2e-2)


@pytest.mark.parametrize("M", [1, 8, 24])
def test_smallm_w4_swiglu_and_splitk(M):
    torch.manual_seed(3)
    I, H = 512, 1024
    g = quantize(torch.randn(I, H) * 0.02, Fmt.INT4)
    u = quantize(torch.randn(I, H) * 0.02, Fmt.INT4)
    lin = W4Linear(interleave_gate_up_q(g, u), DEV, "gu", swiglu=True, workspace=Workspace(DEV))
    x = torch.randn(M, H, device=DEV).bfloat16()
    out = torch.empty(M, I, dtype=torch.bfloat16, device=DEV)
    lin(x, out, "swiglu")
    xc = x.cpu()
    want = ref.swiglu(ref.linear_dequant(xc, g.dequant()), ref.linear_dequant(xc, u.dequant()))
    assert torch.allclose(out.float().cpu(), want, atol=3e-3, rtol=2e-2)
    # short-N long-K shape takes the grid split-K path (scratch + counters); run twice: the counters
    # must be back at zero after the first call
    d = quantize(torch.randn(64, 4096) * 0.02, Fmt.INT4)
    ws = Workspace(DEV)
    lind = W4Linear(d, DEV, "d", workspace=ws)
    assert lind._plan_smallm(M)[1] > 1
    xd = torch.randn(M, 4096, device=DEV).bfloat16()
    wantd = ref.linear_dequant(xd.cpu(), d.dequant())
    for _ in range(2):
        od = torch.empty(M, 64, dtype=torch.float32, device=DEV)
        lind(xd, od, "f32")
        assert torch.allclose(od.cpu(), wantd, atol=3e-3, rtol=1e-3)
    assert int(ws.get("smallm_counters", 8192, torch.int32, zero=True).abs().sum()) == 0   # (one row never creates them)
    _assert_clean()


@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (128, 256, 512), (300, 384, 320), (1024, 1280, 1024), (77, 96, 136),
                                    (4096, 512, 256)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_tcgen05_matches_fp32(M, N, Kd, bn):
    torch.manual_seed(M + N + Kd)
    a = (torch.randn(M, Kd, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(N, Kd, device=DEV) * 0.05).bfloat16()
    want = a.float() @ b.float().t()
    out = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    gemm_bf16(a, b, out, "f32", bn=bn)
    _assert_clean()
    err = float((out - want).abs().max())
    assert torch.allclose(out, want, atol=2e-3, rtol=1e-3), err
    o16 = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    gemm_bf16(a, b, o16, "bf16", bn=bn)
    assert torch.allclose(o16.float(), want, atol=3e-2, rtol=2e-2)
    h = torch.full((M, N), 2.0, dtype=torch.float32, device=DEV)
    gemm_bf16(a, b, h, "add_f32", bn=bn)
    assert torch.allclose(h, want + 2.0, atol=2e-3, rtol=1e-3)
    _assert_clean()


def test_gemm_tcgen05_swiglu_and_few_ctas():
    torch.manual_seed(9)
    M, I, H = 256, 512, 384
    a = (torch.randn(M, H, device=DEV) * 0.5).bfloat16()
    g = (torch.randn(I, H, device=DEV) * 0.05).bfloat16()
    u = (torch.randn(I, H, device=DEV) * 0.05).bfloat16()
    from grimoire_b200.formats.w4_tile_layout import interleave_gate_up
    b = interleave_gate_up(g, u).contiguous()
    out = torch.zeros(M, I, dtype=torch.bfloat16, device=DEV)
    # 3 CTAs for 16 tiles: every CTA walks several tiles, exercising both TMEM buffers and phase flips
    gemm_bf16(a, b, out, "swiglu", bn=128, max_ctas=3)
    want = ref.swiglu(a.float() @ g.float().t(), a.float() @ u.float().t())
    assert torch.allclose(out.float(), want, atol=2e-2, rtol=2e-2)
    _assert_clean()


def test_w4_prefill_path_dequant_gemm():
    torch.manual_seed(11)
    N, Kd, M = 512, 1024, 200
    qw = quantize(torch.randn(N, Kd) * 0.02, Fmt.INT4)
    lin = W4Linear(qw, DEV, "p", workspace=Workspace(DEV))
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    out = torch.zeros(M, N, dtype=torch.float32, device=DEV)
    lin(x, out, "f32")
    wbf = qw.dequant().bfloat16().float()     # the GEMM sees bf16-rounded dequantized weights
    want = x.float().cpu() @ wbf.t()
    assert torch.allclose(out.cpu(), want, atol=3e-3, rtol=1e-3)
    _assert_clean()


@pytest.mark.parametrize("M,H", [(1, 256), (5, 5120), (33, 2048)])
def test_add_rmsnorm(M, H):
    torch.manual_seed(1)
    h = torch.randn(M, H, device=DEV)
    d32 = torch.randn(M, H, device=DEV)
    w = torch.randn(H, device=DEV) * 0.1
    for delta, off in ((None, 0.0), (d32, 1.0), (d32.bfloat16(), 1.0)):
        hh = h.clone()
        x = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        K.add_rmsnorm(hh, w, x, 1e-6, off, delta)
        hr = h.clone() if delta is None else h + delta.float()
        want = ref.rmsnorm(hr, w, 1e-6, off)
        assert torch.allclose(hh, hr, atol=1e-6)
        assert torch.allclose(x.float(), want, atol=2e-2, rtol=1e-2)


def test_gemv_bf16_and_argmax_embed():
    torch.manual_seed(2)
    w = torch.randn(1000, 512) * 0.05
    lin = BF16Linear(w, DEV)
    for M in (1, 3, 8):
        x = torch.randn(M, 512, device=DEV).bfloat16()
        out = torch.empty(M, 1000, dtype=torch.float32, device=DEV)
        lin(x, out, "f32")
        want = x.float().cpu() @ w.bfloat16().float().t()
        assert torch.allclose(out.cpu(), want, atol=2e-3, rtol=1e-3)
    logits = torch.randn(4, 151936, device=DEV)
    logits[1, 77] = 50.0
    logits[1, 99999] = 50.0            # tie -> lowest index
    ids = torch.zeros(4, dtype=torch.int32, device=DEV)
    K.argmax_rows(logits, ids)
    assert ids.cpu().tolist() == ref.argmax_lowest(logits.cpu()).tolist() and int(ids[1]) == 77
    table = torch.randn(100, 64, device=DEV).bfloat16()
    tok = torch.tensor([3, 99, 0], dtype=torch.int32, device=DEV)
    h = torch.empty(3, 64, device=DEV)
    K.embed(tok, table, h)
    assert torch.equal(h, table[tok.long()].float())


def _mk_kv(S, max_ctx, Hkv, D):
    pages = S * (max_ctx // 16)
    kv = K.KvLayer.alloc(pages, Hkv, D, DEV)
    table = torch.arange(pages, dtype=torch.int32).reshape(S, max_ctx // 16)
    # shuffle pages so the block table is really used
    perm = torch.randperm(pages)
    table = perm[table.long()].to(torch.int32)
    return kv, table.to(DEV)


@pytest.mark.parametrize("Hq,Hkv,D,rot,gated,qk", [(8, 2, 128, 128, False, False), (4, 2, 64, 64, False, True),
                                                    (16, 2, 256, 64, True, True), (5, 1, 128, 128, False, False)])
def test_rope_kvwrite_and_paged_decode(Hq, Hkv, D, rot, gated, qk):
    torch.manual_seed(5)
    S, max_ctx = 3, 256
    geom = K.AttnGeom(Hq, Hkv, D, rot, 1.0 / math.sqrt(D), gated, 0, 1e-6, 1.0 if qk else 0.0)
    kv, table = _mk_kv(S, max_ctx, Hkv, D)
    kv_c = K.KvLayer(kv.k.cpu(), kv.v.cpu(), kv.ks.cpu(), kv.vs.cpu())
    inv = ref.rope_inv_freq(rot, 1e6)
    qn = (torch.randn(D) * 0.1) if qk else None
    kn = (torch.randn(D) * 0.1) if qk else None
    lens = [37, 200, 16]
    qsz = Hq * D * (2 if gated else 1)
    ws = Workspace(DEV)
    # fill the caches token by token in a few row batches, on both devices
    for start in range(0, max(lens), 50):
        rows = [(s, p) for s in range(S) for p in range(start, min(start + 50, lens[s]))]
        if not rows:
            continue
        M = len(rows)
        qkv = (torch.randn(M, qsz + 2 * Hkv * D) * 0.7).bfloat16()
        rs = torch.tensor([r[0] for r in rows], dtype=torch.int32)
        rp = torch.tensor([r[1] for r in rows], dtype=torch.int32)
        q_g = torch.empty(M, Hq * D, dtype=torch.bfloat16, device=DEV)
        g_g = torch.empty(M, Hq * D, dtype=torch.bfloat16, device=DEV) if gated else None
        K.rope_kvwrite(qkv.to(DEV), rp.to(DEV), rs.to(DEV), table, inv.to(DEV), geom, q_g, kv,
                       None if qn is None else qn.to(DEV), None if kn is None else kn.to(DEV), g_g)
        q_c = torch.empty(M, Hq * D, dtype=torch.bfloat16)
        g_c = torch.empty(M, Hq * D, dtype=torch.bfloat16) if gated else None
        K.rope_kvwrite(qkv, rp, rs, table.cpu(), inv, geom, q_c, kv_c, qn, kn, g_c)
        assert torch.allclose(q_g.float().cpu(), q_c.float(), atol=3e-2, rtol=2e-2)
    # cache contents: int8 codes may differ by one step where rounding sits on a tie; dequantized values agree
    for s in range(S):
        npg = (lens[s] + 15) // 16
        idx = table[s, :npg].long()
        for a, sa, b, sb in ((kv.k, kv.ks, kv_c.k, kv_c.ks), (kv.v, kv.vs, kv_c.v, kv_c.vs)):
            da = (a[idx].float() * sa[idx][..., None]).cpu().permute(0, 2, 1, 3).reshape(npg * 16, Hkv, D)[: lens[s]]
            db = (b[idx.cpu()].float() * sb[idx.cpu()][..., None]).permute(0, 2, 1, 3).reshape(npg * 16, Hkv, D)[: lens[s]]
            assert torch.allclose(da, db, atol=0.05, rtol=0.02)
    # decode rows: last position of each sequence + a 4-row verify block on sequence 1
    rows = [(0, lens[0] - 1), (1, lens[1] - 1), (2, lens[2] - 1)] + [(1, p) for p in range(100, 104)]
    M = len(rows)
    q = (torch.randn(M, Hq * D) * 0.7).bfloat16()
    gate = (torch.randn(M, Hq * D)).bfloat16() if gated else None
    rs = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    rp = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    kv_gc = K.KvLayer(kv.k.cpu(), kv.v.cpu(), kv.ks.cpu(), kv.vs.cpu())    # same cache bytes for the oracle
    want = torch.empty(M, Hq * D, dtype=torch.float32)
    K.paged_decode_attn(q, rs, rp, table.cpu(), kv_gc, geom, want, 1, None, gate)
    for splits in (1, 3, 8):
        out = torch.zeros(M, Hq * D, dtype=torch.bfloat16, device=DEV)
        for _ in range(2):   # twice: split counters must return to zero
            K.paged_decode_attn(q.to(DEV), rs.to(DEV), rp.to(DEV), table, kv, geom, out, splits, ws,
                                None if gate is None else gate.to(DEV))
        assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), (splits, float((out.float().cpu() - want).abs().max()))
    _assert_clean()


@pytest.mark.parametrize("Hq,Hkv,D", [(8, 2, 128), (4, 2, 64), (4, 1, 256), (6, 2, 256)])
@pytest.mark.parametrize("M,pos0,window", [(64, 0, 0), (200, 0, 0), (100, 77, 0), (130, 300, 128), (1024, 512, 0), (700, 333, 256)])
def test_flash_prefill(Hq, Hkv, D, M, pos0, window):
    torch.manual_seed(7)
    T = pos0 + M
    geom = K.AttnGeom(Hq, Hkv, D, D, 1.0 / math.sqrt(D), False, window)
    q = (torch.randn(M, Hq * D) * 0.8).bfloat16()
    k = (torch.randn(T + 5, Hkv * D) * 0.8).bfloat16()
    v = (torch.randn(T + 5, Hkv * D) * 0.8).bfloat16()
    want = torch.empty(M, Hq * D, dtype=torch.float32)
    K.flash_prefill(q, k, v, geom, want, pos0)
    out = torch.zeros(M, Hq * D, dtype=torch.bfloat16, device=DEV)
    K.flash_prefill(q.to(DEV), k.to(DEV), v.to(DEV), geom, out, pos0)
    assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), float((out.float().cpu() - want).abs().max())
    # gated form (output *= sigmoid(gate)): head_dim 128 / 256 take the tensor-core kernel's epilogue, 64 the warp-MMA kernel
    gate = torch.randn(M, Hq * D).bfloat16()
    K.flash_prefill(q, k, v, geom, want, pos0, gate)
    out.zero_()
    K.flash_prefill(q.to(DEV), k.to(DEV), v.to(DEV), geom, out, pos0, gate.to(DEV))
    assert torch.allclose(out.float().cpu(), want, atol=2e-2, rtol=2e-2), float((out.float().cpu() - want).abs().max())


def test_kv_gather_dequant():
    torch.manual_seed(8)
    Hkv, D = 2, 128
    kv, table = _mk_kv(2, 128, Hkv, D)
    kv.k.copy_(torch.randint(-127, 128, kv.k.shape, dtype=torch.int8))
    kv.ks.copy_(torch.rand(kv.ks.shape) * 0.01)
    kv.v.copy_(torch.randint(-127, 128, kv.v.shape, dtype=torch.int8))
    kv.vs.copy_(torch.rand(kv.vs.shape) * 0.01)
    T = 77
    ok = torch.zeros(T, Hkv * D, dtype=torch.bfloat16, device=DEV)
    ov = torch.zeros(T, Hkv * D, dtype=torch.bfloat16, device=DEV)
    K.gather_kv_dense(kv, table[1], T, ok, ov)
    kvc = K.KvLayer(kv.k.cpu(), kv.v.cpu(), kv.ks.cpu(), kv.vs.cpu())
    ck = torch.zeros(T, Hkv * D, dtype=torch.bfloat16)
    cv = torch.zeros(T, Hkv * D, dtype=torch.bfloat16)
    K.gather_kv_dense(kvc, table[1].cpu(), T, ck, cv)
    assert torch.equal(ok.cpu(), ck) and torch.equal(ov.cpu(), cv)


@pytest.mark.parametrize("M", [1, 3, 8, 17, 32])
@pytest.mark.parametrize("N,Kd,group", [(256, 512, 128), (96, 1024, 64), (2048, 2048, 128), (64, 1280, 256)])
def test_smallm_w4_int8_path_matches_fp32(M, N, Kd, group, monkeypatch):
    """The integer activation path (two int8 levels per weight group, exact int32 group sums) against the
    fp32 product of the same bf16 inputs: its activation rounding (15 bits per group) must not cost
    more than the bf16 path's own tolerance."""
    from grimoire_b200.ops import linear as L
    monkeypatch.setattr(L, "W4_I8", True)
    monkeypatch.setattr(L, "GEMV_W4", False)        # a single row would otherwise take the CUDA-core GEMV
    torch.manual_seed(M * 17 + N)
    w = torch.randn(N, Kd) * 0.02
    qw = quantize(w, Fmt.INT4, group=group)
    lin = W4Linear(qw, DEV, "t", workspace=Workspace(DEV))
    x = (torch.randn(M, Kd) * 0.5).to(DEV).bfloat16()
    x[0, 7] = 40.0                      # an outlier inside one group
    want = ref.linear_dequant(x.cpu(), qw.dequant())
    out32 = torch.empty(M, lin.Np, dtype=torch.float32, device=DEV)
    lin(x, out32, "f32")
    got = out32[:, :N].cpu()
    assert torch.allclose(got, want, atol=2e-3, rtol=1e-3), float((got - want).abs().max())
    h = torch.ones(M, lin.Np, dtype=torch.float32, device=DEV)
    lin(x, h, "add_f32")
    assert torch.allclose(h[:, :N].cpu(), want + 1.0, atol=2e-3, rtol=1e-3)
    one = torch.empty(1, lin.Np, dtype=torch.float32, device=DEV)
    lin(x[M - 1: M], one, "f32")
    assert torch.equal(one[0], out32[M - 1])            # batch invariant
    _assert_clean()


@pytest.mark.parametrize("M", [1, 5, 24])
def test_fused_allreduce_epilogues_with_one_rank(M):
    """The all-reducing epilogues (gemv_w4 for one row, smallm_w4 for more) with a world of one rank: the exchange
    degenerates to this rank's own {value, epoch} slots, the result is the plain accumulate.  Three launches in a row
    exercise both parities and the epoch counters; the multi-rank form runs in the 2-GPU tests."""
    import ctypes
    from grimoire_b200 import _native

    torch.manual_seed(M)
    N, Kd = 1024, 2048
    qw = quantize(torch.randn(N, Kd) * 0.02, Fmt.INT4)
    lin = W4Linear(qw, DEV, "t", workspace=Workspace(DEV))
    t = lin.tiled
    tiles = N // 16
    half = tiles * 2048                                   # floats per parity half of the small-M exchange (world 1)
    recv = torch.zeros(2 * half + 2 * tiles * 32, dtype=torch.float32, device=DEV)
    flags = torch.zeros(tiles, dtype=torch.int32, device=DEV)
    epochs = torch.zeros(tiles, dtype=torch.int32, device=DEV)
    x = torch.randn(M, Kd, device=DEV).bfloat16()
    want = torch.ones(M, N, dtype=torch.float32, device=DEV)
    h = torch.ones(M, N, dtype=torch.float32, device=DEV)
    rp = (ctypes.c_void_p * 1)(recv.data_ptr())
    fp = (ctypes.c_void_p * 1)(flags.data_ptr())
    c = ctypes.c_int
    lib = _native.cuda()
    for _ in range(3):
        lin(x, want, "add_f32")
        if M == 1:
            code = lib.grm_gemv_w4_allreduce(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(h), c(t.N), c(t.K),
                                             c(t.group), rp, ctypes.c_long(2 * half), fp, _native.ptr(epochs), c(1), c(0),
                                             ctypes.c_uint(0), _native.stream_ptr())
        else:
            code = lib.grm_smallm_w4_allreduce(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(h), c(M), c(t.N),
                                               c(t.K), c(x.stride(0)), c(h.stride(0)), c(t.group), rp, fp, _native.ptr(epochs), c(1),
                                               c(0), ctypes.c_uint(0), _native.stream_ptr())
        _native.check(code, "fused allreduce, one rank")
    assert torch.allclose(h, want, atol=2e-3, rtol=1e-3)
    assert int(epochs.min()) == 3 and int(epochs.max()) == 3
    _assert_clean()


@pytest.mark.parametrize("Hq,Hkv,D,rot,qk_norm", [(10, 2, 128, 128, True), (8, 2, 128, 64, False), (4, 2, 64, 64, True), (4, 1, 256, 64, True)])
@pytest.mark.parametrize("splits", [1, 4])
def test_decode_attn_with_fused_rope_kv_append_equals_two_kernels(Hq, Hkv, D, rot, qk_norm, splits):
    """q/k norm + RoPE + KV append inside the decode attention kernel against rope_kvwrite followed by the attention
    kernel: same arithmetic, so the appended cache bytes and the outputs are equal bit for bit.  Positions include a
    page boundary (first slot of a new page) and the last slot of a page."""
    torch.manual_seed(D + Hq)
    S, pages_per = 3, 12
    geom = K.AttnGeom(Hq, Hkv, D, rot, 1.0 / math.sqrt(D), False, 0, 1e-6, 0.0)
    inv = ref.rope_inv_freq(rot, 10000.0).to(DEV)
    qn = (torch.rand(D) + 0.5).to(DEV) if qk_norm else None
    kn = (torch.rand(D) + 0.5).to(DEV) if qk_norm else None
    table = torch.arange(S * pages_per, dtype=torch.int32).reshape(S, pages_per).to(DEV)
    ws = Workspace(DEV)

    def filled():
        kv = K.KvLayer.alloc(S * pages_per, Hkv, D, DEV)
        g = torch.Generator().manual_seed(1)
        for s, n in enumerate((150, 96, 47)):
            qkv = (torch.randn(n, (Hq + 2 * Hkv) * D, generator=g) * 0.7).bfloat16().to(DEV)
            rs = torch.full((n,), s, dtype=torch.int32, device=DEV)
            rp = torch.arange(n, dtype=torch.int32, device=DEV)
            K.rope_kvwrite(qkv, rp, rs, table, inv, geom, torch.empty(n, Hq * D, dtype=torch.bfloat16, device=DEV), kv, qn, kn, None)
        return kv

    kv_a, kv_b = filled(), filled()
    for s, pos in ((0, 150), (1, 96), (2, 47), (0, 151)):      # 96 opens a new page, 47 is a page's last slot
        qkv = (torch.randn(1, (Hq + 2 * Hkv) * D) * 0.7).bfloat16().to(DEV)
        rs = torch.tensor([s], dtype=torch.int32, device=DEV)
        rp = torch.tensor([pos], dtype=torch.int32, device=DEV)
        q = torch.empty(1, Hq * D, dtype=torch.bfloat16, device=DEV)
        want = torch.zeros(1, Hq * D, dtype=torch.bfloat16, device=DEV)
        K.rope_kvwrite(qkv, rp, rs, table, inv, geom, q, kv_a, qn, kn, None)
        K.paged_decode_attn(q, rs, rp, table, kv_a, geom, want, splits, ws, None)
        got = torch.zeros(1, Hq * D, dtype=torch.bfloat16, device=DEV)
        assert K.paged_decode_attn_fused(qkv, inv, qn, kn, rs, rp, table, kv_b, geom, got, splits, ws)
        assert torch.equal(got, want), float((got.float() - want.float()).abs().max())
    # three rows of three different sequences in one launch
    qkv = (torch.randn(3, (Hq + 2 * Hkv) * D) * 0.7).bfloat16().to(DEV)
    rs = torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV)
    rp = torch.tensor([152, 97, 48], dtype=torch.int32, device=DEV)
    q = torch.empty(3, Hq * D, dtype=torch.bfloat16, device=DEV)
    want = torch.zeros(3, Hq * D, dtype=torch.bfloat16, device=DEV)
    K.rope_kvwrite(qkv, rp, rs, table, inv, geom, q, kv_a, qn, kn, None)
    K.paged_decode_attn(q, rs, rp, table, kv_a, geom, want, splits, ws, None)
    got = torch.zeros(3, Hq * D, dtype=torch.bfloat16, device=DEV)
    assert K.paged_decode_attn_fused(qkv, inv, qn, kn, rs, rp, table, kv_b, geom, got, splits, ws)
    assert torch.equal(got, want)
    for a, b in ((kv_a.k, kv_b.k), (kv_a.v, kv_b.v), (kv_a.ks, kv_b.ks), (kv_a.vs, kv_b.vs)):
        assert torch.equal(a, b)
    _assert_clean()


def test_out_of_range_token_id_is_reported_not_read():
    """A token id outside the vocabulary gives a zero row and GRM_ERR_BOUNDS in the status block; nothing is read."""
    table = torch.randn(100, 64, device=DEV).bfloat16()
    ids = torch.tensor([3, 100, -1, 99], dtype=torch.int32, device=DEV)
    h = torch.full((4, 64), 7.0, device=DEV)
    K.embed(ids, table, h)
    torch.cuda.synchronize()
    code, detail, n = K.status_read()
    assert code == 3 and n == 2 and (detail & 0xffff) in (1, 2)
    assert torch.equal(h[0], table[3].float()) and torch.equal(h[3], table[99].float())
    assert float(h[1].abs().max()) == 0.0 and float(h[2].abs().max()) == 0.0
    _assert_clean()


@pytest.mark.parametrize("N,K,group", [(256, 5120, 128), (5120, 17408, 128), (512, 2048, 64)])
@pytest.mark.parametrize("xmax", [1.0e3, 3.0e3, 2.0e-2])
def test_gemv_w4_single_row_survives_outlier_activations(N, K, group, xmax):
    """A few columns of |x| ~ 1e3 .. 1e4 (routine for down_proj inputs of real checkpoints), or tiny activations overall: the
    fp16 partial sums must neither overflow nor lose the small columns (the reference accumulates its GEMV in fp32,
    src/gemv_decode.cpp:77-347).  Beyond |x| = 3840 the staged value saturates: the result stays finite."""
    torch.manual_seed(N + K)
    qw = quantize(torch.randn(N, K) * 0.02 + 0.004, Fmt.INT4, group=group)
    lin = W4Linear(qw, DEV, "t", workspace=Workspace(DEV))
    x = torch.randn(1, K) * (xmax / 30 if xmax < 1 else 1.0)
    if xmax >= 1:
        x[0, 5] = xmax
        x[0, K // 2 + 3] = -0.8 * xmax
        x[0, K - 9] = 0.5 * xmax
    x = x.to(DEV).bfloat16()
    want = x.float().cpu() @ qw.dequant().float().t()
    out = torch.empty(1, lin.Np, dtype=torch.float32, device=DEV)
    lin(x, out, "f32")
    got = out[:, :N].cpu()
    assert torch.isfinite(got).all()
    tol = 2e-3 * float(want.abs().max()) + 1e-6
    assert float((got - want).abs().max()) < tol, (float((got - want).abs().max()), tol)
    # the fused-norm prologue takes the same path with its own scale
    h = (torch.randn(1, K) * (1.0 if xmax >= 1 else xmax)).to(DEV)
    if xmax >= 1:
        h[0, 7] = xmax
    nw = torch.ones(K, device=DEV)
    if lin.fused_norm(h, nw, out, "f32", 1e-6, 0.0):
        xn = (h * torch.rsqrt((h * h).mean() + 1e-6)).bfloat16().float().cpu()
        want = xn @ qw.dequant().float().t()
        got = out[:, :N].cpu()
        assert float((got - want).abs().max()) < 2e-3 * float(want.abs().max()) + 1e-6
    _assert_clean()


def test_gemv_w4_single_row_saturates_instead_of_overflowing():
    torch.manual_seed(1)
    qw = quantize(torch.randn(256, 2048) * 0.02, Fmt.INT4)
    lin = W4Linear(qw, DEV, "t", workspace=Workspace(DEV))
    x = torch.randn(1, 2048)
    x[0, 11] = 3.0e5
    x[0, 400] = -2.0e5
    out = torch.empty(1, lin.Np, dtype=torch.float32, device=DEV)
    lin(x.to(DEV).bfloat16(), out, "f32")
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("Hq,Hkv,D,gated,window", [(40, 8, 128, False, 0), (32, 8, 128, False, 0), (8, 8, 64, False, 0),
                                                     (16, 2, 256, True, 0), (8, 2, 128, False, 64)])
def test_verify_attention_one_pass_equals_row_wise(Hq, Hkv, D, gated, window):
    """A verify block's rows x the GQA group's heads as MMA rows, one pass over the pages per group of rows
    (attn_verify.cu), against the per-row kernel on the same cache: causal inside the block, several blocks and a
    single row in one launch, with and without split-KV (launch_verify_attn_dpas, src/attn_verify.hpp:48-69)."""
    torch.manual_seed(9)
    S, max_ctx = 3, 512
    geom = K.AttnGeom(Hq, Hkv, D, min(D, 128), 1.0 / math.sqrt(D), gated, window, 1e-6, 0.0)
    kv, table = _mk_kv(S, max_ctx, Hkv, D)
    kv.k.random_(-127, 127)
    kv.v.random_(-127, 127)
    kv.ks.uniform_(0.005, 0.02)
    kv.vs.uniform_(0.005, 0.02)
    per = K.verify_rows_per_group(geom)
    assert per == 16 // (Hq // Hkv)
    # a 5-row block on sequence 1 near a page boundary, a 2-row block on sequence 0, one plain row on sequence 2
    rows = [(1, p) for p in range(300, 305)] + [(0, 14), (0, 15)] + [(2, 499)]
    M = len(rows)
    groups = K.verify_groups([r[0] for r in rows], [r[1] for r in rows], per)
    assert sum(g[2] for g in groups) == M and all(g[2] <= per for g in groups)
    blocks = torch.tensor(groups, dtype=torch.int32).t().contiguous().to(DEV)
    q = (torch.randn(M, Hq * D) * 0.7).bfloat16().to(DEV)
    gate = torch.randn(M, Hq * D).bfloat16().to(DEV) if gated else None
    rs = torch.tensor([r[0] for r in rows], dtype=torch.int32, device=DEV)
    rp = torch.tensor([r[1] for r in rows], dtype=torch.int32, device=DEV)
    ws = Workspace(DEV)
    want = torch.zeros(M, Hq * D, dtype=torch.bfloat16, device=DEV)
    K.paged_decode_attn(q, rs, rp, table, kv, geom, want, 1, ws, gate)
    for splits in (1, 4):
        out = torch.zeros(M, Hq * D, dtype=torch.bfloat16, device=DEV)
        assert K.paged_verify_attn(q, blocks, len(groups), table, kv, geom, out, splits, ws, gate)
        err = float((out.float() - want.float()).abs().max())
        assert err < 2e-2 * max(1.0, float(want.float().abs().max())), (splits, err)
    _assert_clean()
