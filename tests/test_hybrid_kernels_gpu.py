"""Gated DeltaNet and MoE kernels against their fp32 oracles (same wrapper, CPU tensors)."""
import pytest
import torch

from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.ops import hybrid as Hb

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rows(spec):
    """spec: list of (slot, first_pos, n) -> row_seq, row_pos, runs"""
    rs, rp, runs, m = [], [], [], 0
    for slot, p0, n in spec:
        rs += [slot] * n
        rp += list(range(p0, p0 + n))
        runs.append((slot, m, n))
        m += n
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    return i32(rs), i32(rp), i32([r[0] for r in runs]), i32([r[1] for r in runs]), i32([r[2] for r in runs])


@pytest.mark.parametrize("spec", [[(0, 0, 70)], [(2, 5, 1), (0, 9, 1), (1, 3, 1)], [(1, 4, 3), (0, 0, 40), (2, 100, 1)]])
def test_conv4_silu_matches_oracle(spec):
    torch.manual_seed(0)
    C_, slots = 512, 3
    rs, rp, _, _, _ = _rows(spec)
    M = rs.shape[0]
    x = (torch.randn(M, C_) * 0.7).bfloat16()
    w = torch.randn(C_, 4) * 0.5
    ring = torch.randn(slots, C_, 3)
    y_ref = torch.zeros(M, C_, dtype=torch.bfloat16)
    ring_ref = ring.clone()
    Hb.conv4_silu(x, w, ring_ref, None, rs, rp, y_ref, None)
    y = torch.zeros(M, C_, dtype=torch.bfloat16, device=DEV)
    ring_g, tmp = ring.clone().to(DEV), torch.zeros_like(ring).to(DEV)
    touched = torch.tensor(sorted({s for s, _, _ in spec}), device=DEV)
    Hb.conv4_silu(x.to(DEV), w.to(DEV), ring_g, tmp, rs.to(DEV), rp.to(DEV), y, touched)
    assert torch.allclose(y.float().cpu(), y_ref.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(ring_g.cpu(), ring_ref, atol=1e-6)


@pytest.mark.parametrize("spec", [[(0, 0, 70)], [(1, 7, 1), (0, 3, 1)], [(2, 0, 5), (0, 10, 1)]])
def test_gdn_runs_match_sequential_oracle(spec):
    torch.manual_seed(1)
    Hk, Hv, D = 2, 4, 128
    rs, rp, run_slot, run_start, run_len = _rows(spec)
    M = rs.shape[0]
    qkv = (torch.randn(M, 2 * Hk * D + Hv * D) * 0.5).bfloat16()
    ab = torch.randn(M, 2 * Hv)
    z = torch.randn(M, Hv * D).bfloat16()
    A_log, dt_bias, nw = torch.randn(Hv) * 0.5, torch.randn(Hv) * 0.5, 1 + 0.1 * torch.randn(D)
    state = torch.randn(3, Hv, D, D) * 0.1
    out_ref = torch.zeros(M, Hv * D, dtype=torch.bfloat16)
    st_ref = state.clone()
    Hb.gdn_runs(qkv, ab, z, A_log, dt_bias, nw, 1e-6, st_ref, run_slot, run_start, run_len, out_ref, Hk, Hv, D, D)
    out = torch.zeros(M, Hv * D, dtype=torch.bfloat16, device=DEV)
    st = state.clone().to(DEV)
    Hb.gdn_runs(qkv.to(DEV), ab.to(DEV), z.to(DEV), A_log.to(DEV), dt_bias.to(DEV), nw.to(DEV), 1e-6, st, run_slot.to(DEV),
                run_start.to(DEV), run_len.to(DEV), out, Hk, Hv, D, D)
    assert torch.allclose(out.float().cpu(), out_ref.float(), atol=3e-2, rtol=3e-2), float((out.float().cpu() - out_ref.float()).abs().max())
    assert torch.allclose(st.cpu(), st_ref, atol=2e-3, rtol=2e-3)


def test_moe_route_softmax_topk_renorm_and_ties():
    torch.manual_seed(2)
    M, E, k = 33, 512, 10
    lg = torch.randn(M, E + 1)
    lg[0, 7] = lg[0, 300] = 8.0            # tie -> lower index first
    ids_r, w_r = torch.zeros(M, k, dtype=torch.int32), torch.zeros(M, k)
    Hb.moe_route(lg, E, k, True, ids_r, w_r)
    ids, w = torch.zeros(M, k, dtype=torch.int32, device=DEV), torch.zeros(M, k, device=DEV)
    cnt = torch.zeros(E, dtype=torch.int32, device=DEV)
    Hb.moe_route(lg.to(DEV), E, k, True, ids, w, cnt)
    assert torch.equal(ids.cpu(), ids_r) and ids_r[0, 0] == 7 and ids_r[0, 1] == 300
    assert torch.allclose(w.cpu(), w_r, atol=1e-5) and torch.allclose(w.sum(-1).cpu(), torch.ones(M), atol=1e-5)
    assert int(cnt.sum()) == M * k


@pytest.mark.parametrize("M", [1, 5, 16, 37])
def test_grouped_gemm_fp8_modes(M):
    torch.manual_seed(3)
    E, I, H = 4, 128, 256
    wgu = torch.randn(E, 2 * I, H) * 0.05
    q = [quantize(wgu[e], Fmt.FP8_BLOCK) for e in range(E)]
    w8 = torch.stack([t.payload for t in q])
    sc = torch.stack([t.scales for t in q])
    x = (torch.randn(M, H) * 0.5).bfloat16()
    # rows grouped by expert: expert of grouped row r = r % E, source row = r
    order = sorted(range(M), key=lambda r: (r % E, r))
    row_ids = torch.tensor(order, dtype=torch.int32)
    tiles = []
    r0 = 0
    for e in range(E):
        n = len([r for r in order if r % E == e])
        while n > 0:
            tiles.append((e, r0, min(16, n)))
            r0 += min(16, n)
            n -= 16
    te, t0, tn = (torch.tensor([t[i] for t in tiles], dtype=torch.int32) for i in range(3))
    for mode, shape, dt in (("swiglu", (M, I), torch.bfloat16), ("f32", (M, 2 * I), torch.float32), ("bf16", (M, 2 * I), torch.bfloat16)):
        ref = torch.zeros(shape, dtype=dt)
        Hb.grouped_gemm_fp8(x, row_ids, te, t0, tn, w8, sc, ref, mode)
        out = torch.zeros(shape, dtype=dt, device=DEV)
        Hb.grouped_gemm_fp8(x.to(DEV), row_ids.to(DEV), te.to(DEV), t0.to(DEV), tn.to(DEV), w8.to(DEV), sc.to(DEV), out, mode)
        assert torch.allclose(out.float().cpu(), ref.float(), atol=2e-2, rtol=2e-2), (mode, float((out.float().cpu() - ref.float()).abs().max()))
    lin = Hb.FP8BlockLinear(wgu[0], DEV)
    out = torch.ones(M, 2 * I, dtype=torch.float32, device=DEV)
    lin(x.to(DEV), out, "add_f32")
    ref = torch.ones(M, 2 * I)
    Hb.FP8BlockLinear(wgu[0], "cpu")(x, ref, "add_f32")
    assert torch.allclose(out.cpu(), ref, atol=2e-2, rtol=2e-2)


def test_moe_combine_is_slot_ordered():
    torch.manual_seed(4)
    M, slots, H = 9, 5, 256
    y = torch.randn(M * slots, H)
    pos = torch.randperm(M * slots).reshape(M, slots).to(torch.int32)
    pos[2, 3] = -1
    w = torch.rand(M, slots)
    h_ref = torch.randn(M, H)
    h = h_ref.clone().to(DEV)
    Hb.moe_combine(h_ref, y, pos, w)
    Hb.moe_combine(h, y.to(DEV), pos.to(DEV), w.to(DEV))
    assert torch.allclose(h.cpu(), h_ref, atol=1e-5)


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("H,I", [(256, 128), (640, 256), (2048, 512)])
def test_grouped_gemv_fp8_small_rows(M, H, I):
    """The weight-streaming GEMV form (tiles of at most 8 rows) against the CPU oracle: one tile per
    (row, expert) pair as in a decode step, and one dense tile of M rows."""
    torch.manual_seed(M * 11 + H)
    E = 4
    wgu = torch.randn(E, 2 * I, H) * 0.05
    q = [quantize(wgu[e], Fmt.FP8_BLOCK) for e in range(E)]
    w8, sc = torch.stack([t.payload for t in q]), torch.stack([t.scales for t in q])
    x = (torch.randn(M, H) * 0.5).bfloat16()
    k = 2
    pairs = M * k
    te = torch.tensor([(r * 3 + j) % E for r in range(M) for j in range(k)], dtype=torch.int32)
    t0 = torch.arange(pairs, dtype=torch.int32)
    tn = torch.ones(pairs, dtype=torch.int32)
    src = (t0 // k).to(torch.int32)
    for mode, shape, dt in (("swiglu", (pairs, I), torch.bfloat16), ("f32", (pairs, 2 * I), torch.float32), ("bf16", (pairs, 2 * I), torch.bfloat16)):
        ref = torch.zeros(shape, dtype=dt)
        Hb.grouped_gemm_fp8(x, src, te, t0, tn, w8, sc, ref, mode)
        out = torch.zeros(shape, dtype=dt, device=DEV)
        Hb.grouped_gemm_fp8(x.to(DEV), src.to(DEV), te.to(DEV), t0.to(DEV), tn.to(DEV), w8.to(DEV), sc.to(DEV), out, mode, small=True)
        err = float((out.float().cpu() - ref.float()).abs().max())
        assert err < 2e-2 * max(1.0, float(ref.float().abs().max())), (mode, err)
    lin, cpu = Hb.FP8BlockLinear(wgu[1], DEV), Hb.FP8BlockLinear(wgu[1], "cpu")
    out = torch.ones(M, 2 * I, dtype=torch.float32, device=DEV)
    lin(x.to(DEV), out, "add_f32")
    ref = torch.ones(M, 2 * I)
    cpu(x, ref, "add_f32")
    assert torch.allclose(out.cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M", [65, 200])
def test_fp8_block_linear_tall_inputs_use_dequant_gemm(M):
    """More than 64 rows: dequantise once + tcgen05 GEMM (bf16 rounding of the dequantised weights)."""
    torch.manual_seed(M)
    N, H = 512, 384
    w = torch.randn(N, H) * 0.05
    x = (torch.randn(M, H) * 0.5).bfloat16()
    lin, cpu = Hb.FP8BlockLinear(w, DEV), Hb.FP8BlockLinear(w, "cpu")
    for epi, shape, dt in (("bf16", (M, N), torch.bfloat16), ("f32", (M, N), torch.float32), ("swiglu", (M, N // 2), torch.bfloat16)):
        ref = torch.zeros(shape, dtype=dt)
        cpu(x, ref, epi)
        out = torch.zeros(shape, dtype=dt, device=DEV)
        lin(x.to(DEV), out, epi)
        err = float((out.float().cpu() - ref.float()).abs().max())
        assert err < 3e-2 * max(1.0, float(ref.float().abs().max())), (epi, err)
    out = torch.ones(M, N, dtype=torch.float32, device=DEV)
    lin(x.to(DEV), out, "add_f32")
    ref = torch.ones(M, N)
    cpu(x, ref, "add_f32")
    assert torch.allclose(out.cpu(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("lens", [[64], [200], [37, 130], [1, 64, 65]])
def test_gdn_chunked_matches_sequential_oracle(lens):
    """The 64-token chunked form (UT-transform of the gated delta rule) against the token-by-token fp32
    oracle: outputs, final state, partial last chunks, several runs with different slots."""
    torch.manual_seed(sum(lens))
    Hk, Hv, D = 2, 4, 128
    M = sum(lens)
    run_slot = torch.tensor([(2 * i + 1) % 3 for i in range(len(lens))], dtype=torch.int32)
    run_len = torch.tensor(lens, dtype=torch.int32)
    run_start = (torch.cumsum(run_len, 0) - run_len).to(torch.int32)
    qkv = (torch.randn(M, 2 * Hk * D + Hv * D) * 0.5).bfloat16()
    ab = torch.randn(M, 2 * Hv)
    z = torch.randn(M, Hv * D).bfloat16()
    A_log, dt_bias, nw = torch.randn(Hv) * 0.5, torch.randn(Hv) * 0.5, 1 + 0.1 * torch.randn(D)
    state = torch.randn(3, Hv, D, D) * 0.1
    out_ref = torch.zeros(M, Hv * D, dtype=torch.bfloat16)
    st_ref = state.clone()
    Hb.gdn_runs(qkv, ab, z, A_log, dt_bias, nw, 1e-6, st_ref, run_slot, run_start, run_len, out_ref, Hk, Hv, D, D)
    out = torch.zeros(M, Hv * D, dtype=torch.bfloat16, device=DEV)
    st = state.clone().to(DEV)
    Hb.gdn_runs(qkv.to(DEV), ab.to(DEV), z.to(DEV), A_log.to(DEV), dt_bias.to(DEV), nw.to(DEV), 1e-6, st, run_slot.to(DEV),
                run_start.to(DEV), run_len.to(DEV), out, Hk, Hv, D, D, chunked=True)
    assert torch.allclose(out.float().cpu(), out_ref.float(), atol=3e-2, rtol=3e-2), float((out.float().cpu() - out_ref.float()).abs().max())
    assert torch.allclose(st.cpu(), st_ref, atol=2e-3, rtol=2e-3), float((st.cpu() - st_ref).abs().max())


@pytest.mark.parametrize("M", [1, 3, 8])
def test_ep_decode_tiles_and_allreducing_combine_single_rank(M):
    """The expert-parallel decode route with one rank owning experts [0, E): tiles from replicated choices (a choice
    outside the range becomes an empty tile and a skipped slot), then the combine kernel whose all-reduce over one
    rank is the plain slot-ordered combine.  Run twice: the epoch counters carry over between launches."""
    from grimoire_b200.parallel.ep import ExpertParallel

    torch.manual_seed(M)
    E, k, H, I = 16, 4, 512, 128
    ep = ExpertParallel(None, DEV, E, k, H, I, max_rows=8, fused=True)
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(M)]).to(torch.int32)
    ep.E_loc = 12                                   # pretend experts 12..15 live elsewhere
    te, nr, pos = ep.decode_tiles(ids.to(DEV), M)
    local = ids < 12
    flat = torch.arange(M * k, dtype=torch.int32).reshape(M, k)
    assert torch.equal(te.cpu().reshape(M, k), torch.where(local, ids, torch.zeros_like(ids)))
    assert torch.equal(nr.cpu().reshape(M, k), local.to(torch.int32))
    assert torch.equal(pos.cpu()[:, :k], torch.where(local, flat, torch.full_like(flat, -1)))
    assert torch.equal(pos.cpu()[:, k], torch.arange(M * k, M * (k + 1), dtype=torch.int32))
    y = torch.randn(M * (k + 1), H)
    w = torch.rand(M, k + 1)
    h_ref = torch.randn(M, H)
    h = h_ref.clone().to(DEV)
    for _ in range(2):
        Hb.moe_combine(h_ref, y, pos.cpu(), w)
        ep.combine_allreduce(h, y.to(DEV), pos, w.to(DEV), M)
    assert torch.allclose(h.cpu(), h_ref, atol=1e-5)
    from grimoire_b200.ops import core as K
    assert K.status_read()[0] == 0
