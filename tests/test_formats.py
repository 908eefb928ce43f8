"""Codec / quantizer / layout properties (host only), in the style of the reference's
tests/test_formats.cpp and tests/test_gptq.cpp: bit-exact round trips and documented conventions."""
import pytest
import torch

from grimoire_b200.formats import codecs as C
from grimoire_b200.formats import gptq
from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.formats.w4_tile_layout import interleave_gate_up, tile_w4, untile_w4


def test_e2m1_roundtrip_all_codes():
    codes = torch.arange(16, dtype=torch.uint8)
    vals = C.e2m1_to_f32(codes)
    back = C.f32_to_e2m1(vals)
    # -0 encodes as 8; everything else is the identity
    assert torch.equal(back, codes)


def test_e2m1_rounding_ties_to_even_and_saturation():
    x = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 100.0, -100.0, 0.26, 0.74])
    got = C.e2m1_to_f32(C.f32_to_e2m1(x))
    want = torch.tensor([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0, 6.0, -6.0, 0.5, 0.5])
    assert torch.equal(got, want)


def test_e8m0_and_pick():
    e = torch.tensor([0, 126, 127, 128, 254], dtype=torch.uint8)
    assert torch.equal(C.e8m0_to_f32(e), torch.tensor([2.0 ** -127, 0.5, 1.0, 2.0, 2.0 ** 127]))
    # amax 6 with emax 2 -> scale 1; amax 12 -> 2; exact powers of two do not slip
    assert C.pick_e8m0(torch.tensor([6.0, 12.0, 4.0, 3.99, 448.0]), 2).tolist() == [127, 128, 127, 126, 133]


def test_bf16_bits_rne():
    x = torch.tensor([1.0, 1.00390625, 1.01171875, -2.5, 3.140625])
    bits = C.f32_to_bf16_bits(x)
    assert torch.equal(C.bf16_bits_to_f32(bits), x.bfloat16().float())


@pytest.mark.parametrize("fmt,tol", [(Fmt.INT8, 0.01), (Fmt.FP8_E4M3, 0.07), (Fmt.FP8_E5M2, 0.15), (Fmt.INT4, 0.2),
                                     (Fmt.MXFP4, 0.3), (Fmt.MXFP8, 0.07), (Fmt.FP8_BLOCK, 0.07), (Fmt.NVFP4, 0.3),
                                     (Fmt.BF16, 0.005)])
def test_quantize_error_bounds(fmt, tol):
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.02
    qw = quantize(w, fmt)
    d = qw.dequant()
    assert d.shape == w.shape
    rel = (d - w).norm() / w.norm()
    assert rel < tol, (fmt, float(rel))


def test_int4_symmetric_zero_is_8_and_search_not_worse():
    torch.manual_seed(1)
    w = torch.randn(32, 256) * 0.02
    s = quantize(w, Fmt.INT4, symmetric=True)
    assert int(s.zeros.min()) == 8 and int(s.zeros.max()) == 8
    a = quantize(w, Fmt.INT4)
    b = quantize(w, Fmt.INT4, search=True)
    assert (b.dequant() - w).norm() <= (a.dequant() - w).norm() + 1e-7


def test_gptq_triple_roundtrip_and_plus_one_zero():
    torch.manual_seed(2)
    w = torch.randn(64, 256) * 0.02
    qw = quantize(w, Fmt.INT4, group=128)
    qweight, qzeros, scales = gptq.gptq_pack(qw)
    assert qweight.shape == (256 // 8, 64) and qzeros.shape == (2, 8) and scales.shape == (2, 64)
    assert gptq.gptq_group_size(qweight, scales) == 128
    back = gptq.gptq_unpack(qweight, qzeros, scales)
    assert torch.equal(back.payload, qw.payload) and torch.equal(back.zeros, qw.zeros)
    assert torch.equal(back.dequant(), qw.dequant())
    # the stored zero code is zero-1: decoding without the +1 must NOT reproduce the weights
    z_raw = gptq._unpack_i32_nibbles(qzeros, 1)[:, :64].t()
    assert not torch.equal(z_raw.to(torch.uint8), qw.zeros)


def test_gptq_rejects_act_order():
    torch.manual_seed(3)
    qw = quantize(torch.randn(32, 256), Fmt.INT4)
    a, b, c = gptq.gptq_pack(qw)
    g_idx = torch.arange(256) // 128
    gptq.gptq_unpack(a, b, c, g_idx)
    with pytest.raises(ValueError):
        gptq.gptq_unpack(a, b, c, g_idx.flip(0))


@pytest.mark.parametrize("N,K,group", [(32, 128, 128), (96, 256, 64), (50, 512, 256)])
def test_w4_tile_roundtrip_and_element_map(N, K, group):
    torch.manual_seed(4)
    qw = quantize(torch.randn(N, K) * 0.05, Fmt.INT4, group=group)
    t = tile_w4(qw)
    assert t.N % 32 == 0 and t.w.shape == (t.N // 32, K // 64, 2, 32, 4)
    back = untile_w4(t)
    assert torch.equal(back.payload[:N], qw.payload)
    assert torch.equal(back.scales[:N], qw.scales) and torch.equal(back.zeros[:N], qw.zeros)
    q = C.unpack_nibbles(qw.payload)
    gen = torch.Generator().manual_seed(5)
    for _ in range(64):
        ns, kt, half, lane, j, i = [int(torch.randint(0, hi, (1,), generator=gen)) for hi in
                                    (t.N // 32, K // 64, 2, 32, 4, 8)]
        row = 16 * (2 * ns + half) + lane // 4 + 8 * (i & 1)
        k = 64 * kt + 16 * (lane % 4) + 4 * j + 2 * ((i >> 1) & 1) + (i >> 2)
        word = int(t.w[ns, kt, half, lane, j]) & 0xFFFFFFFF
        want = int(q[row, k]) if row < N else 8
        assert (word >> (4 * i)) & 0xF == want


def test_gate_up_interleave():
    g = torch.arange(32).float()[:, None].expand(32, 4)
    u = g + 100
    f = interleave_gate_up(g, u)
    assert f[:16, 0].tolist() == list(range(16)) and f[16:32, 0].tolist() == [100 + i for i in range(16)]
    assert f[32:48, 0].tolist() == list(range(16, 32))


def test_gptq_stored_zero_15_means_16():
    """AutoGPTQ stores zero - 1; a stored nibble of 15 is the zero point 16, not 0 (the reference dequantises with
    znib + 1 without wrapping, src/gptq.cpp:44)."""
    import torch
    from grimoire_b200.formats import gptq

    K, N, g = 128, 8, 128
    codes = torch.randint(0, 16, (K, N))
    qweight = gptq._pack_i32_nibbles(codes, 0)                       # [K/8][N]
    zc = torch.tensor([[15, 0, 7, 15, 3, 14, 15, 8]])                # stored zero - 1 per output column
    qzeros = gptq._pack_i32_nibbles(zc, 1)                           # [1][N/8]
    scales = (torch.rand(1, N) * 0.01 + 0.001).half()
    qw = gptq.gptq_unpack(qweight, qzeros, scales)
    assert qw.zeros[:, 0].tolist() == [16, 1, 8, 16, 4, 15, 16, 9]
    want = (codes.t().float() - (zc[0].float() + 1)[:, None]) * scales[0].float()[:, None]
    assert torch.allclose(qw.dequant(), want, atol=1e-7)
    a, b, c = gptq.gptq_pack(qw)
    assert torch.equal(b, qzeros) and torch.equal(a, qweight)


def test_safetensors_rejects_length_mismatch_and_escaping_shards(tmp_path):
    import json
    import struct

    import pytest
    import torch
    from grimoire_b200.formats.safetensors_io import CheckpointDir, SafeTensorsFile

    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4, 4], "data_offsets": [0, 32]}}).encode()     # 16 floats need 64 bytes
    (tmp_path / "bad.safetensors").write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 32)
    with pytest.raises(Exception):
        SafeTensorsFile(tmp_path / "bad.safetensors")
    d = tmp_path / "ck"
    d.mkdir()
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"w": "../bad.safetensors"}}))
    with pytest.raises(ValueError):
        CheckpointDir(d)
