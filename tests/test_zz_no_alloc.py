"""The allocation-free entry point of the int4 small-M product, called through its exported C
symbol, against the ordinary entry point on the same inputs.

Why the entry point exists: some hosts of this library may not allocate device memory while they
run (they handed the whole GPU to their own pool at start-up, or they sit in a latency-bound loop
that cannot afford the synchronisation an allocation may imply).  For them the split-K scratch is
a fixed array inside the library.  The test makes two calls in a row, because both share that one
array: the second call must not be disturbed by what the first one left behind.  This file is
collected last so that a run that stops at the first failure has already run every other test.
"""
import ctypes

import pytest
import torch

from grimoire_b200 import _native
from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.formats.w4_tile_layout import tile_w4

pytestmark = pytest.mark.gpu


def _c(v):
    return ctypes.c_int(int(v))


def _scratch_floats(M, N, rows, ksplit, epi):
    mt = 1
    while mt * 8 < M:
        mt *= 2
    r = 2 if epi == 3 else (2 if rows == 32 and mt <= 2 else 1)
    return ksplit * (N // (16 * r)) * r * mt * 128, N // (16 * r)


def _call_plain(lib, t, x, out, ksplit, rows, epi=1):
    M = x.shape[0]
    nf, tiles = _scratch_floats(M, t.N, rows, ksplit, epi)
    scratch = torch.empty(nf, dtype=torch.float32, device="cuda")
    counters = torch.zeros(tiles, dtype=torch.int32, device="cuda")
    rc = lib.grm_smallm_w4(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(out), _native.ptr(scratch),
                           _native.ptr(counters), _c(M), _c(t.N), _c(t.K), _c(x.stride(0)), _c(out.stride(0)), _c(t.group),
                           _c(epi), _c(rows), _c(ksplit), _native.stream_ptr())
    assert rc == 0


def _call_noalloc(lib, t, x, out, ksplit, rows, epi=1):
    M = x.shape[0]
    fn = lib.grm_smallm_w4_noalloc           # resolved by name from the shared library
    return fn(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(out), _c(M), _c(t.N), _c(t.K),
              _c(x.stride(0)), _c(out.stride(0)), _c(t.group), _c(epi), _c(rows), _c(ksplit), _native.stream_ptr())


def test_noalloc_entry_point_matches_ordinary_entry_point_twice():
    lib = _native.cuda()
    torch.manual_seed(0)
    cases = [(3, 64, 4096, 4), (17, 96, 2048, 2)]          # (M, N, K, ksplit): two different shapes in a row
    for M, N, K, ksplit in cases:
        qw = quantize(torch.randn(N, K) * 0.02, Fmt.INT4)
        t = tile_w4(qw).to("cuda")
        x = torch.randn(M, K, device="cuda").bfloat16()
        want = torch.zeros(M, t.N, dtype=torch.float32, device="cuda")
        _call_plain(lib, t, x, want, ksplit, 16)
        got = torch.full((M, t.N), float("nan"), dtype=torch.float32, device="cuda")
        free_before = torch.cuda.mem_get_info()[0]
        assert _call_noalloc(lib, t, x, got, ksplit, 16) == 0
        torch.cuda.synchronize()
        assert free_before - torch.cuda.mem_get_info()[0] < (2 << 20)   # nothing was taken from the device
        assert torch.allclose(got, want, atol=2e-3, rtol=1e-3), float((got - want).abs().max())
        # against the fp32 dequantised product as well, with the tolerance of the kernel tests
        ref = x.float().cpu() @ qw.dequant().t()
        assert torch.allclose(got[:, :N].cpu(), ref, atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("M,N,K,ksplit,rows,epi", [(5, 256, 2048, 2, 32, 3),     # SwiGLU tiles (two 16-row tiles per CTA), split K
                                                   (9, 128, 4096, 4, 32, 1),     # 32-row CTAs with two batch tiles
                                                   (64, 64, 2048, 2, 16, 1),     # the widest batch the kernel is built for
                                                   (2, 96, 1024, 1, 16, 2)])     # one K slice: scratch untouched, accumulate epilogue
def test_noalloc_entry_point_covers_every_scratch_sizing(M, N, K, ksplit, rows, epi):
    """Each (batch tile count, rows per CTA, epilogue) combination sizes the shared scratch differently; all of them must
    agree with the ordinary entry point."""
    lib = _native.cuda()
    torch.manual_seed(M + N)
    qw = quantize(torch.randn(N, K) * 0.02, Fmt.INT4)
    t = tile_w4(qw).to("cuda")
    x = torch.randn(M, K, device="cuda").bfloat16()
    if epi == 3:
        mk = lambda: torch.zeros(M, t.N // 2, dtype=torch.bfloat16, device="cuda")
    else:
        mk = lambda: torch.ones(M, t.N, dtype=torch.float32, device="cuda")
    want, got = mk(), mk()
    _call_plain(lib, t, x, want, ksplit, rows, epi)
    assert _call_noalloc(lib, t, x, got, ksplit, rows, epi) == 0
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_noalloc_entry_point_rejects_oversized_problems():
    lib = _native.cuda()
    qw = quantize(torch.randn(32, 512) * 0.02, Fmt.INT4)
    t = tile_w4(qw).to("cuda")
    x = torch.randn(1, 512, device="cuda").bfloat16()
    out = torch.zeros(1, 32, dtype=torch.float32, device="cuda")
    # a made-up N far beyond the tile limit of a split-K call: refused before anything is read or launched
    fn = lib.grm_smallm_w4_noalloc
    rc = fn(_native.ptr(t.w), _native.ptr(t.sz), _native.ptr(x), _native.ptr(out), _c(1), _c(32 * 8192), _c(512), _c(512),
            _c(32), _c(128), _c(1), _c(16), _c(2), _native.stream_ptr())
    assert rc == -5
