"""Auxiliary subsystems: timeline / probe tracing, expert heat + placement, DFlash config resolution."""
import json

import pytest
import torch

from grimoire_b200.models.dflash import resolve_dflash_config
from grimoire_b200.models.expert_placement import ExpertHeat, HeatParams, balanced_placement, rank_loads
from grimoire_b200.utils import trace


def test_timeline_regions_and_probe(capsys, monkeypatch):
    tl = trace.Timeline()
    tl.enable(True)
    for tag in ("a", "b", "a", "end"):
        tl.mark(tag)
    d = tl.dump()
    assert list(d) == ["a", "b"] and all(v >= 0 for v in d.values())
    assert len(tl.dump(per_mark=True)) == 3
    assert "a" in tl.format()
    tl.enable(False)
    tl.mark("x")
    assert tl.dump() == {}
    t = torch.tensor([3.0, -4.0, float("nan"), float("inf")])
    st = trace.probe_stats(t, exact=True)
    assert st["nan"] == 1 and st["inf"] == 1 and st["max"] == 4.0 and len(st["fnv1a"]) == 16
    assert trace.probe_stats(t, exact=True)["fnv1a"] == st["fnv1a"]
    assert trace.fnv1a(b"") == 0xCBF29CE484222325 and trace.fnv1a(b"a") == 0xAF63DC4C8601EC8C
    assert trace.probe("off", t) is None
    monkeypatch.setenv("GRIMOIRE_DEBUG", "1")
    assert trace.probe("h", t)["n"] == 4 and "[probe] h:" in capsys.readouterr().out
    store = {}
    with trace.FencedTimer(store, "verify"):
        pass
    assert store["verify"] >= 0.0


def test_dense_forward_marks_regions():
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import tiny_dense
    from grimoire_b200.models.dense import DenseModel
    from grimoire_b200.models.synthetic import random_state_dict

    cfg = tiny_dense()
    eng = Engine(DenseModel.from_state_dict(cfg, random_state_dict(cfg, seed=0), "cpu"), EngineLimits(max_slots=1, max_ctx=64, prefill_chunk=32,
                                                                                                 max_decode_rows=2))
    trace.timeline.enable(True)
    try:
        eng.generate([1, 2, 3, 4], 2)
        d = trace.timeline.dump()
    finally:
        trace.timeline.enable(False)
    assert {"norm+qkv", "rope+attn", "o_proj", "norm+gate_up", "down", "head"} <= set(d)


def test_expert_heat_credit_cap_decay_and_swaps(tmp_path):
    h = ExpertHeat(2, 8, HeatParams(decay=0.5, credit_cap=4, moves_per_step=2, hysteresis=1.25, min_gain=1.5))
    h.credit(0, [1, 1, 1, -1])                # out-of-range ids are skipped
    assert h.h[0, 1] == 3.0 and h.h[0].sum() == 3.0
    h.credit(0, [2] * 16)                      # 16 selections capped to 4 credits in total; older heat halves
    assert abs(h.h[0, 2] - 4.0) < 1e-6 and abs(h.h[0, 1] - 1.5) < 1e-6
    resident = lambda l, e: e in (0, 1)        # experts 0,1 resident; 2 is hot and not resident
    swaps = h.propose_swaps(resident, lambda l, e: l == 0)
    assert len(swaps) == 1 and (swaps[0].promote_expert, swaps[0].demote_expert) == (2, 0)   # coldest victim first
    # hysteresis: a marginally hotter expert does not displace a resident one
    g = ExpertHeat(1, 4, HeatParams(decay=1.0, min_gain=1.5))
    g.credit(0, [0, 0, 1, 1, 1])
    assert g.propose_swaps(lambda l, e: e == 0, lambda l, e: True) == []
    p = str(tmp_path / "hits.json")
    h.save(p)
    h2 = ExpertHeat(2, 8)
    assert h2.load(p) and (h2.hits == h.hits).all()
    assert not ExpertHeat(3, 8).load(p)


def test_balanced_placement_evens_rank_loads():
    heat = [100, 90, 80, 70, 1, 1, 1, 1]
    naive = rank_loads(heat, list(range(8)), 2)
    perm = balanced_placement(heat, 2)
    bal = rank_loads(heat, perm, 2)
    assert sorted(perm) == list(range(8))
    assert max(bal) - min(bal) < max(naive) - min(naive)
    assert max(bal) - min(bal) <= 20
    assert balanced_placement(heat, 2) == perm            # deterministic


STANDARD = {
    "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 6, "num_attention_heads": 32, "num_key_value_heads": 4,
    "head_dim": 128, "rms_norm_eps": 1e-06, "vocab_size": 262144, "draft_vocab_size": 32768, "sliding_window": None,
    "rope_parameters": {"rope_type": "default", "rope_theta": 5000000.0},
    "dflash_config": {"mask_token_id": 248077, "block_size": 16}, "target_layer_ids": [1, 6, 11, 16, 22, 27, 32, 37]}


def test_dflash_config_standard_and_precedence():
    s = resolve_dflash_config(json.dumps(STANDARD))
    assert not s.error and s.n_layers == 6 and s.head_dim == 128 and s.rope_theta == 5e6 and s.mask_token == 248077
    assert s.draft_vocab == 32768 and s.target_layers == [1, 6, 11, 16, 22, 27, 32, 37] and s.tap_key == "target_layer_ids"
    assert not s.attn_from_config and all(l.window == 0 and not l.causal for l in s.layers) and len(s.layers) == 6
    # dflash_config wins over eagle_config wins over the top level
    c = dict(STANDARD, eagle_config={"num_hidden_layers": 5, "rms_norm_eps": 1e-5}, dflash_config={"num_hidden_layers": 4, "mask_token_id": 7})
    s = resolve_dflash_config(json.dumps(c))
    assert s.n_layers == 4 and abs(s.rms_eps - 1e-5) < 1e-12 and s.mask_token == 7
    # defaults that are not checkpoint facts are reported
    s = resolve_dflash_config(json.dumps({"num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4}))
    assert s.rope_theta == 1e6 and s.head_dim == 64 and s.mask_token == -1 and len(s.notes) >= 3


def test_dflash_config_attention_shape_rules():
    base = {"num_hidden_layers": 4, "hidden_size": 256, "num_attention_heads": 4}
    # use_swa with no layer_types: every layer slides with the dflash window
    s = resolve_dflash_config(json.dumps(dict(base, dflash_config={"use_swa": 1, "swa_window_size": 512})))
    assert s.attn_from_config and [l.window for l in s.layers] == [512] * 4 and not any(l.causal for l in s.layers)
    # layer_types decide per layer; sliding layers are causal unless overridden
    lt = ["sliding_attention", "full_attention", "sliding_attention", "full_attention"]
    s = resolve_dflash_config(json.dumps(dict(base, layer_types=lt, sliding_window=1024)))
    assert [l.window for l in s.layers] == [1024, 0, 1024, 0] and [l.causal for l in s.layers] == [True, False, True, False]
    s = resolve_dflash_config(json.dumps(dict(base, layer_types=lt, sliding_window=1024, is_causal=False)))
    assert not any(l.causal for l in s.layers)
    s = resolve_dflash_config(json.dumps(dict(base, layer_types=lt, sliding_window=1024, dflash_config={"causal": True})))
    assert all(l.causal for l in s.layers)
    # use_swa with layer_types that name no sliding layer: the flag wins for all layers
    s = resolve_dflash_config(json.dumps(dict(base, layer_types=["full_attention"] * 4, dflash_config={"use_swa": True, "swa_window_size": 64})))
    assert [l.window for l in s.layers] == [64] * 4
    # errors: sliding without a window, short layer_types, bad JSON
    assert "no window" in resolve_dflash_config(json.dumps(dict(base, dflash_config={"use_swa": True}))).error
    assert "only 2 entries" in resolve_dflash_config(json.dumps(dict(base, layer_types=lt[:2]))).error
    assert resolve_dflash_config("{nope").error and resolve_dflash_config("[1]").error
    assert resolve_dflash_config(json.dumps({"hidden_size": 8})).error


def test_verify_groups_and_split_heuristic():
    """Host-side planning of a decode step's attention: verify blocks are cut into groups of at most 16 // G rows of one
    conversation at consecutive positions; the split-KV factor follows the measured table."""
    from grimoire_b200.ops import core as K

    slots = [3, 3, 3, 3, 3, 1, 2, 2, 2]
    pos = [10, 11, 12, 13, 14, 99, 7, 8, 20]
    assert K.verify_groups(slots, pos, 3) == [(3, 0, 3, 10), (3, 3, 2, 13), (1, 5, 1, 99), (2, 6, 2, 7), (2, 8, 1, 20)]
    assert K.verify_groups(slots, pos, 16)[0] == (3, 0, 5, 10)
    assert K.verify_rows_per_group(K.AttnGeom(40, 8, 128, 128, 0.1)) == 3
    assert K.verify_rows_per_group(K.AttnGeom(32, 8, 128, 128, 0.1)) == 4
    # one row, 8 kv heads: 16 splits up to 8,192 tokens (cluster merge), 32 from 16,384; never fewer than 8 pages a split
    assert [K.decode_splits(n, 1, 8) for n in (100, 512, 1024, 4096, 8192, 16384, 32768, 131072)] == [1, 4, 8, 16, 16, 32, 32, 32]
    assert K.decode_splits(4096, 8, 8) == 4 and K.decode_splits(4096, 1, 1) == 16


def test_perplexity_scores_second_halves_and_dumps_candidates(tmp_path):
    """``--ppl``: complete chunks only, positions ctx/2 .. ctx-2 scored, running mean with its standard error; ``--ppl-dump``
    writes a line per scored token with the eight best candidates; ``--ppl-selfcheck`` compares decode with batched prefill."""
    import math

    import torch

    from grimoire_b200.api import Grimoire
    from grimoire_b200.config import EngineConfig

    g = Grimoire.load(EngineConfig(model="synthetic:tiny_dense", ctx=64, seq_slots=2, prefill_chunk=32), device="cpu")
    V = g.model.cfg.vocab_size
    ids = torch.randint(0, V, (2 * 16 + 5,), generator=torch.Generator().manual_seed(0)).tolist()
    dump = tmp_path / "ppl.tsv"
    res = g.perplexity(ids, ctx=16, dump=str(dump), selfcheck=True)
    assert res["chunks"] == 2 and res["tokens"] == 2 * 7                     # positions 8..14 of each 16-token chunk; 5 tokens dropped
    want = []
    for c in range(2):
        w = ids[c * 16: (c + 1) * 16]
        lp = torch.log_softmax(g.score_ids(w[:-1]).double(), -1)
        want += [-float(lp[p, w[p + 1]]) for p in range(8, 15)]
    mean = sum(want) / len(want)
    assert res["ppl"] == pytest.approx(math.exp(mean), rel=1e-9)
    var = sum((x - mean) ** 2 for x in want) / (len(want) - 1)
    assert res["ppl_stderr"] == pytest.approx(math.exp(mean) * math.sqrt(var / len(want)), rel=1e-6)
    assert res["selfcheck_max_abs_diff"] < 0.05
    lines = dump.read_text().splitlines()
    assert len(lines) == 14
    f = lines[0].split("\t")
    assert f[:3] == ["1", "8", str(ids[9])] and len(f) == 6 + 8 and float(f[3]) == pytest.approx(-want[0], rel=1e-9)
    assert f[6].split(":")[0] == f[4] and float(f[6].split(":")[1]) == pytest.approx(float(f[5]))
    assert g.perplexity(ids, ctx=16, chunks=1)["tokens"] == 7
    with pytest.raises(ValueError, match="no complete"):
        g.perplexity(ids[:10], ctx=16)
    g.close()


def test_kld_base_file_round_trip_and_statistics(tmp_path):
    """The llama-perplexity base format (header, tokens, quantised log-probability rows) and its statistics: a model scored
    against its own base gives a near-zero divergence and full top-1 agreement; a perturbed one does not."""
    import numpy as np
    import torch

    from grimoire_b200.api import Grimoire
    from grimoire_b200.config import EngineConfig
    from grimoire_b200.utils.kld import KldBase, KldStats, write_kld_base

    g = Grimoire.load(EngineConfig(model="synthetic:tiny_dense", ctx=64, seq_slots=2, prefill_chunk=32), device="cpu")
    V, ctx = g.model.cfg.vocab_size, 16
    ids = torch.randint(0, V, (3 * ctx,), generator=torch.Generator().manual_seed(1)).tolist()
    chunks = [ids[c * ctx: (c + 1) * ctx] for c in range(3)]
    rows = [g.score_ids(w[:-1])[ctx // 2: ctx - 1].float().numpy() for w in chunks]
    path = tmp_path / "base.kld"
    write_kld_base(str(path), ctx, chunks, rows)
    b = KldBase(str(path))
    assert (b.ctx, b.vocab, b.chunks, b.scored) == (ctx, V, 3, 7)
    tok, sc, mn, q = b.read_chunk(1)
    assert tok.tolist() == chunks[1] and q.shape == (7, V)
    lp = torch.log_softmax(torch.tensor(rows[1]).double(), -1).numpy()
    back = sc[:, None] * q.astype(np.float32) + mn[:, None]
    keep = lp > lp.max(1, keepdims=True) - 15.9
    assert np.abs(back - lp)[keep].max() < 2e-3                     # 16 nats over 65,535 steps
    res = g.perplexity([], kld_base=str(path))
    k = res["kld"]
    assert res["chunks"] == 3 and k["count"] == 21 and k["kld_mean"] < 1e-5 and k["same_top"] == 1.0 and abs(k["ln_ppl_ratio"]) < 1e-3
    assert res["kld_report"] == ""                                  # under 100 scored tokens nothing is printed, as in llama.cpp
    st = KldStats()
    noisy = rows[0] + np.random.default_rng(0).normal(0, 1.0, rows[0].shape).astype(np.float32)
    _, sc0, mn0, q0 = b.read_chunk(0)
    st.add_rows(noisy, sc0, mn0, q0, chunks[0][ctx // 2 + 1:])
    s = st.summary()
    assert s["kld_mean"] > 0.05 and s["kld_max"] >= s["kld_median"] >= s["kld_min"] >= 0 and s["dp_rms"] > 0
    bad = tmp_path / "bad.kld"
    bad.write_bytes(path.read_bytes()[:-2])
    with pytest.raises(ValueError, match="size mismatch"):
        KldBase(str(bad))
    g.close()


def test_host_expert_rows_match_a_plain_product():
    """csrc/host/cpu_experts.cpp: block-scaled e4m3 expert FFN rows on CPU threads -- same numbers for any thread count,
    refusal of unsorted pairs and of widths that are no multiple of the scale block."""
    import ctypes

    import torch

    from grimoire_b200 import _native
    from grimoire_b200.formats.codecs import Fmt
    from grimoire_b200.formats.quantize import quantize
    from grimoire_b200.ops.cpu_experts import CpuExperts

    torch.manual_seed(0)
    E, H, I, M, k = 3, 256, 128, 6, 2
    gu, dn = torch.randn(E, 2 * I, H) * 0.05, torch.randn(E, H, I) * 0.05

    def q3(t):
        n, kk = t.shape[1], t.shape[2]
        q = quantize(t.reshape(E * n, kk), Fmt.FP8_BLOCK)
        return q.payload.reshape(E, n, kk), q.scales.reshape(E, n, kk // 128).float(), q.dequant().float().reshape(E, n, kk)

    g8, gs, gd = q3(gu)
    d8, ds, dd = q3(dn)
    x = torch.randn(M, H).bfloat16()
    ids = torch.tensor([[0, 1], [2, 1], [0, 0], [1, 2], [2, 0], [1, 1]], dtype=torch.int32)
    w = torch.rand(M, k + 1)
    want = torch.zeros(M, H)
    for m in range(M):
        for j in range(k):
            e = int(ids[m, j])
            if e >= 1:
                xf = x[m].float()
                a = (torch.nn.functional.silu(gd[e, :I] @ xf) * (gd[e, I:] @ xf)).bfloat16().float()
                want[m] += w[m, j] * (dd[e] @ a)
    outs = [CpuExperts(1, g8[1:], gs[1:], d8[1:], ds[1:], threads=t).run(x, ids, w) for t in (1, 3, 16)]
    assert float((outs[0] - want).abs().max()) < 1e-5
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])          # one writer per row, pairs in order
    assert CpuExperts(3, g8[:0], gs[:0], d8[:0], ds[:0]).run(x, ids, w) is None       # no route names a host expert
    lib = _native.host()
    rows, exp, wt = torch.tensor([1, 0], dtype=torch.int32), torch.zeros(2, dtype=torch.int32), torch.ones(2)
    out = torch.zeros(M, H)
    args = lambda h, i: (_native.ptr(g8), _native.ptr(gs), _native.ptr(d8), _native.ptr(ds), _native.ptr(x), ctypes.c_int(H), _native.ptr(rows),
                         _native.ptr(exp), _native.ptr(wt), ctypes.c_int(2), _native.ptr(out), ctypes.c_int(H), ctypes.c_int(h), ctypes.c_int(i),
                         ctypes.c_int(2))
    assert lib.grm_cx_moe_rows(*args(H, I)) == -2                                     # rows must not decrease
    assert lib.grm_cx_moe_rows(*args(H + 64, I)) == -2


def test_host_memory_budget_honours_container_limits(tmp_path):
    from grimoire_b200.utils.host_budget import host_available_ram, host_slot_limit

    mem = tmp_path / "meminfo"
    mem.write_text("MemTotal:       1000000 kB\nMemAvailable:    500000 kB\n")
    assert host_available_ram(str(mem), cgroups=()) == 500000 * 1024
    lim, cur = tmp_path / "max", tmp_path / "cur"
    lim.write_text("300000000\n"), cur.write_text("100000000\n")
    assert host_available_ram(str(mem), [(str(lim), str(cur))]) == 200000000          # the container's headroom is the smaller
    lim.write_text("max\n")
    assert host_available_ram(str(mem), [(str(lim), str(cur))]) == 500000 * 1024      # no limit set
    assert host_available_ram(str(tmp_path / "none"), cgroups=()) == 0
    assert host_available_ram() > 0
    # the first buffer exists; three more are asked for, on two ranks, 10 units each, 55 free above the reserve
    assert host_slot_limit(available=65, reserve=10, slot_bytes=10, ranks=2, requested=4) == 3
    assert host_slot_limit(65, 10, 10, 2, 1) == 1 and host_slot_limit(5, 10, 10, 2, 4) == 1 and host_slot_limit(65, 10, 0, 2, 4) == 4
