"""Offline quantizer + artifact container round trip, imatrix file IO, KLD statistics, DP routing."""
import json

import torch

from grimoire_b200.formats.artifact import Artifact, quantize_checkpoint, write_artifact
from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.imatrix import importance_for, read_imatrix, write_imatrix
from grimoire_b200.formats.quantize import QuantWeight, quantize
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.parallel.dp import Replica, Router
from grimoire_b200.utils.kld import kld_stats
from tests.fixtures.mini_model import write_checkpoint


def test_artifact_roundtrip_all_formats(tmp_path):
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.02
    entries = [(f.name, quantize(w, f)) for f in (Fmt.INT4, Fmt.INT8, Fmt.FP8_E4M3, Fmt.MXFP4, Fmt.MXFP8, Fmt.FP8_BLOCK, Fmt.NVFP4, Fmt.BF16)]
    entries.append(("norm.weight", torch.ones(256)))
    write_artifact(tmp_path / "a.grm", entries)
    a = Artifact(tmp_path / "a.grm")
    for name, qw in entries[:-1]:
        back = a.get(name)
        assert isinstance(back, QuantWeight) and back.fmt == qw.fmt and back.group == qw.group
        assert torch.equal(back.dequant(), qw.dequant()), name
    assert torch.equal(a.get("norm.weight"), torch.ones(256))
    a.close()


def test_quantize_cli_bundle_on_checkpoint(tmp_path):
    cfg = tiny_dense()
    cfg.tie_word_embeddings = False
    write_checkpoint(tmp_path / "src", cfg, seed=3, quant="bf16", tokenizer=True)
    st = quantize_checkpoint(tmp_path / "src", tmp_path / "out", Fmt.INT4, policy="linear", bundle=True)
    assert st["quantized"] == 2 * 7 + 1 and (tmp_path / "out" / "manifest.json").exists() and (tmp_path / "out" / "tokenizer.json").exists()
    a = Artifact(st["path"])
    q = a.get("model.layers.0.mlp.down_proj.weight")
    assert isinstance(q, QuantWeight) and q.fmt == Fmt.INT4 and (q.N, q.K) == (256, 768)
    assert not isinstance(a.get("model.layers.0.input_layernorm.weight"), QuantWeight)
    assert not isinstance(a.get("model.embed_tokens.weight"), QuantWeight)


def test_imatrix_io_and_name_mapping(tmp_path):
    v = torch.rand(256)
    write_imatrix(tmp_path / "im.dat", {"blk.3.ffn_down.weight": v}, ncall=4)
    im = read_imatrix(tmp_path / "im.dat")
    got = importance_for(im, "model.layers.3.mlp.down_proj.weight")
    assert torch.allclose(got, v, atol=1e-6) and importance_for(im, "model.layers.2.mlp.down_proj.weight") is None


def test_kld_stats_identity_and_perturbation():
    torch.manual_seed(1)
    a = torch.randn(50, 1000)
    s = kld_stats(a, a)
    assert s["kld_mean"] < 1e-12 and s["top1_agreement"] == 1.0
    s2 = kld_stats(a, a + 0.3 * torch.randn_like(a))
    assert s2["kld_mean"] > 1e-3 and s2["top1_agreement"] < 1.0


def test_dp_router_affinity_and_least_loaded():
    reps = [Replica("127.0.0.1", 1), Replica("127.0.0.1", 2), Replica("127.0.0.1", 3)]
    r = Router(reps, affinity_slack=1)
    body = {"messages": [{"role": "user", "content": "same prefix"}]}
    first = r.pick(body)
    assert r.pick(body) is first                      # prefix affinity
    third = r.pick(body)
    assert third is not first                         # home replica is 2 ahead of the idlest: spill over
    reps[reps.index(first)].healthy = False
    assert r.pick(body) is not first                  # unhealthy replicas are skipped
