"""decode_mega.cu (persistent phase kernel of the single-row decode step) against fp32 PyTorch references of the same
chain, and the model-level path against the per-projection kernels."""
import pytest
import torch

from grimoire_b200.formats.codecs import Fmt
from grimoire_b200.formats.quantize import quantize
from grimoire_b200.formats.w4_tile_layout import interleave_gate_up_q
from grimoire_b200.ops import core as K
from grimoire_b200.ops import mega
from grimoire_b200.ops.linear import W4Linear
from grimoire_b200.ops.workspace import Workspace

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _clean():
    code, detail, n = K.status_read()
    assert code == 0, f"device status: code={code} detail={detail:#x} count={n}"


def _bf(x):
    return x.bfloat16().float()


def _rms(h, w, eps=1e-6):
    return _bf(h * torch.rsqrt((h * h).mean() + eps) * w)


@pytest.mark.parametrize("H,I,Q,group,xmag", [(256, 768, 384, 128, 1.0), (5120, 17408, 7168, 128, 1.0), (1024, 2048, 1536, 64, 1.0),
                                             (512, 1024, 512, 256, 1.0), (5120, 17408, 7168, 128, 3000.0), (320, 640, 96, 64, 1.0)])
def test_layer_chain_matches_fp32(H, I, Q, group, xmag):
    """o (+= h) | norm + gate|up + SwiGLU | down (+= h) | norm + qkv in ONE launch, twice in a row (the second launch
    proves the barrier words and counters were left reusable)."""
    torch.manual_seed(H + I)
    ws = Workspace(DEV)
    mk = lambda n, k: quantize(torch.randn(n, k) * 0.02 + 0.003, Fmt.INT4, group=group)
    qo, qg, qu, qd, qq = mk(H, H), mk(I, H), mk(I, H), mk(H, I), mk(Q, H)
    lo, ld, lq = W4Linear(qo, DEV, "o", workspace=ws), W4Linear(qd, DEV, "down", workspace=ws), W4Linear(qq, DEV, "qkv", workspace=ws)
    lgu = W4Linear(interleave_gate_up_q(qg, qu), DEV, "gu", swiglu=True, workspace=ws)
    attn = torch.randn(H) * 0.5
    attn[3] = xmag
    attn[H - 7] = -0.7 * xmag
    h0 = torch.randn(H)
    nw1, nw2 = 1.0 + 0.1 * torch.randn(H), 1.0 + 0.1 * torch.randn(H)
    d_attn = attn.to(DEV).bfloat16()
    d_h = h0.clone().to(DEV)
    d_act = torch.zeros(I, dtype=torch.bfloat16, device=DEV)
    d_qkv = torch.zeros(lq.Np, dtype=torch.bfloat16, device=DEV)
    d_nw1, d_nw2 = nw1.to(DEV), nw2.to(DEV)
    phases = [mega._phase(lo, mega.PRO_X, mega.EPI_ADD, d_attn, None, d_h, 1e-6, 0.0),
              mega._phase(lgu, mega.PRO_NORM, mega.EPI_SWIGLU, None, d_nw1, d_act, 1e-6, 0.0),
              mega._phase(ld, mega.PRO_X, mega.EPI_ADD, d_act, None, d_h, 1e-6, 0.0),
              mega._phase(lq, mega.PRO_NORM, mega.EPI_BF16, None, d_nw2, d_qkv, 1e-6, 0.0)]
    tab = mega.MegaTable(phases, DEV, d_h)
    # fp32 reference with the kernel's rounding points
    Wo, Wg, Wu, Wd, Wq = (q.dequant().float() for q in (qo, qg, qu, qd, qq))

    def ref(h):
        h = h + Wo @ _bf(attn)
        x = _rms(h, nw1)
        act = _bf(torch.nn.functional.silu(Wg @ x) * (Wu @ x))
        h = h + Wd @ act
        return h, act, _bf(Wq @ _rms(h, nw2))

    h1, act1, qkv1 = ref(h0)
    tab.run(0, 4)
    torch.cuda.synchronize()
    _clean()
    tol = dict(atol=3e-3 * max(1.0, xmag / 30), rtol=2e-3)
    assert torch.allclose(d_act.float().cpu(), act1, atol=2e-2, rtol=2e-2), float((d_act.float().cpu() - act1).abs().max())
    assert torch.allclose(d_h.cpu(), h1, **tol), float((d_h.cpu() - h1).abs().max())
    assert torch.allclose(d_qkv[:Q].float().cpu(), qkv1, atol=3e-2, rtol=3e-2), float((d_qkv[:Q].float().cpu() - qkv1).abs().max())
    h2, act2, qkv2 = ref(h1)
    tab.run(0, 4)
    torch.cuda.synchronize()
    _clean()
    assert torch.allclose(d_h.cpu(), h2, atol=2 * tol["atol"], rtol=2 * tol["rtol"]), float((d_h.cpu() - h2).abs().max())
    assert int(tab.sync[0]) == 2 * 4 * tab.grid and int(tab.sync[2]) == 0       # every launch adds one round per phase


def test_phase_runs_are_deterministic_and_graph_replayable():
    torch.manual_seed(5)
    ws = Workspace(DEV)
    H, N = 2048, 4096
    lin = W4Linear(quantize(torch.randn(N, H) * 0.02, Fmt.INT4), DEV, "p", workspace=ws)
    x = torch.randn(H, device=DEV).bfloat16()
    out = torch.zeros(N, dtype=torch.float32, device=DEV)
    tab = mega.MegaTable([mega._phase(lin, mega.PRO_X, mega.EPI_F32, x, None, out, 1e-6, 0.0)] * 3, DEV, out)
    tab.run(0, 3)
    torch.cuda.synchronize()
    first = out.clone()
    g = torch.cuda.CUDAGraph()
    out.zero_()
    with torch.cuda.graph(g):
        tab.run(0, 3)
    for _ in range(3):
        out.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, first)
    _clean()


def test_model_decode_matches_per_projection_kernels(monkeypatch):
    """Greedy tokens and logits of a small dense model: phase kernel vs the one-launch-per-projection path."""
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import ModelConfig
    from grimoire_b200.models.dense import DenseModel

    cfg = ModelConfig(vocab_size=4096, hidden_size=512, intermediate_size=1536, num_hidden_layers=3, num_attention_heads=8,
                      num_key_value_heads=2, head_dim=64, tie_word_embeddings=False)
    prompt = torch.randint(0, 4096, (40,), generator=torch.Generator().manual_seed(3)).tolist()
    outs = {}
    for flag in (True, False):
        monkeypatch.setattr(mega, "MEGA", flag)
        model = DenseModel.random(cfg, DEV, seed=2, std=0.05)
        eng = Engine(model, EngineLimits(max_slots=2, max_ctx=256))
        toks, logits = eng.generate(prompt, 12, collect_logits=True)
        outs[flag] = (toks, torch.stack(logits))
        assert model._mega_ready() == flag
    _clean()
    d = (outs[True][1] - outs[False][1]).abs().max()
    scale = outs[False][1].abs().max()
    assert float(d) < 2e-2 * float(scale), (float(d), float(scale))
    assert outs[True][0][:4] == outs[False][0][:4]
