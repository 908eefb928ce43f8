"""Sampling: the host reference (temperature / top-k / top-p with a counter-based uniform, include/b70/sampling.hpp),
speculative coupled sampling (include/b70/speculative_sampling.hpp:39-61), the device sampler against the host reference
(tools/test_sampling.cpp, test_coupled_sampling.cpp in the reference), and the serving path that uses it."""
import pytest
import torch

from grimoire_b200.engine.sampling import SamplingOptions, coupled_sample, sample_ref, uniform


def test_sample_ref_is_a_function_of_seed_and_position():
    lg = torch.randn(1000, generator=torch.Generator().manual_seed(0)) * 3
    o = SamplingOptions(temperature=0.8, top_k=20, top_p=0.9, seed=1234)
    a = [sample_ref(lg, o, p) for p in range(50)]
    b = [sample_ref(lg, o, p) for p in range(50)]
    assert a == b and len(set(a)) > 1
    top20 = set(torch.topk(lg, 20).indices.tolist())
    assert set(a) <= top20
    assert sample_ref(lg, SamplingOptions(temperature=0.0), 3) == int(lg.argmax())
    assert sample_ref(lg, SamplingOptions(temperature=1.0, top_k=1), 3) == int(lg.argmax())
    assert 0.0 <= uniform(7, 11) < 1.0


def test_coupled_sampling_keeps_the_target_distribution():
    g = torch.Generator().manual_seed(1)
    pt = torch.softmax(torch.randn(8, generator=g), 0)
    pd = torch.softmax(torch.randn(8, generator=g), 0)
    counts = torch.zeros(8)
    n = 20000
    u = torch.rand(n, 3, generator=g)
    for i in range(n):
        d = int(torch.searchsorted(torch.cumsum(pd, 0), u[i, 0]).clamp_max(7))
        tok, _ = coupled_sample(pt, pd, d, float(u[i, 1]), float(u[i, 2]))
        counts[tok] += 1
    assert float((counts / n - pt).abs().max()) < 0.015


@pytest.mark.gpu
def test_device_sampler_matches_host_reference():
    from grimoire_b200.engine.sampling import DeviceSampler

    V, M = 151936, 6
    g = torch.Generator().manual_seed(5)
    logits = (torch.randn(M, V, generator=g) * 2.5).cuda()
    opts = [SamplingOptions(0.7, 20, 0.95, 11), SamplingOptions(1.3, 64, 1.0, 12), SamplingOptions(0.0, 20, 1.0, 13),
            SamplingOptions(0.5, 5, 0.5, 2 ** 63 + 5), SamplingOptions(1.0, 1, 1.0, 3), SamplingOptions(2.0, 40, 0.8, 0)]
    ds = DeviceSampler(8, "cuda")
    ds.set_rows(opts)
    for base in (0, 17, 4096):
        pos = torch.arange(base, base + M, dtype=torch.int32, device="cuda")
        out = torch.zeros(M, dtype=torch.int32, device="cuda")
        ds.sample(logits, pos, out)
        want = [sample_ref(logits[i].cpu(), opts[i], base + i) for i in range(M)]
        assert out.tolist() == want
    assert int(ds.counters.abs().sum()) == 0


@pytest.mark.gpu
def test_sampled_requests_keep_logits_on_the_device():
    from grimoire_b200.engine.engine import Engine, EngineLimits
    from grimoire_b200.models.config import small_dense
    from grimoire_b200.models.dense import DenseModel
    from grimoire_b200.sched.scheduler import Scheduler

    eng = Engine(DenseModel.random(small_dense(2), "cuda", seed=1), EngineLimits(max_slots=2, max_ctx=256, max_decode_rows=8))
    sched = Scheduler(eng, width=2, hold_ms=0.0)
    prompt = torch.randint(0, 8192, (20,), generator=torch.Generator().manual_seed(2)).tolist()
    opt = SamplingOptions(temperature=0.9, top_k=30, top_p=0.9, seed=77)
    a = sched.generate(prompt, 12, sampling=opt)[0]
    b = sched.generate(prompt, 12, sampling=opt)[0]
    sched.shutdown()
    assert a == b and len(a) == 12                       # same seed, same positions: same draw
    assert eng.counters.get("sample_d2h_bytes", 0) == 4 * 12 * 2      # four bytes per sampled token came back, nothing else
