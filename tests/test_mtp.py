"""MTP draft head: speculative decoding with the head must reproduce plain greedy tokens (drafts only
change how many tokens a verify pass yields), the head's KV is warmed during prefill and caught up
after accepted blocks, and a head that copies the target's knowledge gets drafts accepted."""
import dataclasses

import pytest
import torch

from grimoire_b200.engine.engine import Engine, EngineLimits
from grimoire_b200.engine.generation import GenerationOptions, generate_tokens
from grimoire_b200.models.config import tiny_dense
from grimoire_b200.models.dense import DenseModel
from grimoire_b200.models.mtp import MtpDrafter, MtpHead


def _run(device, quant="int4", draft_vocab=0, K=3, n_new=24):
    cfg = dataclasses.replace(tiny_dense(), quant=quant, tie_word_embeddings=False)
    lim = EngineLimits(max_slots=2, max_ctx=160, prefill_chunk=16, max_decode_rows=8, extra_kv_layers=1)
    prompt = torch.randint(0, cfg.vocab_size, (37,), generator=torch.Generator().manual_seed(3)).tolist()
    e0 = Engine(DenseModel.random(cfg, device, seed=1, gen_device="cpu"), lim)
    e0.enable_speculation()           # what attaching a drafter does: plain and speculative steps on the same kernels
    plain = e0.generate(prompt, n_new, use_graph=False)
    model = DenseModel.random(cfg, device, seed=1, gen_device="cpu")
    eng = Engine(model, lim)
    drafter = MtpDrafter(eng, MtpHead.random_from_target(model, seed=1, noise=0.01, draft_vocab=draft_vocab, gen_device="cpu"))
    opts = GenerationOptions(max_new=n_new, draft_depth=K, drafter=drafter, use_graph=False)
    toks, reason = generate_tokens(eng, prompt, opts)
    return plain, toks, opts.stats, drafter


def test_mtp_speculation_reproduces_greedy_cpu():
    plain, toks, stats, drafter = _run("cpu")
    assert toks == plain
    assert stats.rounds > 0 and stats.drafted == 3 * stats.rounds - max(0, 3 * stats.rounds - stats.drafted)
    assert drafter.stats["warm_rows"] == 36 and drafter.stats["draft_steps"] == stats.drafted
    assert stats.emitted == len(toks)


def test_mtp_draft_vocab_head_cpu():
    plain, toks, stats, drafter = _run("cpu", draft_vocab=1024)
    assert toks == plain and drafter.head.draft_vocab == 1024


@pytest.mark.gpu
@pytest.mark.parametrize("quant", ["int4", "mxfp4"])
def test_mtp_speculation_reproduces_greedy_gpu(quant):
    """Exact reproduction needs the same kernel for one row and for verify rows: attaching a drafter puts the engine in
    its batch-invariant mode (every height on the tensor-core small-M kernels), with no environment override."""
    from grimoire_b200.ops import core as K
    from grimoire_b200.ops import linear
    plain, toks, stats, drafter = _run("cuda", quant=quant)
    assert linear.BATCH_INVARIANT and not linear.GEMV_W4
    assert toks == plain
    assert stats.rounds > 0 and drafter.stats["warm_rows"] == 36
    assert K.status_read()[0] == 0


def test_mtp_drafter_in_the_scheduler_reproduces_greedy_cpu():
    """Two concurrent conversations through the continuous-batching scheduler with the MTP drafter: tokens equal
    plain greedy decoding, the head's KV is warmed across partial prefill calls."""
    from grimoire_b200.sched.scheduler import Scheduler

    cfg = dataclasses.replace(tiny_dense(), tie_word_embeddings=False)
    lim = EngineLimits(max_slots=3, max_ctx=160, prefill_chunk=16, max_decode_rows=16, extra_kv_layers=1)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (29, 41)]
    plain = [Engine(DenseModel.random(cfg, "cpu", seed=1), lim).generate(p, 12, use_graph=False) for p in prompts]
    model = DenseModel.random(cfg, "cpu", seed=1)
    eng = Engine(model, lim)
    drafter = MtpDrafter(eng, MtpHead.random_from_target(model, seed=1, noise=0.01))
    sched = Scheduler(eng, width=4, prefill_chunk=16, interleave_chunk=16, depths=(3, 3, 3, 3), drafter=drafter, use_graph=False)
    try:
        import threading
        out = [None, None]

        def run(i):
            out[i] = sched.generate(prompts[i], 12)[0]
        ts = [threading.Thread(target=run, args=(i,)) for i in range(2)]
        for t in ts:
            t.start()
        for t in ts:
            t.join(timeout=120)
    finally:
        sched.shutdown()
    assert out[0] == plain[0] and out[1] == plain[1]
    assert drafter.stats["draft_steps"] > 0
