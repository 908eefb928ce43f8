"""Distribution-distance statistics between two runs' logits (accuracy of a quantized build against
a baseline): mean / median / p99 KL divergence, top-1 agreement, mean probability of the baseline's
top token.  Reference: include/b70/kld.hpp and the --ppl-kld-base mode of the CLI."""
from __future__ import annotations

import torch


def kld_stats(base_logits: torch.Tensor, test_logits: torch.Tensor) -> dict:
    n = min(base_logits.shape[0], test_logits.shape[0])
    b = torch.log_softmax(base_logits[:n].double(), dim=-1)
    t = torch.log_softmax(test_logits[:n].double(), dim=-1)
    kl = (b.exp() * (b - t)).sum(dim=-1).clamp_min(0.0)
    top_b, top_t = b.argmax(-1), t.argmax(-1)
    p_same = t.exp().gather(1, top_b[:, None])[:, 0]
    srt = kl.sort().values
    return {"positions": int(n), "kld_mean": float(kl.mean()), "kld_median": float(srt[n // 2]),
            "kld_p99": float(srt[min(n - 1, int(0.99 * n))]), "kld_max": float(kl.max()),
            "top1_agreement": float((top_b == top_t).double().mean()), "mean_p_of_base_top1": float(p_same.mean()),
            "cosine": float(torch.nn.functional.cosine_similarity(base_logits[:n].double(), test_logits[:n].double(), dim=-1).mean())}
