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


# ---- llama-perplexity ``--kl-divergence-base`` files and its statistics (include/b70/kld.hpp) ----
import math
import struct

import numpy as np


class KldBase:
    """Reader of a ``--kl-divergence-base`` file: magic ``_logits_``, int32 n_ctx / n_vocab / n_chunk, the chunks' tokens
    (int32 [n_chunk][n_ctx]), then for every chunk its scored rows (positions n_ctx/2 .. n_ctx-2): float32 scale, float32
    minimum log-probability, n_vocab uint16 quantised log-probabilities padded to an even count."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            head = f.read(20)
            f.seek(0, 2)
            size = f.tell()
        if len(head) < 20:
            raise ValueError(f"truncated header: {path}")
        if head[:8] != b"_logits_":
            raise ValueError(f"invalid magic: {path}")
        self.ctx, self.vocab, self.chunks = struct.unpack("<iii", head[8:])
        if self.ctx < 4 or self.vocab <= 0 or self.chunks <= 0:
            raise ValueError(f"invalid n_ctx, n_vocab, or n_chunk: {path}")
        self.scored = self.ctx - 1 - self.ctx // 2
        self.row_words = 2 * ((self.vocab + 1) // 2) + 4
        self._records = 20 + 4 * self.ctx * self.chunks
        if size != self._records + 2 * self.row_words * self.scored * self.chunks:
            raise ValueError(f"size mismatch (truncated or trailing data): {path}")

    def read_chunk(self, chunk: int):
        """(tokens int32 [n_ctx], scale fp32 [scored], min log-prob fp32 [scored], q uint16 [scored][n_vocab])."""
        if not 0 <= chunk < self.chunks:
            raise IndexError("chunk index")
        with open(self.path, "rb") as f:
            f.seek(20 + 4 * self.ctx * chunk)
            tokens = np.frombuffer(f.read(4 * self.ctx), dtype="<i4")
            f.seek(self._records + 2 * self.row_words * self.scored * chunk)
            rows = np.frombuffer(f.read(2 * self.row_words * self.scored), dtype="<u2").reshape(self.scored, self.row_words)
        hdr = np.ascontiguousarray(rows[:, :4]).view("<f4")
        return tokens, hdr[:, 0].copy(), hdr[:, 1].copy(), rows[:, 4: 4 + self.vocab]


def write_kld_base(path: str, ctx: int, chunks_tokens, chunks_logits) -> None:
    """Write a base file from a baseline run: per chunk its ``ctx`` tokens and the logits rows of positions ctx/2 .. ctx-2
    ([scored][n_vocab]).  Log-probabilities below (max - 16) are clamped; the rest are spread over 65,535 steps."""
    vocab = int(chunks_logits[0].shape[-1])
    scored = ctx - 1 - ctx // 2
    with open(path, "wb") as f:
        f.write(b"_logits_" + struct.pack("<iii", ctx, vocab, len(chunks_tokens)))
        for t in chunks_tokens:
            f.write(np.asarray(t, dtype="<i4").tobytes())
        for lg in chunks_logits:
            lg = np.asarray(lg, dtype=np.float32)
            if lg.shape != (scored, vocab):
                raise ValueError("a chunk's logits must cover positions ctx/2 .. ctx-2")
            for row in lg:
                mx = row.max()
                lse = np.float32(math.log(np.exp((row - mx).astype(np.float64)).sum()))
                lo = max(row.min(), mx - np.float32(16.0)) - mx - lse
                hi = -lse
                scale = np.float32((hi - lo) / 65535.0) if hi > lo else np.float32(1.0)
                q = np.clip(np.rint((np.maximum(row - mx - lse, lo) - lo) / scale), 0, 65535).astype("<u2")
                f.write(struct.pack("<ff", float(scale), float(lo)) + q.tobytes() + (b"\0\0" if vocab % 2 else b""))


class KldStats:
    """Running statistics of a model's logits against a base file's rows, with llama.cpp's definitions: the KL divergence sums
    base probabilities above e^-16 only, uncertainties are the standard error of the mean (zero under ten samples)."""

    def __init__(self):
        self.nll, self.nll_base, self.kld, self.p_diff, self.same_top = [], [], [], [], 0

    def add_rows(self, logits, scale, min_lp, q, targets) -> None:
        """logits fp32 [rows][n_vocab] of the scored positions; the base chunk's scale / min / q rows; the target tokens."""
        lg = np.asarray(logits, dtype=np.float32)
        mx = lg.max(axis=1, keepdims=True)
        lse = np.log(np.exp((lg - mx).astype(np.float64)).sum(axis=1, keepdims=True)).astype(np.float32)
        logp = lg - (mx + lse)
        base = scale[:, None].astype(np.float32) * q.astype(np.float32) + min_lp[:, None].astype(np.float32)
        rows = np.arange(lg.shape[0])
        tg = np.asarray(targets, dtype=np.int64)
        nll, nll_b = -logp[rows, tg], -base[rows, tg]
        keep = base > -16.0
        kld = np.where(keep, np.exp(base) * (base - logp), 0.0).astype(np.float64).sum(axis=1)
        self.nll += nll.tolist()
        self.nll_base += nll_b.tolist()
        self.kld += kld.tolist()
        self.p_diff += (np.exp(-nll) - np.exp(-nll_b)).astype(np.float32).tolist()
        self.same_top += int((lg.argmax(1) == base.argmax(1)).sum())

    @property
    def count(self) -> int:
        return len(self.kld)

    @staticmethod
    def _mean_unc(v):
        n = len(v)
        if not n:
            return 0.0, 0.0
        a = np.asarray(v, dtype=np.float64)
        mean = float(a.mean())
        var = float((a * a).mean()) - mean * mean
        return mean, math.sqrt(var / (n - 1)) if var > 0 and n > 10 else 0.0

    @staticmethod
    def _percentile(srt, frac: float) -> float:
        if frac <= 0:
            return float(srt[0])
        if frac >= 1:
            return float(srt[-1])
        p = frac * (len(srt) - 1)
        ip = int(p)
        p -= ip
        return float((1 - p) * srt[ip] + p * srt[min(ip + 1, len(srt) - 1)])

    def summary(self) -> dict:
        n = self.count
        if not n:
            return {"count": 0}
        lq, lb = self._mean_unc(self.nll), self._mean_unc(self.nll_base)
        a, b = np.asarray(self.nll, dtype=np.float64), np.asarray(self.nll_base, dtype=np.float64)
        cov = float(((a * b).mean() - a.mean() * b.mean()) / (n - 1)) if n >= 10 else 0.0
        ratio_unc = math.sqrt(max(0.0, lq[1] ** 2 + lb[1] ** 2 - 2 * cov))
        ks, ps = np.sort(np.asarray(self.kld, dtype=np.float32)), np.sort(np.asarray(self.p_diff, dtype=np.float32))
        med = lambda s: float(0.5 * (s[len(s) // 2] + s[len(s) // 2 - 1])) if len(s) % 2 == 0 else float(s[len(s) // 2])
        kld, dp = self._mean_unc(self.kld), self._mean_unc(self.p_diff)
        mse = self._mean_unc([x * x for x in self.p_diff])
        same = self.same_top / n
        return {"count": n, "ppl": math.exp(lq[0]), "ppl_unc": math.exp(lq[0]) * lq[1], "ppl_base": math.exp(lb[0]),
                "ppl_base_unc": math.exp(lb[0]) * lb[1], "cor_ln_ppl": cov / (lq[1] * lb[1]) if lq[1] and lb[1] else 0.0,
                "ln_ppl_ratio": lq[0] - lb[0], "ln_ppl_ratio_unc": ratio_unc, "kld_mean": kld[0], "kld_unc": kld[1], "kld_max": float(ks[-1]),
                "kld_min": float(ks[0]), "kld_median": med(ks),
                "kld_percentiles": {f"{100 * f:g}": self._percentile(ks, f) for f in (0.999, 0.99, 0.95, 0.9, 0.1, 0.05, 0.01, 0.001)},
                "dp_mean": dp[0], "dp_unc": dp[1], "dp_max": float(ps[-1]), "dp_min": float(ps[0]), "dp_median": med(ps),
                "dp_percentiles": {f"{100 * f:g}": self._percentile(ps, f) for f in (0.999, 0.99, 0.95, 0.9, 0.75, 0.25, 0.1, 0.05, 0.01, 0.001)},
                "dp_rms": math.sqrt(mse[0]), "same_top": same, "same_top_unc": math.sqrt(same * (1 - same) / (n - 1)) if n > 1 else 0.0}

    def report(self) -> str:
        """The summary in llama-perplexity's layout (nothing under 100 scored tokens, as there)."""
        if self.count < 100:
            return ""
        s = self.summary()
        L = ["====== Perplexity statistics ======",
             f"Mean PPL(Q)                   : {s['ppl']:10.6f} ± {s['ppl_unc']:10.6f}",
             f"Mean PPL(base)                : {s['ppl_base']:10.6f} ± {s['ppl_base_unc']:10.6f}",
             f"Cor(ln(PPL(Q)), ln(PPL(base))): {100 * s['cor_ln_ppl']:6.2f}%",
             f"Mean ln(PPL(Q)/PPL(base))     : {s['ln_ppl_ratio']:10.6f} ± {s['ln_ppl_ratio_unc']:10.6f}",
             "", "====== KL divergence statistics ======", f"Mean    KLD: {s['kld_mean']:10.6f} ± {s['kld_unc']:10.6f}",
             f"Maximum KLD: {s['kld_max']:10.6f}"]
        L += [f"{float(k):4.1f}%   KLD: {v:10.6f}" for k, v in list(s["kld_percentiles"].items())[:4]]
        L += [f"Median  KLD: {s['kld_median']:10.6f}"]
        L += [f"{float(k):4.1f}%   KLD: {v:10.6f}" for k, v in list(s["kld_percentiles"].items())[4:]]
        L += [f"Minimum KLD: {s['kld_min']:10.6f}", "", "====== Token probability statistics ======",
              f"Mean    Δp: {100 * s['dp_mean']:6.3f} ± {100 * s['dp_unc']:5.3f} %", f"Maximum Δp: {100 * s['dp_max']:6.3f}%",
              f"Median  Δp: {100 * s['dp_median']:6.3f}%", f"Minimum Δp: {100 * s['dp_min']:6.3f}%", f"RMS Δp    : {100 * s['dp_rms']:6.3f} %",
              f"Same top p: {100 * s['same_top']:6.3f} ± {100 * s['same_top_unc']:5.3f} %"]
        return "\n".join(L)
