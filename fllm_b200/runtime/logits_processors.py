"""Logit processors that run on the host before the device sampler: locally typical sampling,
the DRY repetition penalty, Mirostat (versions 1 and 2) and multi-token banned sequences.

They are the rarely used part of the sampling contract (rust/engine/src/sampling.rs:6-49), so they
are kept out of the CUDA sampler: each one edits the fp32 logit row of its request (a ban or a
penalty), and the device sampler then applies the common filters (penalties, bias, mask,
temperature, top-k / top-p / min-p, the seeded Gumbel draw) to the edited row. Typical sampling and
Mirostat look at the distribution at the request's temperature; combined with count penalties they
see the logits before those penalties.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

NEG_INF = float("-inf")


def typical_keep_mask(logits: torch.Tensor, typical_p: float, temperature: float) -> torch.Tensor:
    """Locally typical sampling (Meister et al. 2022): keep the tokens whose surprise is closest to the
    entropy of the distribution, smallest set with mass >= typical_p. Returns a bool mask [vocab]."""
    t = temperature if temperature > 0 else 1.0
    logp = torch.log_softmax(logits.float() / t, -1)
    p = logp.exp()
    ent = -(p * torch.where(p > 0, logp, torch.zeros_like(logp))).sum()
    dev = (-logp - ent).abs()
    dev = torch.where(torch.isfinite(dev), dev, torch.full_like(dev, float("inf")))
    order = torch.argsort(dev, stable=True)
    cum = p[order].cumsum(0)
    last = int((cum < typical_p).sum().item())            # index of the first position reaching the mass
    keep = torch.zeros_like(p, dtype=torch.bool)
    keep[order[: last + 1]] = True
    return keep


def dry_penalties(context: Sequence[int], multiplier: float, base: float = 1.75, allowed_length: int = 2,
                  breakers: Sequence[int] = (), last_n: int = 1024) -> Dict[int, float]:
    """DRY ("don't repeat yourself"): a token that would extend a sequence already present in the
    context by its n-th repeated token is penalised by multiplier * base ** (n - allowed_length) once
    n >= allowed_length. Sequence breakers stop a match. -> {token: penalty to subtract}."""
    if multiplier <= 0 or not context:
        return {}
    ctx = list(context[-last_n:]) if last_n > 0 else list(context)
    L = len(ctx)
    brk = set(int(b) for b in breakers)
    if ctx[-1] in brk:
        return {}
    out: Dict[int, float] = {}
    for i in range(L - 1):                                  # ctx[i] ends an earlier copy of the current suffix
        if ctx[i] != ctx[-1]:
            continue
        n = 1
        while i - n >= 0 and ctx[i - n] == ctx[L - 1 - n] and ctx[i - n] not in brk:
            n += 1
            if n > 256:
                break
        if n >= allowed_length:
            tok = ctx[i + 1]                                # the token that followed the earlier copy
            if tok in brk:
                continue
            pen = multiplier * base ** (n - allowed_length)
            if pen > out.get(tok, 0.0):
                out[tok] = pen
    return out


def banned_by_sequences(context: Sequence[int], bad_words: Sequence[Sequence[int]]) -> List[int]:
    """Last tokens of the banned sequences whose other tokens are the current suffix of the context
    (a one-token sequence is always banned)."""
    out = []
    for seq in bad_words:
        seq = [int(t) for t in seq]
        if not seq:
            continue
        k = len(seq) - 1
        if k == 0 or (len(context) >= k and list(context[-k:]) == seq[:-1]):
            out.append(seq[-1])
    return out


class Mirostat:
    """Mirostat (Basu et al. 2021), one instance per request. Version 2 drops the tokens whose surprise
    exceeds mu; version 1 estimates the Zipf exponent s of the distribution from its `m` most probable
    tokens, turns mu into a top-k cut k = ((eps * 2^mu) / (1 - n^-eps))^(1/s) with eps = s - 1, and keeps
    the k most probable tokens. In both, one of the kept tokens is drawn and mu moves by
    eta * (tau - observed surprise)."""

    def __init__(self, tau: float = 5.0, eta: float = 0.1, version: int = 2, m: int = 100):
        self.tau, self.eta, self.version, self.m = tau, eta, int(version), int(m)
        self.mu = 2.0 * tau
        self._logp2: Optional[torch.Tensor] = None

    def zipf_cut(self, logp2: torch.Tensor) -> int:
        """Version 1's k for the current mu (at least 1, at most the vocabulary)."""
        n = logp2.shape[-1]
        m = max(2, min(self.m, n))
        top = torch.topk(logp2, m).values.double() * math.log(2.0)          # natural-log probabilities, sorted
        i = torch.arange(1, m, dtype=torch.float64)
        t = torch.log((i + 1) / i)                                          # ln((i+1)/i)
        b = top[:-1] - top[1:]                                              # ln(p_i / p_{i+1})
        ok = torch.isfinite(b)
        den = float((t[ok] * t[ok]).sum())
        s_hat = float((t[ok] * b[ok]).sum()) / den if den > 0 else 1.0
        eps = s_hat - 1.0
        if abs(eps) < 1e-6 or s_hat <= 0:
            return n
        try:
            k = ((eps * 2.0 ** self.mu) / (1.0 - float(n) ** (-eps))) ** (1.0 / s_hat)
        except (OverflowError, ZeroDivisionError):
            return n
        if not math.isfinite(k) or isinstance(k, complex):
            return n
        return max(1, min(n, int(round(k))))

    def keep_mask(self, logits: torch.Tensor, temperature: float) -> torch.Tensor:
        t = temperature if temperature > 0 else 1.0
        logp2 = torch.log_softmax(logits.float() / t, -1) / math.log(2.0)
        if self.version == 1:
            k = self.zipf_cut(logp2)
            keep = torch.zeros_like(logp2, dtype=torch.bool)
            keep[torch.topk(logp2, k).indices] = True
        else:
            keep = (-logp2) <= self.mu
        if not bool(keep.any()):
            keep[int(torch.argmax(logp2))] = True
        trunc = torch.where(keep, logp2, torch.full_like(logp2, NEG_INF))
        self._logp2 = trunc - torch.logsumexp(trunc * math.log(2.0), -1) / math.log(2.0)   # renormalised over the kept set
        return keep

    def observe(self, token: int) -> None:
        if self._logp2 is None:
            return
        s = -float(self._logp2[token])
        if math.isfinite(s):
            self.mu -= self.eta * (s - self.tau)
        self._logp2 = None


def apply_before_sampling(req, row: torch.Tensor, position: int) -> None:
    """Edit the logit row of `req` in place. `position` = number of output tokens that precede this row
    (a verify row of speculative decoding sees the draft tokens before it as context)."""
    p = req.params
    ctx = req.prompt + req.output[:position] if position <= len(req.output) else req.prompt + req.output + req.draft[: position - len(req.output)]
    if p.bad_words:
        for t in banned_by_sequences(ctx, p.bad_words):
            if 0 <= t < row.shape[0]:
                row[t] = NEG_INF
    if p.dry_multiplier > 0.0:
        for t, pen in dry_penalties(ctx, p.dry_multiplier, p.dry_base, p.dry_allowed_length, p.dry_sequence_breakers,
                                    p.dry_penalty_last_n).items():
            if 0 <= t < row.shape[0]:
                row[t] -= pen
    if p.typical_p < 1.0:
        row.masked_fill_(~typical_keep_mask(row, p.typical_p, p.temperature), NEG_INF)
    if p.mirostat_mode != 0:
        if req.mirostat is None:
            req.mirostat = Mirostat(p.mirostat_tau, p.mirostat_eta, version=1 if p.mirostat_mode == 1 else 2)
        row.masked_fill_(~req.mirostat.keep_mask(row, p.temperature), NEG_INF)


def observe_sampled(req, token: int) -> None:
    if req.params.mirostat_mode != 0 and req.mirostat is not None:
        req.mirostat.observe(int(token))
