"""Host side of sampling: turns per-request parameters into the packed rows the
device sampler reads, keeps per-request draw counters and sparse penalty lists
(unique token ids + counts), and runs the sampler only on rows that need more than
a greedy pick. A CPU restatement of the same filters serves machines without a GPU."""
from __future__ import annotations

from collections import Counter
from typing import List

import numpy as np
import torch

from ..ops.reference import sample_reference
from .logits_processors import apply_before_sampling, observe_sampled


def _row_params(req, draw: int, default_seed: int):
    p = req.params
    seed = p.seed if p.seed is not None else (default_seed * 1000003 + req.seq_id) & 0xFFFFFFFFFFFF
    return (float(p.temperature), float(p.top_p), float(p.min_p), float(p.repetition_penalty),
            float(p.presence_penalty), float(p.frequency_penalty), int(p.top_k), int(draw), int(seed))


def sample_step(engine, step, logits: torch.Tensor, greedy: torch.Tensor) -> torch.Tensor:
    """logits: [R, vocab] for the step's logit rows (verify rows included). Returns ids [R]."""
    rows = []           # (row index, request)
    r_i = 0
    for s in step.seqs:
        if not s.wants_logits:
            continue
        n = s.count if s.verify else 1
        # verify rows of a sampled request are decided by the speculative acceptance rule, not drawn here
        if not (s.verify and s.req.params.spec_mode == "sampled"):
            for j in range(n):
                if s.req.params.needs_full_sampler:
                    rows.append((r_i + j, s.req, len(s.req.output) + j))
        r_i += n
    if not rows:
        return greedy
    out = greedy.clone()
    idx = torch.tensor([r for r, _, _ in rows], dtype=torch.long, device=logits.device)
    sub = logits.index_select(0, idx).float().contiguous()
    vocab = sub.shape[1]
    raw_lsm = {}                                       # log-probabilities of the raw distribution (before any filter)
    for i, (_, req, _) in enumerate(rows):
        if req.params.logprobs:
            raw_lsm[i] = torch.log_softmax(sub[i], -1)
            if req.params.top_logprobs > 0:
                # stable order: among equal log-probabilities (bf16 logits tie often) the lower token id comes
                # first, which is the token a greedy pick returns
                lp, tid = torch.sort(raw_lsm[i], descending=True, stable=True)
                n_alt = min(req.params.top_logprobs, vocab)
                req.top_logprobs.append(list(zip(tid[:n_alt].tolist(), lp[:n_alt].tolist())))
    for i, (_, req, draw) in enumerate(rows):          # typical-p, DRY, Mirostat, banned sequences: edits of the row
        if req.params.needs_host_processors:
            apply_before_sampling(req, sub[i], draw)
    params = [_row_params(req, draw, engine.cfg.seed) for _, req, draw in rows]
    # sparse penalty / bias lists
    pen_lists, bias_lists = [], []
    for _, req, _ in rows:
        p = req.params
        if p.repetition_penalty != 1.0 or p.presence_penalty or p.frequency_penalty:
            c = Counter(req.output)
            if p.repetition_penalty != 1.0:
                for t in set(req.prompt):
                    c.setdefault(t, 0)
            pen_lists.append(c)
        else:
            pen_lists.append({})
        bias = dict(p.logit_bias or {})
        for t in (p.bad_words_ids or ()):
            bias[int(t)] = float("-inf")
        bias_lists.append(bias)
    allow = None
    if any(req.params.allowed_token_ids is not None or req.params.guided is not None for _, req, _ in rows):
        words = (vocab + 31) // 32
        allow_np = np.full((len(rows), words), 0xFFFFFFFF, dtype=np.uint32)
        for i, (_, req, _) in enumerate(rows):
            a = req.params.allowed_token_ids
            if a is not None:
                allow_np[i] = 0
                for t in a:
                    allow_np[i, t >> 5] |= np.uint32(1 << (t & 31))
            if req.params.guided is not None:          # structured output: the grammar's mask for this state
                allow_np[i] &= req.params.guided.mask_words(vocab)
        allow = allow_np
    if logits.is_cuda:
        from ..ops.native import pack_sample_rows
        dev = logits.device
        prm = torch.frombuffer(bytearray(pack_sample_rows(params)), dtype=torch.uint8).to(dev)

        def to_dev(lists, as_float):
            width = max((len(l) for l in lists), default=0)
            if width == 0:
                return None, None
            ids = np.full((len(lists), width), -1, dtype=np.int32)
            vals = np.zeros((len(lists), width), dtype=np.float32 if as_float else np.int32)
            for i, l in enumerate(lists):
                for j, (k, v) in enumerate(l.items()):
                    ids[i, j] = k
                    vals[i, j] = v
            return torch.from_numpy(ids).to(dev), torch.from_numpy(vals).to(dev)

        pen_ids, pen_cnt = to_dev(pen_lists, False)
        b_ids, b_vals = to_dev(bias_lists, True)
        allow_t = torch.from_numpy(allow.view(np.int32)).to(dev) if allow is not None else None
        ids = engine.ops.sample(sub, prm, pen_ids, pen_cnt, b_ids, b_vals, allow_t)
    else:
        picked: List[int] = []
        for i, (_, req, draw) in enumerate(rows):
            x = sub[i].clone()
            p = req.params
            for t, cnt in pen_lists[i].items():
                v = x[t]
                if p.repetition_penalty != 1.0:
                    v = v / p.repetition_penalty if v > 0 else v * p.repetition_penalty
                if cnt > 0:
                    v = v - p.presence_penalty - p.frequency_penalty * cnt
                x[t] = v
            for t, bv in bias_lists[i].items():
                x[t] = x[t] + bv
            if allow is not None and (p.allowed_token_ids is not None or p.guided is not None):
                bits = np.unpackbits(allow[i].view(np.uint8), bitorder="little")[:vocab].astype(bool)
                x = torch.where(torch.from_numpy(bits), x, torch.full_like(x, float("-inf")))
            prm = params[i]
            picked.append(sample_reference(x, prm[0], prm[6], prm[1], prm[2], prm[8], prm[7]))
        ids = torch.tensor(picked, dtype=torch.int32, device=logits.device)
    if raw_lsm:
        picked_ids = ids.tolist()
        for i, (_, req, _) in enumerate(rows):
            if i in raw_lsm:
                req.logprobs.append(float(raw_lsm[i][picked_ids[i]]))
    if any(req.params.mirostat_mode for _, req, _ in rows):
        for (_, req, _), t in zip(rows, ids.tolist()):
            observe_sampled(req, t)
    out[idx] = ids.to(out.dtype)
    return out
