"""Speculative decoding: draft proposers and the acceptance bookkeeping.

Sources of drafts (rust/engine/src/draft.rs:23-78, rust/engine/src/scheduler.rs:1163-1226):
* ``NgramProposer``  prompt-lookup: find the latest earlier occurrence of the sequence's last
  n-gram in its own tokens and propose what followed it;
* ``DraftModelProposer``  a small decoder that shares the target's block tables (its KV lives at
  the same slots of its own, thinner pool), catches up on the tokens it has not seen and then
  decodes ``k`` tokens greedily for the whole batch.

Verification feeds ``last token + drafts`` as one ragged chunk through the target and accepts the
longest prefix the target agrees with, plus the target's own next token (the exact rule for
greedy decoding, rust/engine/src/speculative.rs:103); rejected KV is rolled back by truncating
the block table. ``AdaptiveDraft`` shrinks or grows the draft length from the running acceptance
rate (rust/engine/src/speculative.rs:251-380).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.decoder import Decoder, KVCache, StepBatch
from ..models.weights import init_random_weights, make_shard_spec


class AdaptiveDraft:
    def __init__(self, k_max: int, k_min: int = 1, alpha: float = 0.2):
        self.k_max, self.k_min, self.alpha = k_max, k_min, alpha
        self.rate = 0.7
        self.proposed = self.accepted = 0

    def update(self, proposed: int, accepted: int) -> None:
        if proposed <= 0:
            return
        self.proposed += proposed
        self.accepted += accepted
        self.rate = (1 - self.alpha) * self.rate + self.alpha * (accepted / proposed)

    def length(self) -> int:
        # expected accepted tokens of a k-draft is sum_{i<=k} rate^i; stop growing when the marginal
        # token is accepted less than ~30 % of the time
        k, p = 0, 1.0
        while k < self.k_max:
            p *= self.rate
            if p < 0.3 and k >= self.k_min:
                break
            k += 1
        return max(self.k_min, k)


class NgramProposer:
    def __init__(self, k: int = 4, max_n: int = 3, min_n: int = 1, window: int = 4096):
        self.k, self.max_n, self.min_n, self.window = k, max_n, min_n, window

    def propose(self, tokens: Sequence[int], k: Optional[int] = None) -> List[int]:
        k = k or self.k
        toks = list(tokens[-self.window:])
        L = len(toks)
        for n in range(min(self.max_n, L - 1), self.min_n - 1, -1):
            tail = toks[L - n:]
            for start in range(L - n - 1, -1, -1):          # latest earlier match first
                if toks[start:start + n] == tail:
                    follow = toks[start + n:start + n + k]
                    if follow:
                        return follow
        return []


class DraftModelProposer:
    """Greedy k-token drafts from a small decoder that reuses the target's block tables."""

    def __init__(self, engine, draft_cfg, k: int = 4, seed: int = 1, weights=None):
        self.eng, self.cfg, self.k = engine, draft_cfg, k
        dev = engine.device
        self.spec = make_shard_spec(draft_cfg)
        self.weights = weights or init_random_weights(draft_cfg, dev, torch.bfloat16, seed)
        self.kv = KVCache(draft_cfg.num_layers, engine.kv.num_blocks, self.spec.hkv_local, engine.block_size,
                          draft_cfg.head_dim, dev)
        self.decoder = Decoder(draft_cfg, self.weights, self.kv, engine.ops, self.spec)
        self.computed: Dict[int, int] = {}                  # seq id -> tokens whose draft KV is stored

    def forget(self, seq_id: int) -> None:
        self.computed.pop(seq_id, None)

    def _batch(self, rows: List[tuple]) -> StepBatch:
        """rows: (request, start, tokens list) - one ragged chunk per request."""
        eng = self.eng
        bs = eng.block_size
        dev = eng.device
        ids, pos, slots, rseq, lrows, qst, kvl = [], [], [], [], [], [0], []
        max_blocks = max(len(eng.blocks.table(r.seq_id)) for r, _, _ in rows)
        tab = np.zeros((len(rows), max_blocks), dtype=np.int32)
        for i, (r, start, toks) in enumerate(rows):
            tb = eng.blocks.np_table(r.seq_id)
            tab[i, :tb.shape[0]] = tb
            p = np.arange(start, start + len(toks))
            ids += list(toks)
            pos += p.tolist()
            slots += (tb[p // bs] * bs + p % bs).tolist()
            rseq += [i] * len(toks)
            lrows.append(len(ids) - 1)
            qst.append(len(ids))
            kvl.append(start + len(toks))
        t = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
        n = [len(x[2]) for x in rows]
        return StepBatch(t(ids), t(pos), t(slots), t(rseq), torch.from_numpy(tab).to(dev), t(lrows),
                         num_seqs=len(rows), num_tokens=len(ids), max_kv_len=max(kvl), all_decode=False,
                         seq_lens=t(kvl), q_starts=t(qst), max_q_len=max(n), min_q_len=min(n))

    @torch.inference_mode()
    def propose_batch(self, reqs: List, k: Optional[int] = None) -> Dict[int, List[int]]:
        """Drafts for decode-phase requests (capacity for k extra slots must already be reserved)."""
        k = k or self.k
        if not reqs:
            return {}
        rows = []
        for r in reqs:
            done = min(self.computed.get(r.seq_id, 0), r.num_tokens - 1)
            rows.append((r, done, r.all_tokens[done:]))
        drafts: Dict[int, List[int]] = {r.seq_id: [] for r in reqs}
        for step in range(k):
            b = self._batch(rows)
            lg = self.decoder.forward(b)
            nxt = self.decoder.greedy_tokens(lg).tolist()
            new_rows = []
            for (r, start, toks), tok in zip(rows, nxt):
                drafts[r.seq_id].append(int(tok))
                new_rows.append((r, start + len(toks), [int(tok)]))
            rows = new_rows
        for r in reqs:
            # the draft cache is valid for the verified tokens only; accepted drafts are re-fed next time
            self.computed[r.seq_id] = r.num_tokens
        return drafts
