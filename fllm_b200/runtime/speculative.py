"""Speculative decoding: draft proposers and the acceptance bookkeeping.

Sources of drafts (rust/engine/src/draft.rs:23-78, rust/engine/src/scheduler.rs:1163-1226):
* ``NgramProposer``  prompt-lookup: find the latest earlier occurrence of the sequence's last
  n-gram in its own tokens and propose what followed it;
* ``SuffixProposer``  the same lookup, then a shared index over everything the server generated before;
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


class SuffixProposer:
    """Drafts from what this server has generated before (rust/engine/src/draft.rs:365-446, the suffix source): a
    bounded index from the last `n` tokens of any finished output (or prompt) to the tokens that followed them.
    A lookup tries the sequence's own context first (the n-gram rule) and then the shared index, longest n first.
    Repeated answers, boiler-plate and code completions accept long drafts across requests."""

    MAGIC = b"FLLMSFX1"

    def __init__(self, k: int = 4, max_n: int = 4, min_n: int = 2, capacity: int = 200_000, max_documents: int = 4096):
        self.k, self.max_n, self.min_n, self.capacity = k, max_n, min_n, capacity
        self.own = NgramProposer(k, max_n=max_n, min_n=1)
        self.index: "Dict[tuple, List[int]]" = {}
        self.hits = self.lookups = 0
        self.documents: "List[List[int]]" = []          # what the index was built from: this is what a restart needs
        self.max_documents = max_documents

    # ------------------------------------------------------------------ disk tier
    def save(self, path: str, digest: bytes) -> None:
        """The observed documents in one file (the index is rebuilt on load): magic | digest length u32 | digest |
        document count u64 | per document: token count u32, tokens i32. Written under a temporary name and renamed,
        so a crash leaves the old file or none (rust/engine/src/mem/suffix_tier.rs:1-16 keeps the same kind of file,
        one per model fingerprint, so that speculation does not start cold after a restart)."""
        import os
        import struct
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(self.MAGIC + struct.pack("<I", len(digest)) + digest + struct.pack("<Q", len(self.documents)))
            for d in self.documents:
                f.write(struct.pack("<I", len(d)) + struct.pack(f"<{len(d)}i", *d))
        os.replace(tmp, path)

    def load(self, path: str, digest: bytes) -> int:
        """Re-index the documents of a file written for the same model digest; a missing, foreign, truncated or damaged
        file counts as absent. Returns the number of documents taken."""
        import os
        import struct
        try:
            raw = open(path, "rb").read()
        except OSError:
            return 0
        try:
            if raw[:8] != self.MAGIC:
                return 0
            (dl,) = struct.unpack_from("<I", raw, 8)
            if dl > 256 or raw[12:12 + dl] != digest:
                return 0
            at = 12 + dl
            (count,) = struct.unpack_from("<Q", raw, at)
            at += 8
            if count > (16 << 20):
                return 0
            docs = []
            for _ in range(count):
                (n,) = struct.unpack_from("<I", raw, at)
                at += 4
                if at + 4 * n > len(raw):
                    return 0
                docs.append(list(struct.unpack_from(f"<{n}i", raw, at)))
                at += 4 * n
        except struct.error:
            return 0
        for d in docs:
            self.observe(d)
        return len(docs)

    def observe(self, tokens: Sequence[int]) -> None:
        """Index a finished sequence (prompt + output)."""
        toks = [int(t) for t in tokens]
        if toks and max(toks) < (1 << 31):
            self.documents.append(toks)
            if len(self.documents) > self.max_documents:
                del self.documents[0]
        for n in range(self.min_n, self.max_n + 1):
            for i in range(len(toks) - n):
                if len(self.index) >= self.capacity:
                    self.index.pop(next(iter(self.index)))          # oldest entry out
                self.index[tuple(toks[i:i + n])] = toks[i + n:i + n + self.k]

    def propose(self, tokens: Sequence[int], k: Optional[int] = None) -> List[int]:
        k = k or self.k
        self.lookups += 1
        got = self.own.propose(tokens, k)
        if got:
            return got
        toks = list(tokens[-self.max_n:])
        for n in range(min(self.max_n, len(toks)), self.min_n - 1, -1):
            nxt = self.index.get(tuple(toks[len(toks) - n:]))
            if nxt:
                self.hits += 1
                return nxt[:k]
        return []


class DraftTree:
    """A tree of draft tokens for one sequence (rust/engine/src/speculative.rs:146 ``verify_tree``): node i carries
    `tokens[i]` and hangs under `parents[i]` (-1 = directly under the last committed token); parents come before their
    children. At most 64 nodes, so a node's visibility over the tree is one 64-bit word."""

    def __init__(self, tokens: Sequence[int], parents: Sequence[int]):
        if len(tokens) != len(parents) or not 0 < len(tokens) <= 64:
            raise ValueError("a draft tree has 1 to 64 nodes, one parent per node")
        for i, p in enumerate(parents):
            if not -1 <= p < i:
                raise ValueError("parents must precede their children")
        self.tokens, self.parents = [int(t) for t in tokens], [int(p) for p in parents]

    def __len__(self) -> int:
        return len(self.tokens)

    @classmethod
    def from_chains(cls, chains: Sequence[Sequence[int]]) -> "DraftTree":
        """Merge several candidate continuations into a prefix tree."""
        tokens, parents, index = [], [], {}
        for ch in chains:
            par = -1
            for t in ch:
                key = (par, int(t))
                if key not in index:
                    if len(tokens) == 64:
                        break
                    index[key] = len(tokens)
                    tokens.append(int(t))
                    parents.append(par)
                par = index[key]
        return cls(tokens, parents)

    def depths(self) -> List[int]:
        d = []
        for p in self.parents:
            d.append(0 if p < 0 else d[p] + 1)
        return d

    def masks(self) -> List[int]:
        """Per node: bit j set when node j is the node itself or one of its ancestors (the row of the M x M mask)."""
        m = []
        for i, p in enumerate(self.parents):
            m.append((1 << i) | (m[p] if p >= 0 else 0))
        return m

    def masks_i64(self) -> List[int]:
        """The masks as signed 64-bit integers (what an int64 tensor holds)."""
        return [x - (1 << 64) if x >= (1 << 63) else x for x in self.masks()]

    def verify_greedy(self, root_target: int, node_targets: Sequence[int]) -> "tuple[List[int], int]":
        """The longest root-to-node path the target agrees with. `root_target` is the target's token after the
        committed context, `node_targets[i]` its token after node i (given the node's ancestors). Returns
        (indices of the accepted nodes in path order, the token to emit after them)."""
        children: Dict[int, List[int]] = {}
        for i, p in enumerate(self.parents):
            children.setdefault(p, []).append(i)
        path, cur, want = [], -1, int(root_target)
        while True:
            nxt = next((c for c in children.get(cur, []) if self.tokens[c] == want), None)
            if nxt is None:
                return path, want
            path.append(nxt)
            cur, want = nxt, int(node_targets[nxt])


class DraftModelProposer:
    """k-token drafts from a small decoder that reuses the target's block tables.

    One call = one ragged catch-up step (the tokens the draft model has not seen, built on the host into one
    pinned staging array and sent with a single copy) and k - 1 decode steps whose inputs are made on the
    device from the previous step's tokens (positions + 1, slots from the block table), so nothing crosses
    the bus between draft tokens; the k tokens come back in one read at the end. Greedy requests take the
    draft's argmax; sampled requests draw from the draft's temperature-scaled distribution with their own
    counter-based stream and keep the logit rows, which the exact acceptance rule needs
    (rust/engine/src/speculative.rs:103). Under tensor parallelism the draft is sharded over the same group
    when its head counts divide, otherwise every rank runs a whole copy; both give every rank the same drafts.
    """

    DRAFT_SEED_SALT = 0x5DEECE66D

    def __init__(self, engine, draft_cfg, k: int = 4, seed: int = 1, weights=None):
        self.eng, self.cfg, self.k = engine, draft_cfg, k
        dev = engine.device
        tp, rank, group = 1, 0, None
        etp = getattr(engine.par, "tp", 1)
        if etp > 1 and weights is None and draft_cfg.num_heads % etp == 0 and draft_cfg.num_kv_heads % etp == 0:
            tp, rank, group = etp, engine.tp_rank, engine.tp_group
        self.spec = make_shard_spec(draft_cfg, tp, rank)
        self.weights = weights or init_random_weights(draft_cfg, dev, torch.bfloat16, seed, tp=tp, tp_rank=rank)
        self.kv = KVCache(draft_cfg.num_layers, engine.kv.num_blocks, self.spec.hkv_local, engine.block_size,
                          draft_cfg.head_dim, dev)
        self.decoder = Decoder(draft_cfg, self.weights, self.kv, engine.ops, self.spec, group)
        self.computed: Dict[int, int] = {}                  # seq id -> tokens whose draft KV is stored
        self._stage: Optional[torch.Tensor] = None          # pinned host staging, grown on demand
        self.h2d_copies = 0                                 # copies issued by the last propose_batch (tests read it)

    def forget(self, seq_id: int) -> None:
        self.computed.pop(seq_id, None)

    def _staging(self, n: int) -> torch.Tensor:
        if self._stage is None or self._stage.numel() < n:
            cap = max(n, 4096)
            self._stage = torch.empty(cap, dtype=torch.int32, pin_memory=self.eng.is_cuda)
        return self._stage[:n]

    def _first_batch(self, rows: List[tuple]) -> StepBatch:
        """rows: (request, start, tokens list) - one ragged chunk per request, one host-to-device copy."""
        eng = self.eng
        bs = eng.block_size
        B = len(rows)
        T = sum(len(t) for _, _, t in rows)
        max_blocks = max(len(eng.blocks.table(r.seq_id)) for r, _, _ in rows)
        # layout of the staging array: ids | pos | slots | row_seq | logit_rows | q_starts | kv_lens | table
        sizes = [T, T, T, T, B, B + 1, B, B * max_blocks]
        offs = np.concatenate([[0], np.cumsum(sizes)])
        stage = self._staging(int(offs[-1]))
        h = stage.numpy()
        ids, pos, slots, rseq, lrows, qst, kvl, tab = (h[offs[j]:offs[j + 1]] for j in range(8))
        tab = tab.reshape(B, max_blocks)
        tab[:] = 0
        at = 0
        qst[0] = 0
        for i, (r, start, toks) in enumerate(rows):
            tb = eng.blocks.np_table(r.seq_id)
            tab[i, :tb.shape[0]] = tb
            n = len(toks)
            p = np.arange(start, start + n)
            ids[at:at + n] = toks
            pos[at:at + n] = p
            slots[at:at + n] = tb[p // bs] * bs + p % bs
            rseq[at:at + n] = i
            at += n
            lrows[i] = at - 1
            qst[i + 1] = at
            kvl[i] = start + n
        d = stage.to(eng.device, non_blocking=eng.is_cuda)
        self.h2d_copies += 1
        v = [d[offs[j]:offs[j + 1]] for j in range(8)]
        ns = [len(x[2]) for x in rows]
        return StepBatch(v[0], v[1], v[2], v[3], v[7].view(B, max_blocks), v[4],
                         num_seqs=B, num_tokens=T, max_kv_len=int(kvl.max()), all_decode=False,
                         seq_lens=v[6], q_starts=v[5], max_q_len=max(ns), min_q_len=min(ns))

    def _next_batch(self, prev: StepBatch, tokens: torch.Tensor, first: bool) -> StepBatch:
        """The decode step after `prev`, made on the device: every sequence feeds the token it just drew."""
        B = prev.num_seqs
        bs = self.eng.block_size
        if first:
            ar = torch.arange(B, dtype=torch.int32, device=tokens.device)
            pos = prev.seq_lens.clone()                      # the new token sits at the old visible length
            rseq, lrows = ar, ar
            qst = torch.arange(B + 1, dtype=torch.int32, device=tokens.device)
        else:
            pos = prev.positions + 1
            rseq, lrows, qst = prev.row_seq, prev.logit_rows, prev.q_starts
        blk = torch.gather(prev.block_tables, 1, (pos // bs).long().view(B, 1)).view(B)
        slots = (blk * bs + pos % bs).to(torch.int32)
        return StepBatch(tokens.to(torch.int32), pos, slots, rseq, prev.block_tables, lrows,
                         num_seqs=B, num_tokens=B, max_kv_len=prev.max_kv_len + 1, all_decode=True,
                         seq_lens=pos + 1, q_starts=qst, max_q_len=1, min_q_len=1)

    def _draw(self, reqs: List, lg: torch.Tensor, step: int) -> torch.Tensor:
        """Next draft token per row: argmax, or a draw from softmax(logits / T) for sampled requests."""
        full = self.decoder.full_logits(lg)
        toks = self.decoder.greedy_tokens(lg)
        rows = [i for i, r in enumerate(reqs) if r.params.spec_mode == "sampled"]
        if not rows:
            return toks, None
        from .sampler import _row_params
        from ..ops.reference import sample_reference
        idx = torch.tensor(rows, dtype=torch.long, device=lg.device)
        sub = full.index_select(0, idx).float().contiguous()
        prm = []
        for i in rows:
            t = list(_row_params(reqs[i], len(reqs[i].output) + step, self.eng.cfg.seed))
            t[8] = (t[8] ^ self.DRAFT_SEED_SALT) & 0xFFFFFFFFFFFF        # a stream of its own
            prm.append(tuple(t))
        if lg.is_cuda:
            from ..ops.native import pack_sample_rows
            pb = torch.frombuffer(bytearray(pack_sample_rows(prm)), dtype=torch.uint8).to(lg.device)
            ids = self.eng.ops.sample(sub, pb)
        else:
            ids = torch.tensor([sample_reference(sub[j], p[0], 0, 1.0, 0.0, p[8], p[7]) for j, p in enumerate(prm)],
                               dtype=torch.int32)
        toks = toks.clone()
        toks[idx] = ids.to(toks.dtype)
        return toks, (idx, full.index_select(0, idx))

    @torch.inference_mode()
    def propose_batch(self, reqs: List, k: Optional[int] = None) -> Dict[int, List[int]]:
        """Drafts for decode-phase requests (capacity for k extra slots must already be reserved)."""
        k = k or self.k
        if not reqs:
            return {}
        self.h2d_copies = 0
        rows = []
        for r in reqs:
            done = min(self.computed.get(r.seq_id, 0), r.num_tokens - 1)
            rows.append((r, done, r.all_tokens[done:]))
        b = self._first_batch(rows)
        drawn, kept = [], []
        for step in range(k):
            lg = self.decoder.forward(b)
            toks, keep = self._draw(reqs, lg, step)
            drawn.append(toks)
            kept.append(keep)
            if step + 1 < k:
                b = self._next_batch(b, toks, first=(step == 0))
        host = torch.stack(drawn, 1).cpu().tolist()          # [B, k], one read for the whole call
        drafts: Dict[int, List[int]] = {}
        for i, r in enumerate(reqs):
            drafts[r.seq_id] = [int(t) for t in host[i]]
            r.draft_logits = None
            # the draft cache is valid for the verified tokens only; accepted drafts are re-fed next time
            self.computed[r.seq_id] = r.num_tokens
        if kept[0] is not None:
            idx = kept[0][0].tolist()
            stack = torch.stack([kp[1] for kp in kept], 1)   # [n sampled, k, vocab]
            for j, i in enumerate(idx):
                reqs[i].draft_logits = stack[j]
        return drafts
