"""Continuous batching: admit -> prefill chunks -> decode / verify rows under a
token budget, with preemption when KV blocks run out.

Same contract as the reference scheduler (rust/engine/src/scheduler.rs:156-249 config,
:340-470 ``schedule``, :494-625 admission, :933-968 preemption): a step holds prefill
chunks, decode rows and speculative verify rows; decode rows are scheduled first and
reserve their budget; at most ``max_partial_prefills`` prompts are being chunked at a
time; when blocks run out the lowest-priority running request is preempted by
recompute (its blocks are freed and it re-enters the waiting queue keeping its output).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

from ..config import EngineConfig
from .block_manager import BlockManager
from .request import Request, RequestStatus


@dataclass
class ScheduledSeq:
    req: Request
    start: int                 # first token position fed this step
    count: int                 # number of tokens fed this step
    wants_logits: bool         # sample after this chunk
    verify: int = 0            # number of draft tokens among `count` (rows count = 1 + verify)


@dataclass
class ScheduledStep:
    seqs: List[ScheduledSeq] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    cow: List[Tuple[int, int]] = field(default_factory=list)     # (src block, dst block) copies
    cow_owner: List[Request] = field(default_factory=list)       # request each copy belongs to (same order as cow)
    expired: List[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(s.count for s in self.seqs)

    @property
    def all_decode(self) -> bool:
        return bool(self.seqs) and all(s.count == 1 and s.req.output for s in self.seqs)

    @property
    def empty(self) -> bool:
        return not self.seqs


class Scheduler:
    def __init__(self, cfg: EngineConfig, blocks: BlockManager, window: int = 0):
        self.cfg, self.blocks = cfg, blocks
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.window = window         # model-wide sliding window (0 when any layer attends fully)
        # swap preemption: the engine installs an object with swap_out(req) -> bool / swap_in(req) / drop(req)
        # that moves a request's KV blocks to host memory and back (rust/engine/src/kv_tier.rs)
        self.swapper = None
        # called with a request whose device-side state outside the block pool is stale or no longer needed
        # (recompute preemption, abort, expiry, finish): the draft-model proposer forgets its KV marks there
        self.on_drop = None
        self.now_override = None     # step control: judge deadlines with the leader's clock instead of the local one
        self.chunk_align = 0         # recurrent-state checkpoints: prompt chunks end on multiples of this
        self._refund = 0             # token budget given back by victims preempted inside the current schedule()
        self.stats = {"steps": 0, "preemptions": 0, "scheduled_tokens": 0}

    def _dropped(self, r: Request) -> None:
        if self.on_drop is not None:
            self.on_drop(r)

    # ------------------------------------------------------------------ queue
    def add(self, req: Request) -> None:
        req.status = RequestStatus.WAITING
        if self.cfg.scheduling_policy == "priority":
            # stable insert by (priority, arrival)
            idx = len(self.waiting)
            for i, r in enumerate(self.waiting):
                if (req.params.priority, req.arrival) < (r.params.priority, r.arrival):
                    idx = i
                    break
            self.waiting.insert(idx, req)
        else:
            self.waiting.append(req)

    def abort(self, request_id: str) -> Optional[Request]:
        for q in (self.running, self.waiting):
            for r in list(q):
                if r.request_id == request_id:
                    q.remove(r)
                    if r.swapped and self.swapper is not None:
                        self.swapper.drop(r)
                    self.blocks.free_seq(r.seq_id)
                    r.status = RequestStatus.ABORTED
                    r.finish_reason = "abort"
                    self._dropped(r)
                    return r
        return None

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ helpers
    def _salt(self, req: Request) -> bytes:
        return req.params.cache_salt.encode()

    def _preempt_one(self, step: ScheduledStep, protect: Request) -> bool:
        """Evict the most recently admitted / lowest-priority running request."""
        cands = [r for r in self.running if r is not protect]
        if not cands:
            return False
        victim = max(cands, key=lambda r: (r.params.priority, r.arrival))
        self.running.remove(victim)
        victim.draft = []
        if (self.cfg.preemption == "swap" and self.swapper is not None and victim.is_decode
                and self.swapper.swap_out(victim)):
            victim.swapped = True                 # KV kept (on the host): nothing to recompute
        else:
            victim.num_computed = 0
            self._dropped(victim)                 # its KV will be recomputed into other blocks
        self.blocks.free_seq(victim.seq_id)
        victim.status = RequestStatus.PREEMPTED
        victim.preemptions += 1
        self.waiting.appendleft(victim)
        step.preempted.append(victim)
        # take the victim's rows, its copy-on-write pairs (their destination block was just freed and may be
        # handed to another sequence inside this same schedule()) and its token budget back out of the step
        self._refund += sum(s.count for s in step.seqs if s.req is victim)
        step.seqs = [s for s in step.seqs if s.req is not victim]
        keep = [i for i, o in enumerate(step.cow_owner) if o is not victim]
        step.cow = [step.cow[i] for i in keep]
        step.cow_owner = [step.cow_owner[i] for i in keep]
        self.stats["preemptions"] += 1
        return True

    def _reserve(self, step: ScheduledStep, req: Request, total_tokens: int) -> bool:
        while not self.blocks.ensure_capacity(req.seq_id, total_tokens):
            if not self._preempt_one(step, protect=req):
                return False
        return True

    def _chunk(self, r, budget: int) -> int:
        """Tokens of ``r`` to feed this step. With ``chunk_align`` set (recurrent-state checkpoints) a prompt chunk
        ends on a multiple of it whenever one lies inside the chunk: before the budget's end, and before the last
        prompt token, so that a copy of the state can be kept on a block boundary close to the prompt's end."""
        n = min(r.remaining, budget)
        a = self.chunk_align
        if a and r.remaining > 1:
            end = min(r.num_computed + n, r.num_tokens - 1)
            cut = end // a * a
            if cut > r.num_computed:
                n = cut - r.num_computed
        return n

    def _take_refund(self) -> int:
        n, self._refund = self._refund, 0
        return n

    # ------------------------------------------------------------------ main
    def schedule(self) -> ScheduledStep:
        cfg = self.cfg
        step = ScheduledStep()
        now = self.now_override if self.now_override is not None else time.monotonic()
        budget = cfg.max_num_batched_tokens

        # deadlines
        for q in (self.running, self.waiting):
            for r in list(q):
                if r.deadline_passed(now):
                    q.remove(r)
                    if r.swapped and self.swapper is not None:
                        self.swapper.drop(r)
                    self.blocks.free_seq(r.seq_id)
                    r.status = RequestStatus.ABORTED
                    r.finish_reason = "timeout"
                    self._dropped(r)
                    step.expired.append(r)

        # 1. decode / verify rows of running requests (decode-first)
        decoders = [r for r in self.running if r.is_decode and r.num_tokens < cfg.max_model_len]
        prefilling = [r for r in self.running if not r.is_decode]
        for r in list(decoders):
            if r not in self.running:
                continue            # preempted while making room for an earlier one
            n_draft = len(r.draft)
            count = 1 + n_draft
            if budget < count:
                break
            ok = self._reserve(step, r, r.num_tokens + n_draft)
            budget += self._take_refund()
            if not ok:
                continue
            cow = self.blocks.cow_last_block(r.seq_id)
            if cow:
                step.cow.append(cow)
                step.cow_owner.append(r)
            step.seqs.append(ScheduledSeq(r, r.num_computed, count, True, verify=n_draft))
            budget -= count

        # 2. continue partially prefilled prompts
        partial = 0
        for r in prefilling:
            if r not in self.running or budget <= 0:
                continue
            n = self._chunk(r, budget)
            ok = self._reserve(step, r, r.num_computed + n)
            budget += self._take_refund()
            if not ok:
                continue
            step.seqs.append(ScheduledSeq(r, r.num_computed, n, n == r.remaining))
            budget -= n
            if n < r.remaining:
                partial += 1

        # 3. admit waiting requests
        while self.waiting and budget > 0 and len(self.running) < cfg.max_num_seqs:
            if partial >= cfg.max_partial_prefills:
                break
            r = self.waiting[0]
            if r.swapped and r.seq_id not in self.blocks.seqs:
                self.blocks.allocate(r.seq_id, [])             # fresh table: the KV comes back from the host
            elif r.seq_id not in self.blocks.seqs:
                cached = self.blocks.allocate(r.seq_id, r.all_tokens, self._salt(r))
                r.num_computed = cached
                r.num_cached = cached
            n = self._chunk(r, budget)
            need = self.blocks.blocks_needed(r.num_computed + n) - len(self.blocks.table(r.seq_id))
            if not self.blocks.can_allocate(max(need, 0)) or not self.blocks.ensure_capacity(r.seq_id, r.num_computed + n):
                # not enough room right now: leave it queued (its cached prefix stays referenced)
                if not self.running and not step.seqs:
                    # nothing else holds memory: the prompt can never fit
                    self.waiting.popleft()
                    self.blocks.free_seq(r.seq_id)
                    r.status = RequestStatus.ABORTED
                    r.finish_reason = "kv_capacity"
                    step.expired.append(r)
                    continue
                break
            self.waiting.popleft()
            r.status = RequestStatus.RUNNING
            self.running.append(r)
            if r.swapped:
                self.swapper.swap_in(r)
                r.swapped = False
                self.blocks.commit_tokens(r.seq_id, r.all_tokens, r.num_computed, self._salt(r))
            step.seqs.append(ScheduledSeq(r, r.num_computed, n, n == r.remaining))
            budget -= n
            if n < r.remaining:
                partial += 1

        self.stats["steps"] += 1
        self.stats["scheduled_tokens"] += step.num_tokens
        return step

    # ------------------------------------------------------------------ commit
    def commit(self, s: ScheduledSeq, new_tokens: List[int], accepted_drafts: int = 0, register: bool = True) -> None:
        """Account for a finished step of one sequence: `count - verify + accepted` fed tokens now
        have KV; `new_tokens` (possibly empty for a non-final prefill chunk) are appended."""
        r = s.req
        fed = s.count - s.verify + accepted_drafts
        r.num_computed = s.start + fed
        if s.verify:
            # tokens fed as drafts and accepted are already in new_tokens; rejected KV is rolled back
            self.blocks.truncate(r.seq_id, r.num_computed)
            r.draft = []
        r.output.extend(new_tokens)
        if register:          # launch-ahead commits a placeholder first and registers once the id is known
            self.blocks.commit_tokens(r.seq_id, r.all_tokens, r.num_computed, self._salt(r))
        if self.window:
            self.blocks.prune_window(r.seq_id, self.window)

    def finish(self, r: Request, reason: str) -> None:
        if r in self.running:
            self.running.remove(r)
        elif r in self.waiting:                    # a preempted request whose in-flight token ended it
            self.waiting.remove(r)
            if r.swapped and self.swapper is not None:
                self.swapper.drop(r)
                r.swapped = False
        self.blocks.free_seq(r.seq_id)
        r.status = RequestStatus.FINISHED
        r.finish_reason = reason
        self._dropped(r)
