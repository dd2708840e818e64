"""Step control across the ranks of one model instance: what lets ONE HTTP front end drive a
tensor- / pipeline-parallel group.

Every rank runs the same engine and the same deterministic scheduler (SPMD). What the ranks
cannot know by themselves is what arrived over HTTP on rank 0, so before every step the leader
broadcasts a small control message: the requests admitted since the previous message (id, prompt
ids, sampling parameters, arrival time), the aborts, the leader's clock (deadlines are judged
with ONE clock), and whether a step follows. Followers apply the message and step; their
schedulers then take exactly the leader's decisions, and the per-step arrays never travel.
The reference broadcasts a full step descriptor - ids, lengths, block tables, logit rows - from
rank 0 each step (rust/engine/src/parallel/decoder_shard.rs:611-622) to worker loops
(rust/engine/src/parallel/group.rs:116-156); here the schedule is recomputed locally instead,
which keeps the message a few hundred bytes.

The channel is a gloo (CPU) group beside the data-plane group, so control traffic never queues
behind kernels. Any failure of a control collective surfaces as ``CommError`` ("[comm] ...")
inside the group's deadline: the leader stops admitting work and reports not-ready; followers
leave their loop (rust/engine/src/parallel/ctx.rs:108-123 is the reference's poisoned-group rule).
"""
from __future__ import annotations

import dataclasses
import datetime
import time
from typing import List, Optional

import torch.distributed as dist

from ..comm.group import CommError
from .request import SamplingParams

KEEPALIVE_S = 2.0           # an idle leader still talks this often, so followers can tell "idle" from "gone"


def params_to_wire(p: SamplingParams) -> dict:
    """Sampling parameters as plain data. A grammar object does not travel; the request fields it was built from
    (`guided_spec`) do, and every rank rebuilds the same recogniser from them."""
    if p.guided is not None and not p.guided_spec:
        raise ValueError("a grammar-constrained request needs its source fields (guided_spec) to reach the other ranks")
    d = dataclasses.asdict(dataclasses.replace(p, guided=None))
    d.pop("guided", None)
    if d.get("logit_bias"):
        d["logit_bias"] = {int(k): float(v) for k, v in d["logit_bias"].items()}
    return d


def params_from_wire(d: dict, guided_builder=None) -> SamplingParams:
    """`guided_builder(spec)` rebuilds the grammar object of a constrained request (server.app.make_guided_builder)."""
    d = dict(d)
    if d.get("logit_bias"):
        d["logit_bias"] = {int(k): float(v) for k, v in d["logit_bias"].items()}
    sp = SamplingParams(**d)
    if sp.guided_spec:
        if guided_builder is None:
            raise ValueError("a grammar-constrained request arrived but this rank has no grammar builder")
        sp.guided = guided_builder(sp.guided_spec)
    return sp


class ControlChannel:
    """Object broadcast from rank 0 over a dedicated gloo group."""

    def __init__(self, timeout_s: float = 30.0, ranks: Optional[List[int]] = None):
        if not dist.is_initialized():
            raise RuntimeError("step control needs an initialised process group")
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.ranks = list(ranks) if ranks is not None else list(range(self.world))
        self.leader = self.ranks[0]
        self.pg = dist.new_group(self.ranks, backend="gloo", timeout=datetime.timedelta(seconds=timeout_s))
        self.broken = False

    @property
    def is_leader(self) -> bool:
        return self.rank == self.leader

    def bcast(self, obj=None):
        """Leader: send `obj`. Follower: return what the leader sent. Raises CommError when the group is broken
        (a rank left, a rank never joined, the deadline ran out)."""
        if self.broken:
            raise CommError("control channel is closed after an earlier failure")
        box = [obj if self.is_leader else None]
        try:
            dist.broadcast_object_list(box, src=self.leader, group=self.pg)
        except Exception as e:                    # RuntimeError / DistBackendError: timeouts, closed connections
            self.broken = True
            raise CommError(f"step control broadcast failed: {e}") from e
        return box[0]


class StepController:
    """Leader side: queues admissions / aborts and announces every step. Follower side: ``follow()``."""

    def __init__(self, engine, channel: ControlChannel, guided_builder=None):
        """guided_builder(spec) -> grammar object: how a follower rebuilds the recogniser of a constrained request
        (server.app.make_guided_builder(engine, tokenizer, tool_parser)); None refuses such requests on followers."""
        self.engine, self.ch, self.guided_builder = engine, channel, guided_builder
        self.pending: List[dict] = []
        self.last_sent = time.monotonic()
        self.steps = 0
        self.steps_seen = 0          # follower-side counter for callers that drive apply() themselves

    # ---------------------------------------------------------------- leader
    def admit(self, rid: str, prompt: List[int], params: SamplingParams) -> None:
        """Add a request on the leader and queue it for the followers. Validation errors are raised
        before anything is queued, so a refused request never reaches the other ranks."""
        wire = params_to_wire(params)
        self.engine.add_request(prompt, params, request_id=rid)
        req = self.engine.requests[rid]
        self.pending.append({"op": "add", "rid": rid, "prompt": list(req.prompt), "params": wire, "arrival": req.arrival})

    def abort(self, rid: str) -> None:
        self.engine.abort_request(rid)
        self.pending.append({"op": "abort", "rid": rid})

    def announce(self, step: bool, stop: bool = False) -> None:
        now = time.monotonic()
        msg = {"cmds": self.pending, "step": bool(step), "stop": bool(stop), "now": now}
        self.pending = []
        self.ch.bcast(msg)
        self.last_sent = now
        if step:
            self.engine.scheduler.now_override = now

    def step(self):
        """Announce and run one step on the leader; returns its token events."""
        self.announce(True)
        self.steps += 1
        return self.engine.step()

    def idle_tick(self) -> None:
        """Call while there is nothing to step: flushes queued commands and keeps the followers' deadline fed."""
        if self.pending or time.monotonic() - self.last_sent > KEEPALIVE_S:
            self.announce(False)

    def shutdown(self) -> None:
        if not self.ch.broken:
            try:
                self.announce(False, stop=True)
            except CommError:
                pass

    # ---------------------------------------------------------------- follower
    def apply(self, msg: dict) -> None:
        eng = self.engine
        for c in msg["cmds"]:
            if c["op"] == "add":
                # one clock for the whole group: deadlines and priority ties use the leader's arrival time
                eng.add_request(c["prompt"], params_from_wire(c["params"], self.guided_builder), request_id=c["rid"],
                                arrival=c["arrival"])
            elif c["op"] == "abort":
                eng.abort_request(c["rid"])

    def follow(self) -> str:
        """Worker loop of a rank without a front end. Returns why it ended: "stop" (the leader shut down) or
        "comm" (the control group broke; the caller should exit so that the data-plane group fails fast too)."""
        while True:
            try:
                msg = self.ch.bcast()
            except CommError:
                return "comm"
            self.apply(msg)
            if msg["stop"]:
                return "stop"
            if msg["step"]:
                self.engine.scheduler.now_override = msg["now"]
                self.engine.step()
                self.steps += 1
