"""Process-group plumbing: one process per GPU, ``torch.distributed`` for bootstrap and
for the library (baseline) collectives. The interface mirrors the reference's
``Communicator`` trait (rust/engine/src/comm/mod.rs:83-143): all_reduce, all_gather,
reduce_scatter, broadcast, all_to_all, send/recv, barrier, split. On CPU ranks the backend
is gloo and every sum is taken in rank order, so results are bit-identical on all ranks
(the property rust/engine/src/comm/mesh.rs:10-75 guarantees for its mesh collectives).
"""
from __future__ import annotations

import datetime
import os
from typing import List, Optional

import torch
import torch.distributed as dist


class CommError(RuntimeError):
    """Raised for any collective failure; the message is prefixed "[comm]" so callers can
    tell a broken group from a model error (rust/engine/src/parallel/ctx.rs:9)."""

    def __init__(self, msg: str):
        super().__init__("[comm] " + msg)


def init_distributed(backend: Optional[str] = None, timeout_s: float = 600.0) -> "tuple[int, int, int]":
    """Reads RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* from the environment (torchrun
    contract). Returns (rank, world, local_rank). A single process needs no group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, local


class Group:
    """A set of ranks with library collectives. ``size == 1`` groups are no-ops."""

    def __init__(self, ranks: Optional[List[int]] = None, pg=None):
        if not dist.is_initialized():
            self.size, self.rank, self.pg, self.ranks = 1, 0, None, [0]
            return
        world = dist.get_world_size()
        self.ranks = list(ranks) if ranks is not None else list(range(world))
        self.size = len(self.ranks)
        me = dist.get_rank()
        self.rank = self.ranks.index(me) if me in self.ranks else -1
        self.pg = pg if pg is not None else (dist.group.WORLD if self.ranks == list(range(world))
                                              else dist.new_group(self.ranks))
        self.deterministic = dist.get_backend(self.pg) == "gloo"

    # -------------------------------------------------------------- collectives
    def _wrap(self, fn, *a, **k):
        try:
            return fn(*a, **k)
        except RuntimeError as e:          # timeouts and aborted groups surface here
            raise CommError(str(e)) from e

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        if self.deterministic:
            # rank-ordered sum in fp32: identical bits on every rank
            parts = self.all_gather(x.contiguous())
            acc = parts[0].float()
            for i in range(1, self.size):
                acc = acc + parts[i].float()
            return acc.to(x.dtype)
        self._wrap(dist.all_reduce, x, group=self.pg)
        return x

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """Returns [size, *x.shape]."""
        if self.size == 1:
            return x.unsqueeze(0)
        flat = x.contiguous().view(-1)
        out = torch.empty(self.size * flat.numel(), dtype=x.dtype, device=x.device)
        self._wrap(dist.all_gather_into_tensor, out, flat, group=self.pg)
        return out.view((self.size,) + tuple(x.shape))

    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """x: [size * n, ...] -> this rank's reduced [n, ...] slice."""
        if self.size == 1:
            return x
        n = x.shape[0] // self.size
        if self.deterministic:
            full = self.all_reduce(x.clone())
            return full[self.rank * n:(self.rank + 1) * n].contiguous()
        out = torch.empty((n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        self._wrap(dist.reduce_scatter_tensor, out, x.contiguous(), group=self.pg)
        return out

    def broadcast(self, x: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.size > 1:
            self._wrap(dist.broadcast, x, src=self.ranks[src], group=self.pg)
        return x

    def all_to_all(self, send: List[torch.Tensor]) -> List[torch.Tensor]:
        """Variable-size exchange: counts first, then payloads."""
        if self.size == 1:
            return [send[0]]
        dev = send[0].device
        counts = torch.tensor([t.shape[0] for t in send], dtype=torch.int64, device=dev)
        rc = torch.empty_like(counts)
        self._wrap(dist.all_to_all_single, rc, counts, group=self.pg)
        tail = tuple(send[0].shape[1:])
        recv = [torch.empty((int(n),) + tail, dtype=send[0].dtype, device=dev) for n in rc.tolist()]
        if self.deterministic:
            # gloo has no list all-to-all: pairwise non-blocking sends and receives
            recv[self.rank].copy_(send[self.rank])
            ops = []
            for d in range(self.size):
                if d != self.rank:
                    ops.append(dist.P2POp(dist.isend, send[d].contiguous(), self.ranks[d], group=self.pg))
                    ops.append(dist.P2POp(dist.irecv, recv[d], self.ranks[d], group=self.pg))
            for w in self._wrap(dist.batch_isend_irecv, ops) if ops else []:
                self._wrap(w.wait)
            return recv
        self._wrap(dist.all_to_all, recv, [t.contiguous() for t in send], group=self.pg)
        return recv

    def send(self, x: torch.Tensor, dst: int) -> None:
        self._wrap(dist.send, x.contiguous(), dst=self.ranks[dst], group=self.pg)

    def recv(self, x: torch.Tensor, src: int) -> torch.Tensor:
        self._wrap(dist.recv, x, src=self.ranks[src], group=self.pg)
        return x

    def isend(self, x: torch.Tensor, dst: int):
        return dist.isend(x.contiguous(), dst=self.ranks[dst], group=self.pg)

    def irecv(self, x: torch.Tensor, src: int):
        return dist.irecv(x, src=self.ranks[src], group=self.pg)

    def barrier(self) -> None:
        if self.size > 1:
            self._wrap(dist.barrier, group=self.pg)

    def split(self, color: int, key: int) -> "Group":
        """Ranks with the same colour form a new group, ordered by key
        (rust/engine/src/comm/mod.rs ``split``)."""
        if self.size == 1:
            return self
        mine = torch.tensor([color, key, dist.get_rank()], dtype=torch.int64)
        dev = "cuda" if dist.get_backend(self.pg) == "nccl" else "cpu"
        allv = self.all_gather(mine.to(dev)).cpu().tolist()
        result = None
        for c in sorted({v[0] for v in allv}):
            members = [v[2] for v in sorted((v for v in allv if v[0] == c), key=lambda v: (v[1], v[2]))]
            g = dist.new_group(members)          # every rank must create every group
            if c == color:
                result = Group(members, g)
        return result

    def abort(self) -> None:
        if self.pg is not None and hasattr(self.pg, "abort"):
            try:
                self.pg.abort()
            except Exception:
                pass


def make_tp_pp_groups(tp: int, pp: int) -> "tuple[Group, Group, int, int]":
    """World = tp x pp, stage-major: rank = stage * tp + tp_rank
    (rust/engine/src/parallel/config.rs:93-100). Returns (tp_group, pp_group, stage, tp_rank)."""
    if not dist.is_initialized():
        return Group(), Group(), 0, 0
    world, rank = dist.get_world_size(), dist.get_rank()
    if world != tp * pp:
        raise ValueError(f"world size {world} != tp {tp} x pp {pp}")
    stage, tp_rank = divmod(rank, tp)
    tp_g = pp_g = None
    for s in range(pp):
        members = list(range(s * tp, (s + 1) * tp))
        g = dist.new_group(members) if pp > 1 else dist.group.WORLD
        if s == stage:
            tp_g = Group(members, g)
    for t in range(tp):
        members = [s * tp + t for s in range(pp)]
        g = dist.new_group(members) if tp > 1 else dist.group.WORLD
        if t == tp_rank:
            pp_g = Group(members, g)
    return tp_g, pp_g, stage, tp_rank


def shutdown_distributed(grace_s: float = 20.0) -> None:
    """Destroy the default process group, but never hang the process on it: if the library does
    not return within `grace_s` (e.g. a CUDA graph still references the communicator) the process
    exits with status 0, since all results have been reported by then."""
    import threading
    if not dist.is_initialized():
        return
    import sys
    sys.stdout.flush()
    sys.stderr.flush()
    t = threading.Timer(grace_s, lambda: os._exit(0))
    t.daemon = True
    t.start()
    try:
        dist.destroy_process_group()
    finally:
        t.cancel()
