"""Peer-memory ("symmetric") buffers and the fused tensor-parallel runtime built on them.

Every rank allocates the same set of device buffers, exports them through CUDA IPC and maps
every peer's copy, so that our own kernels can store into a peer's HBM over NVLink:

* ``rs``    receive buffer ``[tp][rows_per][hidden]``: partial sums that peers' row-parallel
            GEMM epilogues push for the token rows this rank owns;
* ``ag``    gathered activations ``[max_tokens][hidden]``: normalised rows that every rank
            pushes after it reduced its rows; the next GEMM reads it as a local operand;
* ``ar``    slots of the one-shot all-reduce used for small odd messages;
* ``flags`` arrival counters (monotonic, never reset, so CUDA-graph replays need no host
            bookkeeping) plus local "consumed" counters.

The layer-half pipeline is  GEMM->RS (peer stores in the epilogue)  ->  reduce + residual +
RMSNorm + all-gather push (one small kernel)  ->  all-gather->GEMM (TMA producer waits on the
counters). No library collective runs on that path; every device-side wait is bounded and
reports through the status word. ``FusedTP.local_group`` builds the same structure for several
virtual ranks on ONE device (plain pointers, no IPC) so the arithmetic and the counter protocol
can be tested on a single GPU by launching the ranks' kernels phase by phase.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops._lib import load_cuda
from .group import Group


class FusedTP:
    backend = "fused"

    def __init__(self, group: Optional[Group], device, hidden: int = 0, max_tokens: int = 2048,
                 ar_slot_bytes: int = 1 << 20, _local: Optional[dict] = None):
        self.k = load_cuda()
        self.device = torch.device(device)
        self.group = group
        self.hidden, self.max_tokens, self.ar_slot_bytes = hidden, max_tokens, ar_slot_bytes
        self.workspace = None
        self._rs_expected = 0
        self._owned: List[int] = []
        self._imported: List[int] = []
        self.ctx = -1
        if _local is not None:                       # virtual rank of a single-device group
            self.size, self.rank = _local["tp"], _local["rank"]
            self.status = _local["status"]
            self._make_ctx(_local["rs"], _local["ag"], _local["flags"], _local["ar"])
            return
        self.size, self.rank = group.size, group.rank
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        if hidden:
            self.setup(hidden, max_tokens)

    # ------------------------------------------------------------------ setup
    BCAST_ROWS = 128        # steps with at most this many tokens use the one-shot (broadcast) layout

    def _sizes(self):
        rows_per_max = max(-(-self.max_tokens // self.size), self.BCAST_ROWS)
        return (self.size * rows_per_max * self.hidden * 2, self.max_tokens * self.hidden * 2,
                self.k.flag_words() * 4, self.size * self.ar_slot_bytes)

    def setup(self, hidden: int, max_tokens: int) -> None:
        """Allocate, exchange IPC handles over the process group, map peers."""
        self.hidden, self.max_tokens = hidden, max_tokens
        with torch.cuda.device(self.device):
            mine = [self.k.symm_alloc(int(n)) for n in self._sizes()]
        self._owned = mine
        handles = torch.stack([self.k.symm_export(p) for p in mine])          # [4, 64] uint8 (CPU)
        gathered = [None] * self.size
        dist.all_gather_object(gathered, handles.numpy().tobytes(), group=self.group.pg)
        tables = [[0] * self.size for _ in range(4)]
        for r in range(self.size):
            blob = torch.frombuffer(bytearray(gathered[r]), dtype=torch.uint8).view(4, 64)
            for kind in range(4):
                if r == self.rank:
                    tables[kind][r] = mine[kind]
                else:
                    with torch.cuda.device(self.device):
                        p = self.k.symm_import(blob[kind].clone())
                    self._imported.append(p)
                    tables[kind][r] = p
        self._make_ctx(*tables)
        self.group.barrier()

    def _make_ctx(self, rs, ag, flags, ar) -> None:
        self._tables = (list(rs), list(ag), list(flags), list(ar))
        self.ctx = self.k.tp_ctx_create(self.size, self.rank, self.hidden, self.max_tokens, self.BCAST_ROWS,
                                        self.device.index or 0, list(rs), list(ag), list(flags), list(ar),
                                        self.ar_slot_bytes, self.status)
        self.ag_local = self.k.symm_view(ag[self.rank], self.max_tokens * self.hidden * 2,
                                         self.device.index or 0).view(torch.bfloat16).view(self.max_tokens, self.hidden)
        self.workspace = torch.zeros(64 << 20, dtype=torch.uint8, device=self.device)

    @classmethod
    def local_group(cls, tp: int, hidden: int, max_tokens: int, device="cuda:0", ar_slot_bytes: int = 1 << 20):
        """tp virtual ranks on one device sharing plain device pointers (tests / emulation)."""
        k = load_cuda()
        device = torch.device(device)
        probe = cls.__new__(cls)
        probe.k, probe.size, probe.hidden, probe.max_tokens, probe.ar_slot_bytes = k, tp, hidden, max_tokens, ar_slot_bytes
        sizes = probe._sizes()
        with torch.cuda.device(device):
            ptrs = [[k.symm_alloc(int(n)) for n in sizes] for _ in range(tp)]
        tables = [[ptrs[r][kind] for r in range(tp)] for kind in range(4)]
        ranks = []
        for r in range(tp):
            st = torch.zeros(1, dtype=torch.int32, device=device)
            t = cls(None, device, hidden, max_tokens, ar_slot_bytes,
                    _local={"tp": tp, "rank": r, "status": st, "rs": tables[0], "ag": tables[1],
                            "flags": tables[2], "ar": tables[3]})
            t._owned = ptrs[r]
            ranks.append(t)
        return ranks

    # ------------------------------------------------------------------ geometry
    def rows_per(self, tokens: int) -> int:
        return -(-tokens // self.size)

    def my_rows(self, tokens: int) -> "tuple[int, int]":
        rp = self.rows_per(tokens)
        lo = min(tokens, self.rank * rp)
        return lo, min(tokens, lo + rp)

    # ------------------------------------------------------------------ fused steps
    def use_bcast(self, tokens: int) -> bool:
        """Small steps (decode) are latency-bound: every rank pushes its partial sums to every
        rank and reduces all rows itself - one cross-GPU dependency per projection instead of
        two. Large steps (prefill) are bandwidth-bound: reduce-scatter + all-gather."""
        return tokens <= self.BCAST_ROWS

    def linear_rs(self, x: torch.Tensor, w: torch.Tensor, bias=None, bcast: bool = False) -> int:
        """Returns (and remembers) how many arrival-counter bumps each destination receives from
        a source for this projection: the following ``norm`` waits for exactly that many. Every
        rank runs the same shapes, so the local value equals the peers'."""
        self._rs_expected = int(self.k.tp_linear_rs(self.ctx, x, w, bias, self.workspace, bcast))
        return self._rs_expected

    def norm(self, residual: torch.Tensor, tokens: int, has_partials: bool, norm_w, eps, w_offset=0.0,
             bcast: bool = False) -> None:
        """bcast=False: `residual` holds this rank's rows; normalised rows go to every rank's
        gathered buffer. bcast=True: `residual` holds all rows; the output stays in the local
        gathered buffer (``ag_local[:tokens]``)."""
        expected = self._rs_expected if has_partials else 0
        self.k.tp_norm(self.ctx, residual, tokens, expected, norm_w, float(eps), float(w_offset), bcast)

    def linear_ag(self, tokens: int, w: torch.Tensor, bias=None, out=None) -> torch.Tensor:
        if out is None:
            out = torch.empty(tokens, w.shape[0], dtype=torch.bfloat16, device=self.device)
        self.launches_last = self.k.tp_linear_ag(self.ctx, tokens, w, bias, out, self.workspace)
        return out

    # ------------------------------------------------------------------ generic collectives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        """Small messages go through the one-shot peer kernel; large ones through the library."""
        nbytes = x.numel() * x.element_size()
        if x.is_contiguous() and nbytes % 16 == 0 and nbytes <= self.ar_slot_bytes and x.dtype in (torch.bfloat16, torch.float32):
            out = torch.empty_like(x)
            self.k.tp_allreduce(self.ctx, x, out)
            return out
        return self.group.all_reduce(x)

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """Small messages (the (value, id) pairs of a vocabulary-parallel argmax) go through the
        one-shot peer kernel; anything else through the library."""
        nbytes = x.numel() * x.element_size()
        if x.is_contiguous() and nbytes and nbytes % 16 == 0 and nbytes <= self.ar_slot_bytes:
            out = torch.empty((self.size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
            self.k.tp_allgather(self.ctx, x, out)
            return out
        return self.group.all_gather(x)

    def check_status(self) -> int:
        code = int(self.status.item())
        if code:
            self.status.zero_()
        return code

    # ------------------------------------------------------------------ validation / teardown
    def self_check(self) -> bool:
        """Run the fused chain once on random data and compare with library collectives."""
        T, H, K = 24, self.hidden, 256
        g = torch.Generator(device=self.device).manual_seed(1234 + self.rank)
        x = (torch.randn(T, K, generator=g, device=self.device) * 0.5).to(torch.bfloat16)
        w = (torch.randn(H, K, generator=g, device=self.device) * 0.05).to(torch.bfloat16)
        ones = torch.ones(H, dtype=torch.bfloat16, device=self.device)
        lo, hi = self.my_rows(T)
        shard = torch.zeros(max(hi - lo, 1), H, dtype=torch.bfloat16, device=self.device)
        self.linear_rs(x, w)
        self.norm(shard, T, True, ones, 1e-6)
        eye = torch.eye(H, dtype=torch.bfloat16, device=self.device)
        got = self.linear_ag(T, eye)                       # identity weight: returns the gathered rows
        torch.cuda.synchronize(self.device)
        part = (x.float() @ w.float().t())
        full = self.group.all_reduce(part.clone())
        full = full.to(torch.bfloat16).float()
        want = full * torch.rsqrt(full.pow(2).mean(-1, keepdim=True) + 1e-6)
        err = (got.float() - want).abs().max().item()
        ok = torch.tensor([1 if (err < 0.05 and self.check_status() == 0) else 0], device=self.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group.pg)
        return bool(ok.item())

    def close(self, release: bool = False) -> None:
        """Quiesce. Peer mappings and buffers are left to process exit unless `release` is set:
        un-mapping while a peer still tears down its own side gained nothing and cost a hang."""
        try:
            torch.cuda.synchronize(self.device)
        except Exception:
            pass
        if not release:
            return
        for p in self._imported:
            self.k.symm_close(p)
        self._imported = []
        for p in self._owned:
            self.k.symm_free(p)
        self._owned = []
