"""Expert-parallel all-to-all over peer memory: dispatch of token rows to the ranks that hold their
routed experts, and return of the expert outputs to the token's owner (``csrc/moe_a2a.cu``).

Every rank allocates a receive buffer ``[cap][hidden]`` + tags, a combine buffer
``[max_tokens * k][hidden]`` and a small control block, exports them through CUDA IPC and maps its
peers' (same mechanism as ``comm.symm.FusedTP``). One MoE layer is then

    dispatch(x_owned, ids)  ->  ingest  ->  moe_align / gather / grouped GEMM x2 (local experts)
                            ->  return_rows  ->  wait_returns  ->  moe_combine (weighted sum)

with no library collective and no host synchronisation; all device-side waits are bounded.
``EpAllToAll.local_group`` builds the same structure for several virtual ranks on one device so
that the protocol can be tested on a single GPU by running the ranks' kernels phase by phase.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops._lib import load_cuda


class EpAllToAll:
    def __init__(self, ranks: int, rank: int, hidden: int, experts_per_rank: int, max_tokens: int, k: int,
                 device, tables: Optional[list] = None, group=None, cap: Optional[int] = None):
        self.k_ops = load_cuda()
        self.ranks, self.rank, self.hidden, self.k = ranks, rank, hidden, k
        self.experts_per_rank = experts_per_rank
        self.device = torch.device(device)
        self.max_entries = max_tokens * k
        # worst case every entry of every rank lands here; a smaller `cap` is reported through the status word
        self.cap = cap if cap is not None else self.max_entries * ranks
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        # the call number lives on the device (dispatch advances it), so a captured graph replays the layer as is
        self.call_ctr = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._owned: List[int] = []
        if tables is None:
            tables = self._exchange(group)
        self.ctx = self.k_ops.ep_ctx_create(ranks, rank, self.cap, hidden, experts_per_rank, *tables)
        dev = self.device.index or 0
        me = lambda kind, nbytes: self.k_ops.symm_view(tables[kind][rank], nbytes, dev)
        self.recv_x = me(0, self.cap * hidden * 2).view(torch.bfloat16).view(self.cap, hidden)
        self.comb_y = me(3, self.max_entries * hidden * 2).view(torch.bfloat16).view(self.max_entries, hidden)
        self.ids_recv = torch.empty(self.cap, dtype=torch.int32, device=self.device)
        self.count = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ setup
    def _sizes(self):
        return (self.cap * self.hidden * 2, self.cap * 16, 32 * 4, self.max_entries * self.hidden * 2)

    def _alloc(self) -> List[int]:
        with torch.cuda.device(self.device):
            ptrs = [self.k_ops.symm_alloc(int(n)) for n in self._sizes()]
        dev = self.device.index or 0
        self.k_ops.symm_view(ptrs[2], 32 * 4, dev).zero_()
        self._owned = ptrs
        return ptrs

    def _exchange(self, group):
        mine = self._alloc()
        handles = torch.stack([self.k_ops.symm_export(p) for p in mine])
        gathered = [None] * self.ranks
        dist.all_gather_object(gathered, handles.numpy().tobytes(), group=group.pg if group is not None else None)
        tables = [[0] * self.ranks for _ in range(4)]
        for r in range(self.ranks):
            blob = torch.frombuffer(bytearray(gathered[r]), dtype=torch.uint8).view(4, 64)
            for kind in range(4):
                if r == self.rank:
                    tables[kind][r] = mine[kind]
                else:
                    with torch.cuda.device(self.device):
                        tables[kind][r] = self.k_ops.symm_import(blob[kind].clone())
        torch.cuda.synchronize(self.device)
        if group is not None:
            group.barrier()
        return tables

    @classmethod
    def local_group(cls, ranks: int, hidden: int, experts_per_rank: int, max_tokens: int, k: int, device="cuda:0",
                    cap: Optional[int] = None) -> "List[EpAllToAll]":
        """`ranks` virtual ranks on one device sharing plain device pointers."""
        probe = cls.__new__(cls)
        probe.k_ops, probe.device, probe.hidden = load_cuda(), torch.device(device), hidden
        probe.max_entries = max_tokens * k
        probe.cap = cap if cap is not None else probe.max_entries * ranks
        ptrs = [probe._alloc() for _ in range(ranks)]
        tables = [[ptrs[r][kind] for r in range(ranks)] for kind in range(4)]
        torch.cuda.synchronize(probe.device)
        out = [cls(ranks, r, hidden, experts_per_rank, max_tokens, k, device, tables=tables, cap=cap) for r in range(ranks)]
        for r, o in enumerate(out):
            o._owned = ptrs[r]
        return out

    # ------------------------------------------------------------------ steps (all asynchronous on the current stream)
    def dispatch(self, x: torch.Tensor, ids: torch.Tensor) -> None:
        """x: [tokens, hidden] rows this rank owns; ids: [tokens, k] global expert ids (int32)."""
        self.k_ops.ep_dispatch(self.ctx, x, ids, 0, self.status, self.call_ctr)

    def ingest(self) -> "tuple[torch.Tensor, torch.Tensor]":
        """-> (expert id per received row [cap] (-1 = unused), row count [1]); rows are in ``recv_x``."""
        self.k_ops.ep_ingest(self.ctx, 0, self.ids_recv, self.count, self.status, self.call_ctr)
        return self.ids_recv, self.count

    def return_rows(self, y: torch.Tensor, row_of: torch.Tensor) -> None:
        """y: expert outputs in permuted order; row_of: [cap] permuted row of every received row."""
        self.k_ops.ep_return(self.ctx, y, row_of, self.count, 0, self.call_ctr)

    def wait_returns(self) -> torch.Tensor:
        """After this, ``comb_y[token * k + slot]`` holds the output of that (token, slot)."""
        self.k_ops.ep_wait_returns(self.ctx, 0, self.status, self.call_ctr)
        return self.comb_y

    def check_status(self) -> int:
        code = int(self.status.item())
        if code:
            self.status.zero_()
        return code


def moe_ffn_a2a_phases(dec, lw, ep: EpAllToAll, h_owned: torch.Tensor):
    """The MoE layer of one rank in all-to-all mode as a generator of phases (route+dispatch |
    expert compute+return | combine), so that a single-GPU test can interleave virtual ranks. The
    final value is the layer output for the owned rows."""
    from ..models.moe import _grouped, _token_tile
    cfg, ops = dec.cfg, dec.ops
    kk = ops.k
    T, H = h_owned.shape
    k = cfg.experts_per_token
    e_local = lw.exp_gate_up.shape[0]
    lo = ep.rank * ep.experts_per_rank
    i32 = dict(dtype=torch.int32, device=h_owned.device)
    logits = ops.linear(h_owned, lw.router_w, lw.router_b)
    ids = torch.empty(T, k, **i32)
    wts = torch.empty(T, k, dtype=torch.float32, device=h_owned.device)
    kk.moe_route(logits, None, k, cfg.router_kind != "softmax_topk", ids, wts)
    ep.dispatch(h_owned, ids)
    yield "dispatched"
    ids_recv, count = ep.ingest()
    bn = _token_tile(ep.cap / max(e_local, 1) / 4)
    rows_cap = -(-(ep.cap + e_local * (bn - 1)) // bn) * bn
    max_tiles = rows_cap // bn
    row_of = torch.empty(ep.cap, **i32)
    token_of = torch.empty(rows_cap, **i32)
    tile_e, tile_r = torch.empty(max_tiles, **i32), torch.empty(max_tiles, **i32)
    ntiles = torch.zeros(2, **i32)
    kk.moe_align(ids_recv.view(ep.cap, 1), cfg.num_experts, lo, lo + e_local, bn, row_of, token_of, tile_e, tile_r, ntiles)
    xp = torch.empty(rows_cap, H, dtype=h_owned.dtype, device=h_owned.device)
    kk.moe_gather(ep.recv_x, token_of, xp)
    gu = torch.empty(rows_cap, lw.exp_gate_up.shape[1], dtype=h_owned.dtype, device=h_owned.device)
    _grouped(kk, ops, xp, lw.exp_gate_up, lw.exp_gate_up_b, gu, tile_e, tile_r, ntiles, bn)
    act = ops.glu(gu, dec.act_kind, cfg.swiglu_alpha, cfg.swiglu_limit)
    y = torch.empty(rows_cap, H, dtype=h_owned.dtype, device=h_owned.device)
    _grouped(kk, ops, act, lw.exp_down, lw.exp_down_b, y, tile_e, tile_r, ntiles, bn)
    ep.return_rows(y, row_of)
    yield "returned"
    comb = ep.wait_returns()
    out = torch.empty(T, H, dtype=h_owned.dtype, device=h_owned.device)
    ident = torch.arange(T * k, **i32).view(T, k)
    kk.moe_combine(comb, ident, wts, out)
    ops.launches += 12
    yield out
