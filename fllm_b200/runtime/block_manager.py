"""Paged-KV bookkeeping: a ref-counted block allocator with an integrated prefix
cache, and per-sequence block tables.

Behaviour follows the reference's ``BlockManager`` (rust/engine/src/mem/block_allocator.rs:
146-316: ref counts, copy-on-write of a shared tail, sliding-window pruning) and
``PrefixCache`` (rust/engine/src/mem/prefix_cache.rs:96-640: chain hashes of full blocks,
LRU of unreferenced blocks, pinning, per-tenant salts), merged into one structure so that
a cached block and a free block are the same pool: a block whose ref count drops to zero
keeps its contents and its hash until the allocator needs it.
"""
from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np


def chain_hash(parent: bytes, tokens: Sequence[int], salt: bytes = b"") -> bytes:
    h = hashlib.blake2b(digest_size=16)
    h.update(parent)
    h.update(salt)
    h.update(b"".join(int(t).to_bytes(4, "little", signed=False) for t in tokens))
    return h.digest()


@dataclass
class SeqBlocks:
    table: List[int] = field(default_factory=list)      # logical block -> physical block
    num_tokens: int = 0                                  # tokens whose KV is (or will be) stored
    hashes: List[bytes] = field(default_factory=list)    # chain hash of each full, registered block
    first_live_block: int = 0                            # blocks before this were pruned (window)
    state_slot: int = -1                                 # row of the recurrent-state pools (hybrid models)
    _np: Optional["np.ndarray"] = None                   # int32 mirror of `table` for batch building
    _np_len: int = 0
    _np_dirty: bool = True

    def np_table(self) -> "np.ndarray":
        """int32 view of the table; appends are mirrored incrementally, other edits rebuild it."""
        n = len(self.table)
        if self._np is None or self._np.shape[0] < n:
            cap = max(64, 2 * n)
            self._np = np.empty(cap, dtype=np.int32)
            self._np_dirty = True
        if self._np_dirty or self._np_len > n:
            self._np[:n] = self.table
            self._np_dirty = False
        elif self._np_len < n:
            self._np[self._np_len:n] = self.table[self._np_len:n]
        self._np_len = n
        return self._np[:n]


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int = 16, enable_prefix_caching: bool = True,
                 watermark: float = 0.01):
        self.num_blocks, self.block_size = num_blocks, block_size
        self.enable_prefix_caching = enable_prefix_caching
        self.refs = [0] * num_blocks
        self.state_free: Optional[List[int]] = None          # rows of the recurrent-state pools (hybrid models only)
        # recurrent-state checkpoints: a cached prefix is usable only up to a block whose hash has a state copy;
        # state_restore(hash, row) writes that copy into the new sequence's row
        self.state_has = None
        self.state_restore = None
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))   # never-used / invalidated blocks
        self.cached: "OrderedDict[int, bytes]" = OrderedDict()       # ref==0 blocks with valid content (LRU)
        self.hash_to_block: Dict[bytes, int] = {}
        self.block_hash: Dict[int, bytes] = {}
        self.pinned: set = set()
        self.seqs: Dict[int, SeqBlocks] = {}
        self.watermark_blocks = int(watermark * num_blocks)
        self.stats = {"prefix_queries": 0, "prefix_hits": 0, "evictions": 0, "cow": 0, "tier_restored": 0}
        # optional lower tier for evicted prefix blocks (runtime.kv_tier): on_evict(block, hash) is called while
        # the block still holds its KV; tier_has(hash) / tier_restore(hash, block) bring a block back
        self.on_evict = None
        self.tier_has = None
        self.tier_restore = None

    # ------------------------------------------------------------------ pool
    def num_free(self) -> int:
        if not self.pinned:
            return len(self.free) + len(self.cached)
        return len(self.free) + len(self.cached) - sum(1 for b in self.pinned if b in self.cached)

    def num_used(self) -> int:
        return self.num_blocks - len(self.free) - len(self.cached)

    def _take(self) -> int:
        if self.free:
            b = self.free.pop()
        else:
            b = None
            for cand in self.cached:                      # oldest first
                if cand not in self.pinned:
                    b = cand
                    break
            if b is None:
                raise MemoryError("out of KV blocks")
            h = self.cached.pop(b)
            if self.on_evict is not None:
                self.on_evict(b, h)
            self.hash_to_block.pop(h, None)
            self.block_hash.pop(b, None)
            self.stats["evictions"] += 1
        self.refs[b] = 1
        return b

    def _release(self, b: int) -> None:
        self.refs[b] -= 1
        assert self.refs[b] >= 0, "double free of a KV block"
        if self.refs[b] == 0:
            h = self.block_hash.get(b)
            if h is not None and self.enable_prefix_caching:
                self.cached[b] = h
                self.cached.move_to_end(b)
            else:
                self.block_hash.pop(b, None)
                self.free.append(b)

    def blocks_needed(self, num_tokens: int) -> int:
        return -(-num_tokens // self.block_size)

    def can_allocate(self, num_new_blocks: int, respect_watermark: bool = True) -> bool:
        reserve = self.watermark_blocks if respect_watermark else 0
        return self.num_free() - num_new_blocks >= reserve

    # ------------------------------------------------------------------ sequences
    def match_prefix(self, tokens: Sequence[int], salt: bytes = b"") -> Tuple[List[int], List[bytes]]:
        """Longest run of cached full blocks that prefixes `tokens` (never the whole prompt: the
        last token must be computed to produce logits)."""
        self.stats["prefix_queries"] += 1
        if not self.enable_prefix_caching:
            return [], []
        bs = self.block_size
        blocks, hashes = [], []
        parent = b""
        usable = (len(tokens) - 1) // bs
        for i in range(usable):
            h = chain_hash(parent, tokens[i * bs:(i + 1) * bs], salt)
            b = self.hash_to_block.get(h)
            if b is None:
                break
            blocks.append(b)
            hashes.append(h)
            parent = h
        if self.state_has is not None:
            while hashes and not self.state_has(hashes[-1]):
                blocks.pop()
                hashes.pop()
        if blocks:
            self.stats["prefix_hits"] += 1
        return blocks, hashes

    def allocate(self, seq_id: int, tokens: Sequence[int], salt: bytes = b"") -> int:
        """Creates the table of a new sequence, reusing cached prefix blocks. Returns the number
        of prompt tokens whose KV is already present."""
        assert seq_id not in self.seqs
        blocks, hashes = self.match_prefix(tokens, salt)
        for b in blocks:
            if self.refs[b] == 0:
                self.cached.pop(b, None)
            self.refs[b] += 1
        if self.tier_has is not None and self.enable_prefix_caching and self.state_has is None:
            # the prompt may continue with blocks that were evicted to the lower tier: bring them back while the
            # chain holds and the pool has room beyond its watermark
            bs = self.block_size
            parent = hashes[-1] if hashes else b""
            for i in range(len(blocks), (len(tokens) - 1) // bs):
                h = chain_hash(parent, tokens[i * bs:(i + 1) * bs], salt)
                if h in self.hash_to_block or not self.tier_has(h) or not self.can_allocate(1):
                    break
                b = self._take()
                if not self.tier_restore(h, b):
                    self.refs[b] = 0
                    self.free.append(b)
                    break
                self.hash_to_block[h] = b
                self.block_hash[b] = h
                blocks.append(b)
                hashes.append(h)
                parent = h
                self.stats["tier_restored"] += 1
        sb = SeqBlocks(table=list(blocks), num_tokens=len(blocks) * self.block_size, hashes=list(hashes))
        if self.state_free is not None:
            if not self.state_free:
                raise RuntimeError("no free recurrent-state row: more live sequences than max_num_seqs allows")
            sb.state_slot = self.state_free.pop()
            if hashes and self.state_restore is not None and not self.state_restore(hashes[-1], sb.state_slot):
                # the copy went away between the match and now: compute the prompt from its first token
                for b in blocks:
                    self._release(b)
                sb.table, sb.hashes, sb.num_tokens = [], [], 0
        self.seqs[seq_id] = sb
        return sb.num_tokens

    def ensure_capacity(self, seq_id: int, total_tokens: int) -> bool:
        """Grow the table so that `total_tokens` KV slots exist. False if the pool is exhausted
        (nothing is changed in that case)."""
        sb = self.seqs[seq_id]
        need = self.blocks_needed(total_tokens) - len(sb.table)
        if need <= 0:
            return True
        if self.num_free() < need:
            return False
        for _ in range(need):
            sb.table.append(self._take())
        return True

    def slots_for(self, seq_id: int, start: int, count: int) -> List[int]:
        sb = self.seqs[seq_id]
        bs = self.block_size
        return [sb.table[p // bs] * bs + p % bs for p in range(start, start + count)]

    def commit_tokens(self, seq_id: int, all_tokens: Sequence[int], new_total: int, salt: bytes = b"") -> None:
        """Record that KV for tokens [0, new_total) is now stored; register newly full blocks."""
        sb = self.seqs[seq_id]
        sb.num_tokens = new_total
        if not self.enable_prefix_caching:
            return
        bs = self.block_size
        full = new_total // bs
        while len(sb.hashes) < full:
            i = len(sb.hashes)
            parent = sb.hashes[-1] if sb.hashes else b""
            h = chain_hash(parent, all_tokens[i * bs:(i + 1) * bs], salt)
            sb.hashes.append(h)
            b = sb.table[i]
            if b < 0:
                continue
            if h not in self.hash_to_block and b not in self.block_hash:
                self.hash_to_block[h] = b
                self.block_hash[b] = h

    def cow_last_block(self, seq_id: int) -> Optional[Tuple[int, int]]:
        """If the block about to be appended to is shared, give the sequence a private copy.
        Returns (src, dst) for the device copy, or None."""
        sb = self.seqs[seq_id]
        if not sb.table:
            return None
        idx = sb.num_tokens // self.block_size
        if idx >= len(sb.table) or sb.num_tokens % self.block_size == 0:
            return None
        b = sb.table[idx]
        if self.refs[b] <= 1:
            return None
        nb = self._take()
        self._release(b)
        sb.table[idx] = nb
        sb._np_dirty = True
        self.stats["cow"] += 1
        return b, nb

    def fork(self, parent_id: int, child_id: int) -> None:
        if self.state_free is not None:
            raise NotImplementedError("sequences of a recurrent model cannot be forked: their state is not paged")
        p = self.seqs[parent_id]
        for b in p.table:
            if b >= 0:
                self.refs[b] += 1
        self.seqs[child_id] = SeqBlocks(list(p.table), p.num_tokens, list(p.hashes), p.first_live_block)

    def prune_window(self, seq_id: int, window: int) -> int:
        """Free blocks that lie entirely before the sliding window. Pruned entries stay in the
        table as -1 so logical indices keep their meaning."""
        sb = self.seqs[seq_id]
        if window <= 0:
            return 0
        first_needed = max(0, sb.num_tokens - window) // self.block_size
        freed = 0
        for i in range(sb.first_live_block, min(first_needed, len(sb.table))):
            if sb.table[i] >= 0:
                self._release(sb.table[i])
                sb.table[i] = -1
                sb._np_dirty = True
                freed += 1
        sb.first_live_block = max(sb.first_live_block, first_needed)
        return freed

    def truncate(self, seq_id: int, new_total: int) -> None:
        """Roll back KV past `new_total` tokens (rejected speculative tokens)."""
        sb = self.seqs[seq_id]
        keep = self.blocks_needed(new_total)
        while len(sb.table) > keep:
            b = sb.table.pop()
            if b >= 0:
                self._release(b)
        sb.num_tokens = min(sb.num_tokens, new_total)
        del sb.hashes[new_total // self.block_size:]

    def free_seq(self, seq_id: int) -> None:
        sb = self.seqs.pop(seq_id, None)
        if sb is None:
            return
        if sb.state_slot >= 0:
            self.state_free.append(sb.state_slot)
        for b in reversed(sb.table):       # tail blocks become eviction candidates first
            if b >= 0:
                self._release(b)

    def table(self, seq_id: int) -> List[int]:
        return self.seqs[seq_id].table

    def enable_state_slots(self, n: int) -> None:
        """Give every sequence one of ``n`` rows of the recurrent-state pools for as long as it holds blocks."""
        self.state_free = list(range(n - 1, -1, -1))

    def state_slot(self, seq_id: int) -> int:
        return self.seqs[seq_id].state_slot

    def np_table(self, seq_id: int) -> np.ndarray:
        return self.seqs[seq_id].np_table()

    # ------------------------------------------------------------------ admin
    def pin_prefix(self, tokens: Sequence[int], salt: bytes = b"") -> int:
        blocks, _ = self.match_prefix(list(tokens) + [0], salt)
        self.pinned.update(blocks)
        return len(blocks)

    def unpin_all(self) -> None:
        self.pinned.clear()

    def reset_prefix_cache(self) -> int:
        n = 0
        for b in list(self.cached):
            if b in self.pinned:
                continue
            h = self.cached.pop(b)
            self.hash_to_block.pop(h, None)
            self.block_hash.pop(b, None)
            self.free.append(b)
            n += 1
        return n
