"""Response cache and request coalescer for non-streaming, deterministic requests.

A request is deterministic when it is greedy or carries an explicit seed. Its key is a digest of
the model name, the prompt token ids and every sampling field that changes the output (plus the
caller's ``cache_salt``, so tenants can keep their entries apart). A finished response is kept in
an LRU with a time-to-live; identical requests that arrive while the first is still generating
wait for it instead of generating again (rust/engine/src/server/response_cache.rs is the
reference's counterpart).
"""
from __future__ import annotations

import asyncio
import hashlib
import json
import time
from collections import OrderedDict
from typing import Awaitable, Callable, Optional, Sequence


def request_key(model: str, prompt_ids: Sequence[int], sp) -> Optional[str]:
    """None when the request is not cacheable (sampled without a seed, or constrained by an object
    whose state we cannot digest)."""
    if not (sp.greedy or sp.seed is not None):
        return None
    fields = {
        "m": model, "t": sp.temperature, "p": sp.top_p, "k": sp.top_k, "mp": sp.min_p, "rp": sp.repetition_penalty,
        "pp": sp.presence_penalty, "fp": sp.frequency_penalty, "seed": sp.seed, "max": sp.max_tokens,
        "min": sp.min_tokens, "eos": sp.ignore_eos, "stop": list(sp.stop), "stop_ids": list(sp.stop_token_ids),
        "bias": sorted((sp.logit_bias or {}).items()), "allow": sorted(sp.allowed_token_ids or []),
        "bad": sorted(sp.bad_words_ids or []), "lp": sp.logprobs, "salt": sp.cache_salt,
        "badseq": [list(w) for w in (sp.bad_words or [])], "typ": sp.typical_p,
        "dry": [sp.dry_multiplier, sp.dry_base, sp.dry_allowed_length, list(sp.dry_sequence_breakers), sp.dry_penalty_last_n],
        "miro": [sp.mirostat_mode, sp.mirostat_tau, sp.mirostat_eta],
        "guided": type(sp.guided).__name__ if sp.guided is not None else None,
    }
    h = hashlib.sha256(json.dumps(fields, sort_keys=True, default=str).encode())
    h.update(b"|")
    h.update(b",".join(str(int(t)).encode() for t in prompt_ids))
    return h.hexdigest()


class ResponseCache:
    def __init__(self, max_entries: int = 1024, ttl_s: float = 600.0, clock: Callable[[], float] = time.monotonic):
        self.max_entries, self.ttl_s, self.clock = max_entries, ttl_s, clock
        self.entries: "OrderedDict[str, tuple]" = OrderedDict()
        self.inflight: dict = {}
        self.hits = self.misses = self.coalesced = 0

    def get(self, key: Optional[str]):
        if key is None or self.max_entries <= 0:
            return None
        e = self.entries.get(key)
        if e is None:
            return None
        if self.clock() - e[0] > self.ttl_s:
            del self.entries[key]
            return None
        self.entries.move_to_end(key)
        return e[1]

    def put(self, key: Optional[str], value) -> None:
        if key is None or self.max_entries <= 0:
            return
        self.entries[key] = (self.clock(), value)
        self.entries.move_to_end(key)
        while len(self.entries) > self.max_entries:
            self.entries.popitem(last=False)

    def clear(self) -> int:
        n = len(self.entries)
        self.entries.clear()
        return n

    async def get_or_compute(self, key: Optional[str], compute: Callable[[], Awaitable]):
        """Cached value, or the value of an identical request already in flight, or compute()."""
        hit = self.get(key)
        if hit is not None:
            self.hits += 1
            return hit
        if key is None:
            return await compute()
        fut = self.inflight.get(key)
        if fut is not None:
            self.coalesced += 1
            return await asyncio.shield(fut)
        self.misses += 1
        fut = asyncio.get_running_loop().create_future()
        self.inflight[key] = fut
        try:
            value = await compute()
        except BaseException as e:
            if not fut.done():
                fut.set_exception(e)
                fut.exception()                     # mark as retrieved: waiters re-raise it themselves
            raise
        else:
            self.put(key, value)
            if not fut.done():
                fut.set_result(value)
            return value
        finally:
            self.inflight.pop(key, None)

    def stats(self) -> dict:
        return {"entries": len(self.entries), "hits": self.hits, "misses": self.misses, "coalesced": self.coalesced,
                "inflight": len(self.inflight)}
