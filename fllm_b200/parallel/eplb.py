"""Expert-load balancing plan: per-expert hit counters and a placement that replicates the
hottest experts and packs experts onto ranks so that expected load is even
(rust/engine/src/parallel/eplb.rs:11-44 counters, :90-133 planner). Planning half only, like
the reference: the engine consumes a placement at load time."""
from __future__ import annotations

import heapq
from typing import List, Sequence


class ExpertStats:
    def __init__(self, num_layers: int, num_experts: int):
        self.hits = [[0] * num_experts for _ in range(num_layers)]

    def record(self, layer: int, expert_ids: Sequence[int]) -> None:
        row = self.hits[layer]
        for e in expert_ids:
            row[e] += 1

    def load(self, layer: int) -> List[float]:
        tot = sum(self.hits[layer]) or 1
        return [h / tot for h in self.hits[layer]]


def plan_placement(load: Sequence[float], ranks: int, slots_per_rank: int) -> dict:
    """Greedy: give every expert one replica, hand the spare slots to the experts with the
    highest load per replica, then place replicas heaviest-first on the least loaded rank."""
    E = len(load)
    total_slots = ranks * slots_per_rank
    if total_slots < E:
        raise ValueError("not enough slots for one replica per expert")
    replicas = [1] * E
    heap = [(-load[e], e) for e in range(E)]
    heapq.heapify(heap)
    for _ in range(total_slots - E):
        _, e = heapq.heappop(heap)
        replicas[e] += 1
        heapq.heappush(heap, (-load[e] / replicas[e], e))
    items = sorted(((load[e] / replicas[e], e) for e in range(E) for _ in range(replicas[e])), reverse=True)
    rank_load = [0.0] * ranks
    rank_experts: List[List[int]] = [[] for _ in range(ranks)]
    for w, e in items:
        cands = [r for r in range(ranks) if len(rank_experts[r]) < slots_per_rank and e not in rank_experts[r]]
        if not cands:
            cands = [r for r in range(ranks) if len(rank_experts[r]) < slots_per_rank]
        r = min(cands, key=lambda i: rank_load[i])
        rank_experts[r].append(e)
        rank_load[r] += w
    mean = sum(rank_load) / ranks
    return {"replicas": replicas, "rank_experts": rank_experts, "rank_load": rank_load,
            "imbalance": (max(rank_load) / mean) if mean > 0 else 1.0}
