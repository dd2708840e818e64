"""Host-side parallel logic: layouts, sharding rules, the cluster planner and expert placement."""
import pytest
import torch

from fllm_b200.config import ParallelConfig, preset
from fllm_b200.models.weights import attention_split, expert_range, init_random_weights, make_shard_spec
from fllm_b200.parallel.eplb import ExpertStats, plan_placement
from fllm_b200.parallel.planner import GPU_PRESETS, plan_cluster, runnable


def test_rank_numbering_and_stage_layers():
    p = ParallelConfig(tp=4, pp=2)
    assert p.world == 8 and p.coords(5) == (1, 1)
    assert list(p.stage_layers(36, 0)) == list(range(18)) and list(p.stage_layers(36, 1)) == list(range(18, 36))
    q = ParallelConfig(tp=1, pp=3)
    assert [len(q.stage_layers(10, s)) for s in range(3)] == [4, 3, 3]


def test_attention_split_rules():
    cfg = preset("qwen3-8b")
    assert attention_split(cfg, 8, 3) == (4, 1, 12, 3)
    assert attention_split(cfg, 2, 1) == (16, 4, 16, 4)
    tiny = preset("qwen3-tiny")                       # 8 q heads, 2 kv heads: tp 4 replicates kv
    assert attention_split(tiny, 4, 3) == (2, 1, 6, 1)
    with pytest.raises(ValueError):
        attention_split(tiny, 3, 0)
    assert [expert_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 3), (6, 2), (8, 2)]


def test_shards_reassemble_to_the_full_model():
    cfg = preset("qwen3-tiny")
    full = init_random_weights(cfg, "cpu", seed=7)
    tp = 2
    parts = [init_random_weights(cfg, "cpu", seed=7, tp=tp, tp_rank=r) for r in range(tp)]
    D = cfg.head_dim
    l0 = full.layers[0]
    q_full = l0.wqkv[: cfg.q_size]
    q_cat = torch.cat([p.layers[0].wqkv[: cfg.q_size // tp] for p in parts], 0)
    assert torch.equal(q_cat, q_full)
    assert torch.equal(torch.cat([p.layers[0].wo for p in parts], 1), l0.wo)
    I = cfg.intermediate_size
    gate_cat = torch.cat([p.layers[0].w_gate_up[: I // tp] for p in parts], 0)
    assert torch.equal(gate_cat, l0.w_gate_up[:I])
    assert torch.equal(torch.cat([p.layers[0].w_down for p in parts], 1), l0.w_down)
    head = torch.cat([p.lm_head[: p.vocab_local] for p in parts], 0)
    assert torch.equal(head, full.lm_head)
    sp = make_shard_spec(cfg, tp, 1)
    assert sp.vocab_chunk % 128 == 0 and sp.vocab_chunk * tp >= cfg.vocab_size


def test_cluster_planner_ranks_layouts():
    cfg = preset("qwen3-8b")
    plans = plan_cluster(cfg, 8, GPU_PRESETS["b200"], batch=64, ctx=1280)
    assert plans and all(p["gpus"] == 8 for p in plans)
    assert plans[0]["fits"]
    one = plan_cluster(cfg, 1, GPU_PRESETS["b200"], batch=64, ctx=1280)[0]
    assert 2.0 < one["ms_per_step"] < 8.0 and one["bound"] == "memory"
    big = preset("llama3-70b")
    assert not plan_cluster(big, 1, GPU_PRESETS["a100"], batch=8, ctx=1024)[0]["fits"]
    assert runnable(cfg, 3, 1, False)[0] is False


def test_expert_placement_balances_a_skewed_load():
    st = ExpertStats(1, 8)
    st.record(0, [0] * 50 + [1] * 20 + list(range(2, 8)) * 5)
    plan = plan_placement(st.load(0), ranks=4, slots_per_rank=3)
    assert sum(plan["replicas"]) == 12 and plan["replicas"][0] >= 2
    assert all(len(r) == 3 for r in plan["rank_experts"])
    assert plan["imbalance"] < 1.6
    with pytest.raises(ValueError):
        plan_placement([0.5, 0.5, 0.0], ranks=1, slots_per_rank=2)
