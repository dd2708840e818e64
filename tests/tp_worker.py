"""Child process of the tensor-parallel tests: one rank of a TP group (gloo on CPU, NCCL or the
fused peer-memory path on GPUs). Compares this layout's greedy tokens and last-step logits with
a single-device run of the same model on the same rank, and prints one line of JSON on rank 0."""
import faulthandler
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fllm_b200.comm import Group, init_distributed  # noqa: E402
from fllm_b200.config import EngineConfig, ParallelConfig, preset  # noqa: E402
from fllm_b200.parallel.tp import LibraryTP, make_tp_runtime  # noqa: E402
from fllm_b200.runtime import LLMEngine, SamplingParams  # noqa: E402


def ep_a2a_main():
    """Expert-parallel all-to-all across real GPUs: every rank owns a slice of the experts and a set
    of rows; rows travel to the experts' ranks and back through peer memory. Compared with the fp32
    oracle that has all experts local."""
    from types import SimpleNamespace
    from fllm_b200.comm.ep_a2a import EpAllToAll, moe_ffn_a2a_phases
    from fllm_b200.config import ModelConfig
    from fllm_b200.models.moe import moe_reference
    from fllm_b200.models.weights import LayerWeights
    from fllm_b200.ops.native import NativeOps
    rank, world, local = init_distributed("nccl", timeout_s=120)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    grp = Group()
    H, I, E, k, T = 256, 128, 16, 4, 40
    cfg = ModelConfig(hidden_size=H, num_experts=E, experts_per_token=k, moe_intermediate_size=I, act="swiglu_oai",
                      expert_bias=True)

    def rnd(shape, seed, scale=1.0):
        g = torch.Generator().manual_seed(seed)
        return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(dev)
    full = LayerWeights(attn_norm=None, wqkv=None, wo=None, ffn_norm=None)
    full.router_w, full.router_b = rnd((E, H), 1, 0.2), rnd((E,), 2, 0.1)
    full.exp_gate_up, full.exp_gate_up_b = rnd((E, 2 * I, H), 3, 0.05), rnd((E, 2 * I), 4, 0.1)
    full.exp_down, full.exp_down_b = rnd((E, H, I), 5, 0.05), rnd((E, H), 6, 0.1)
    per = E // world
    sl = slice(rank * per, (rank + 1) * per)
    lw = LayerWeights(attn_norm=None, wqkv=None, wo=None, ffn_norm=None)
    lw.router_w, lw.router_b = full.router_w, full.router_b
    lw.exp_gate_up, lw.exp_gate_up_b = full.exp_gate_up[sl].contiguous(), full.exp_gate_up_b[sl].contiguous()
    lw.exp_down, lw.exp_down_b = full.exp_down[sl].contiguous(), full.exp_down_b[sl].contiguous()
    ops = NativeOps(dev)
    ep = EpAllToAll(world, rank, H, per, max_tokens=64, k=k, device=dev, group=grp)
    dec = SimpleNamespace(cfg=cfg, ops=ops, act_kind=2)
    worst = 0.0
    for round_ in range(3):
        h = rnd((T, H), 100 + 13 * round_ + rank)
        out = None
        for out in moe_ffn_a2a_phases(dec, lw, ep, h):
            pass
        torch.cuda.synchronize()
        want = moe_reference(cfg, full, h, 0)
        worst = max(worst, float((out.float() - want).abs().max() / (want.abs().max() + 1e-6)))
    st = torch.tensor([ep.check_status() | ops.check_status(), int(worst * 1e6)], device=dev)
    torch.distributed.all_reduce(st, op=torch.distributed.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({"world": world, "status": int(st[0]), "err": int(st[1]) / 1e6}))
    torch.distributed.barrier()
    from fllm_b200.comm import shutdown_distributed
    shutdown_distributed()


def main():
    faulthandler.dump_traceback_later(int(os.environ.get("FLLM_HANG_DUMP", "150")), exit=True)
    if len(sys.argv) > 2 and sys.argv[2] == "ep_a2a":
        return ep_a2a_main()
    device_kind, backend, model = sys.argv[1], sys.argv[2], sys.argv[3]
    pp = int(sys.argv[4]) if len(sys.argv) > 4 else 1
    ep_mode = sys.argv[5] if len(sys.argv) > 5 else "none"          # none | allreduce | alltoall
    spec = sys.argv[6] if len(sys.argv) > 6 else "off"               # off | ngram | draft: speculation on the parallel engine
    rank, world, local = init_distributed("gloo" if device_kind == "cpu" else "nccl", timeout_s=120)
    dev = torch.device("cpu") if device_kind == "cpu" else torch.device("cuda", local)
    cfg = preset(model)
    if model == "tiny-llama":
        cfg.vocab_size = 2048
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=48, max_model_len=256, num_kv_blocks=96,
                      use_cuda_graphs=(device_kind != "cpu" and backend != "nccl-eager"))
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (7, 40, 21, 90, 3)]
    sp = SamplingParams(max_tokens=10)
    if spec != "off":
        prompts[1] = prompts[1][:8] * 5                                 # repetition gives the n-gram lookup something to find
        sp = SamplingParams(max_tokens=14)
    single = LLMEngine(cfg, ec, ParallelConfig(tp=1), device=dev, seed=3)
    want = single.generate(prompts, sp)
    from fllm_b200.comm import make_tp_pp_groups
    tp = world // pp
    grp, pp_grp, stage, tp_rank = make_tp_pp_groups(tp, pp)
    if backend == "fused":
        tp_rt = make_tp_runtime(tp, tp_rank, dev, backend="fused", group=grp, hidden=cfg.hidden_size,
                                max_tokens=ec.max_num_batched_tokens)
    else:
        tp_rt = LibraryTP(grp)
    par = ParallelConfig(tp=tp, pp=pp, expert_parallel=ep_mode != "none",
                         ep_dispatch=ep_mode if ep_mode != "none" else "allreduce")
    if spec == "ngram":
        import dataclasses
        ec = dataclasses.replace(ec, speculative="ngram")
    eng = LLMEngine(cfg, ec, par, device=dev, tp_group=tp_rt, tp_rank=tp_rank, seed=3,
                    pp_group=pp_grp, stage=stage)
    if spec == "draft":
        eng.enable_draft_model(cfg, k=3, seed=3)                         # same seed: the draft equals the target
    got = eng.generate(prompts, sp)

    def last_logits(e):
        if pp > 1:
            return torch.zeros(1)
        e.add_request(prompts[3][:40], SamplingParams(max_tokens=1))
        step = e.scheduler.schedule()
        batch = e._build_batch(step)
        lg = e.decoder.full_logits(e.decoder.forward(batch)).float()
        toks = lg.argmax(-1).int()
        e._commit(step, toks.tolist())
        return lg[-1].cpu()

    a, b_ = last_logits(single), last_logits(eng)
    logit_err = float((a - b_).abs().max() / (a.abs().max() + 1e-6))
    status = 0
    if hasattr(tp_rt, "check_status"):
        status = tp_rt.check_status()
    # every token of the parallel run, teacher-forced through the single-device engine: how far below the best
    # logit it sits, as a fraction of the row's logit span (0 = the single-device choice, a hair = a bf16 near-tie)
    worst_gap = 0.0
    for p_, o in zip(prompts, got):
        lg = single.token_logits(p_ + o)[len(p_) - 1:len(p_) - 1 + len(o)]
        for j, t in enumerate(o):
            row = lg[j]
            worst_gap = max(worst_gap, float((row.max() - row[t]) / (row.max() - row.min())))
    if rank == 0:
        agree = sum(a == b for o, r in zip(got, want) for a, b in zip(o, r))
        total = sum(len(o) for o in want)
        print(json.dumps({"backend": getattr(tp_rt, "backend", "?"), "world": world, "agree": agree, "total": total,
                          "worst_gap": worst_gap, "status": status, "spec_proposed": eng.stats.spec_proposed,
                          "spec_accepted": eng.stats.spec_accepted, "graph_steps": eng.stats.graph_steps, "logit_err": logit_err}), flush=True)
    from fllm_b200.comm import shutdown_distributed
    eng.close()
    single.close()
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
    if hasattr(tp_rt, "close"):
        tp_rt.close()
    shutdown_distributed()


if __name__ == "__main__":
    main()
