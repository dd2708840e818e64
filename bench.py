#!/usr/bin/env python
"""Headline benchmark: decode throughput of a Qwen3-8B-shaped bf16 model serving 64
concurrent requests (1024-token random prompts, greedy), tensor-parallel over N GPUs.

    python bench.py --gpus 1 --steps 128 --warmup 8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

One "step" is one engine decode step of the whole batch (64 new tokens). Two numbers:

* ``value``      device-timed (CUDA events, max over ranks): K replays of the captured
                 decode step of the live batch, weights (16 GB) streamed from HBM each step,
                 so the working set is far larger than L2;
* ``e2e.value``  the same K steps through ``LLMEngine.step()``: scheduler, batch building,
                 pinned-host -> device copy of the step inputs, graph replay, device -> host
                 read of the sampled ids.

``--config N`` selects another of the five benchmark configurations (default 2, the one above):
1 = tiny Llama Q4_K on the CPU engine (batch 1), 3 = Llama-3-70B-shaped block-FP8 model (TP over all
ranks, batch 128, prompts 512-4096), 4 = gpt-oss-120b-shaped MXFP4 mixture of experts (expert parallel
over all ranks, batch 256 x 2048), 5 = Llama-3.1-70B-shaped NVFP4 model as TP x PP2 (batch 32 x 4096).
Weights are drawn directly in their packed format, layer by layer. ``--model`` overrides the shape
(a tiny preset checks a configuration's plumbing on one GPU).

``--impl reference`` reports why the reference cannot run here (it is a Rust workspace;
no Rust toolchain is installed and pip cannot install it).
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index: int, period: float = 0.1):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), 0
        self._halt = threading.Event()
        if os.environ.get("FLLM_BENCH_SAMPLER", "thread") == "off":
            self.nv = None
            return
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                    nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._halt.wait(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz or None, "reasons": sorted(self.reasons)}


def reference_arm(args) -> None:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is a Rust workspace (Cargo.toml only, no setup.py/pyproject.toml): "
                       "pip cannot install it and no cargo/rustc exists in this image",
    }))


# model preset, weight format, batch, prompt-length range, output tokens, pipeline stages, expert parallel
CONFIGS = {
    2: dict(model="qwen3-8b", fmt="bf16", batch=64, prompt=(1024, 1024), out=256, pp=1, ep=False),
    3: dict(model="llama3-70b", fmt="fp8_block", batch=128, prompt=(512, 4096), out=512, pp=1, ep=False),
    4: dict(model="gpt-oss-120b", fmt="mxfp4", batch=256, prompt=(2048, 2048), out=256, pp=1, ep=True),
    5: dict(model="llama3-70b", fmt="nvfp4", batch=32, prompt=(4096, 4096), out=512, pp=2, ep=False),
}


def config1_cpu(args) -> None:
    """Tiny Llama-architecture decoder, Q4_K weights in a synthetic GGUF, CPU engine, batch 1: prompt of 128
    uniform-random ids, 64 greedy tokens, paged f16 KV in 16-token blocks."""
    import tempfile
    from fllm_b200.cpu_engine import CpuEngine, write_tiny_llama_gguf
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tiny-llama-q4k.gguf")
        cfg = write_tiny_llama_gguf(path, seed=0)
        eng = CpuEngine(path)
        for _ in range(max(args.warmup, 3)):
            eng.bench(128, 64, seed=0)
        runs = [eng.bench(128, 64, seed=0) for _ in range(max(1, min(args.steps, 16)))]
        eng.close()
    dec = statistics.median(r["decode_tok_s"] for r in runs)
    pre = statistics.median(r["prompt_tok_s"] for r in runs)
    print(json.dumps({
        "metric": "decode tok/s (CPU engine, batch 1)", "value": round(dec, 1), "unit": "tok/s", "n_gpus": 0,
        "steps": len(runs), "warmup": max(args.warmup, 3), "ms_per_step": round(1e3 / dec, 4), "higher_is_better": True,
        "scaling": "none", "vs_baseline": None, "dtype": "q4_k weights x q8_k activations, f16 KV",
        "data": "synthetic (uniform random token ids, N(0,0.02) weights quantised to Q4_K)",
        "config": {"config": 1, "model": cfg.name, "global_batch": 1, "seq_len": 128, "output_tokens": 64,
                   "parallelism": "cpu", "threads": os.cpu_count()},
        "prefill_tok_s": round(pre, 1), "gpu_launches": 0,
    }))


def main() -> None:
    if os.environ.get("FLLM_HANG_DUMP"):      # debugging aid: dump all Python stacks and exit if the run stalls
        faulthandler.dump_traceback_later(int(os.environ["FLLM_HANG_DUMP"]), exit=True)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 4, 5])
    ap.add_argument("--model", default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--weight-format", default=None)
    ap.add_argument("--kv-cache-type", default="bf16", choices=["bf16", "fp8_e4m3"],
                    help="element type of the paged KV pool (the headline configuration uses bf16)")
    ap.add_argument("--backend", default=os.environ.get("FLLM_TP_BACKEND", "auto"),
                    help="tensor-parallel collectives: auto | fused | nccl")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--profile-prefill", action="store_true",
                    help="bracket the third 2048-token prefill step with cudaProfilerStart/Stop and exit after the prefill")
    ap.add_argument("--profile-step", action="store_true",
                    help="bracket ONE replay of the decode step with cudaProfilerStart/Stop (for a profiler's "
                         "launch list, run with --profile-from-start off) and exit")
    args = ap.parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:
            reference_arm(args)
        return
    args.warmup = max(args.warmup, 3)
    if args.config == 1:
        return config1_cpu(args)
    conf = CONFIGS[args.config]
    args.model = args.model or conf["model"]
    args.batch = args.batch or conf["batch"]
    p_lo, p_hi = conf["prompt"]
    if args.prompt_len:
        p_lo = p_hi = args.prompt_len
    args.prompt_len = p_hi

    import torch
    from fllm_b200.comm import init_distributed
    from fllm_b200.config import EngineConfig, ParallelConfig, preset
    from fllm_b200.parallel.tp import make_tp_runtime
    from fllm_b200.runtime import LLMEngine, SamplingParams

    rank, world, local = init_distributed()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = preset(args.model)
    cfg.weight_format = args.weight_format or conf["fmt"]
    pp = conf["pp"] if world % conf["pp"] == 0 and world >= conf["pp"] else 1
    tp = world // pp
    # Prompts are prefilled 2048 tokens per step while the sequences that are already through decode
    # along (decode-first scheduling), so the first sequences are `stagger` tokens ahead of the last when
    # the timed region starts: leave room for that, or they would reach the length limit inside it.
    stagger = -(-args.batch * p_hi // 2048) + 2
    out_len = args.warmup + 2 * args.steps + 8 + stagger
    ec = EngineConfig(max_num_seqs=args.batch, max_num_batched_tokens=2048, block_size=16,
                      max_model_len=p_hi + out_len + 16, enable_prefix_caching=False,
                      use_cuda_graphs=not args.no_graphs, kv_cache_dtype=args.kv_cache_type)
    ec.num_kv_blocks = args.batch * (-(-ec.max_model_len // 16)) + 16
    par = ParallelConfig(tp=tp, pp=pp, expert_parallel=bool(conf["ep"] and cfg.is_moe and tp > 1), ep_dispatch="alltoall")
    pp_grp, stage, tp_rank = None, 0, rank
    if pp > 1:
        from fllm_b200.comm import make_tp_pp_groups
        tp_grp, pp_grp, stage, tp_rank = make_tp_pp_groups(tp, pp)
        tp_rt = make_tp_runtime(tp, tp_rank, dev, backend=args.backend, group=tp_grp, hidden=cfg.hidden_size,
                                max_tokens=ec.max_num_batched_tokens)
    else:
        tp_rt = make_tp_runtime(world, rank, dev, backend=args.backend, hidden=cfg.hidden_size,
                                max_tokens=ec.max_num_batched_tokens)
    eng = LLMEngine(cfg, ec, par, device=dev, tp_group=tp_rt, tp_rank=tp_rank, seed=0, pp_group=pp_grp, stage=stage)

    g = torch.Generator().manual_seed(1234)
    lens = [args.prompt_len] * args.batch if p_lo == p_hi else \
        torch.randint(p_lo, p_hi + 1, (args.batch,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    sp = SamplingParams(max_tokens=out_len + 64, ignore_eos=True)
    for p in prompts:
        eng.add_request(p, sp)

    def sync_all():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return float(t.item())

    # ---- prefill (chunked, 2048 tokens per step), device-timed
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall = time.perf_counter()
    e0.record()
    ttft = None
    n_prefill_steps = 0
    while any(not r.output for r in eng.requests.values()):
        mark = args.profile_prefill and n_prefill_steps == 2
        if mark:
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
        eng.step()
        if mark:
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        n_prefill_steps += 1
        if ttft is None and any(r.output for r in eng.requests.values()):
            ttft = time.perf_counter() - t_wall
    e1.record()
    sync_all()
    prefill_ms = max_over_ranks(e0.elapsed_time(e1))
    prefill_tok_s = sum(lens) / (prefill_ms / 1e3)
    if args.profile_prefill:
        if rank == 0:
            print(json.dumps({"profiled_prefill_step": 2, "prefill_steps": n_prefill_steps, "prefill_tok_s": prefill_tok_s}))
        eng.close()
        return

    # ---- warm-up decode steps (captures the graph)
    for _ in range(args.warmup):
        eng.step()
    eng.drain()
    assert len(eng.scheduler.running) == args.batch, "batch shrank during warm-up"

    # ---- kernel-only: K replays of the captured decode step of the live batch
    sampler = ClockSampler(local)
    sampler.start()
    launches_per_step = None
    if eng._graphs:
        graph = next(iter(eng._graphs.values()))
        step_desc = eng.scheduler.schedule()             # builds the static inputs for this state
        eng._build_batch(step_desc, pad_to=graph.bucket)
        launches_per_step = graph.launches
        sync_all()
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        sync_all()
        dev_ms = max_over_ranks(e0.elapsed_time(e1))
        if args.profile_step:
            torch.cuda.profiler.start()
            graph.replay()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
            sampler.stop()
            print(json.dumps({"profiled_step": True, "ms_per_step": dev_ms / args.steps, "launches": launches_per_step}))
            eng.close()
            return
        # finish the scheduled-but-not-committed step so the engine state stays consistent
        toks = graph.tokens.tolist()
        eng._commit(step_desc, toks)
    else:
        dev_ms = None

    # ---- end to end: K engine steps through the public API
    import gc
    eng.settle_host()
    gc_events = []

    def _gc_cb(phase, info, _t=[0.0]):
        if phase == "start":
            _t[0] = time.perf_counter()
        else:
            gc_events.append([info.get("generation"), round((time.perf_counter() - _t[0]) * 1e3, 2)])
    gc.callbacks.append(_gc_cb)
    h2d0, d2h0 = eng.stats.h2d_bytes, eng.stats.d2h_bytes
    l0 = eng.stats.kernel_launches
    sync_all()
    t0 = time.perf_counter()
    e0.record()
    step_ms = []
    for _ in range(args.steps):
        ts = time.perf_counter()
        eng.step()
        step_ms.append((time.perf_counter() - ts) * 1e3)
    eng.drain()                 # the last launched step's ids are read inside the timed region
    e1.record()
    sync_all()
    gc.callbacks.remove(_gc_cb)
    assert len(eng.scheduler.running) == args.batch, "batch shrank inside the timed region"
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    e2e_dev_ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop()
    if dev_ms is None:
        dev_ms = e2e_dev_ms
    itl = []
    for r in eng.requests.values():
        tt = r.token_times[-args.steps:]
        itl += [b - a for a, b in zip(tt, tt[1:])]
    # time to first token per request (all requests are submitted together before the first step)
    ttfts = [r.first_token_time - r.arrival for r in eng.requests.values() if r.first_token_time is not None]
    status = eng.ops.check_status()

    tokens = args.batch * args.steps
    value = tokens / (dev_ms / 1e3)
    e2e_value = tokens / e2e_s
    if rank == 0:
        print(json.dumps({
            "metric": "decode tok/s (device-timed, max over ranks)",
            "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dev_ms / args.steps, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16" if cfg.weight_format == "bf16" else f"bf16 activations, {cfg.weight_format} weights",
            "data": "synthetic (uniform random token ids, random-init N(0,0.02) weights)",
            "config": {"config": args.config, "model": cfg.name, "global_batch": args.batch,
                       "seq_len": args.prompt_len if p_lo == p_hi else f"{p_lo}-{p_hi}",
                       "parallelism": (f"tp{tp}" + (f"xpp{pp}" if pp > 1 else "") + ("+ep" if par.expert_parallel else "")),
                       "tp_backend": getattr(tp_rt, "backend", "none"), "weight_format": cfg.weight_format, "kv_cache": args.kv_cache_type,
                       "kv": "paged bf16, 16-token blocks", "chunked_prefill": 2048,
                       "cuda_graphs": not args.no_graphs, "async_scheduling": eng._async_ok(),
                       "l2": "inputs larger than L2: 16 GB of weights + KV streamed per step"},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 1), "unit": "tok/s",
                    "h2d_bytes_per_step": (eng.stats.h2d_bytes - h2d0) // args.steps,
                    "d2h_bytes_per_step": (eng.stats.d2h_bytes - d2h0) // args.steps,
                    "ms_per_step": round(e2e_s * 1e3 / args.steps, 4),
                    "step_ms_p50": round(statistics.median(step_ms), 4), "step_ms_max": round(max(step_ms), 4),
                    "slowest_steps": sorted(((round(v, 2), i) for i, v in enumerate(step_ms)), reverse=True)[:4],
                    "gc_pauses_ms": sorted(gc_events, key=lambda e: -e[1])[:4]},
            "gpu_launches": (launches_per_step or 0) * args.steps + (eng.stats.kernel_launches - l0),
            "prefill_tok_s": round(prefill_tok_s, 1), "ttft_s_first": round(ttft or 0.0, 4),
            "ttft_p50_s": round(statistics.median(ttfts), 4) if ttfts else None,
            "itl_p50_ms": round(statistics.median(itl) * 1e3, 4) if itl else None,
            "kernel_status": status,
        }))
    if world > 1:
        from fllm_b200.comm import shutdown_distributed
        eng.close()
        torch.distributed.barrier()
        tp_rt.close()
        shutdown_distributed()


if __name__ == "__main__":
    main()
