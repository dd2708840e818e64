"""Command line: ``python -m fllm_b200 <command>``.

Sub-commands keep the reference's names (rust/engine/src/cli.rs:16-170,
rust/engine/src/bin/serve.rs:85-119): serve, run, bench, bench-kernel, devices, formats,
inspect, quantize, make-tiny-model, plan-cluster, selftest-cpu / -gpu / -comm / -parallel.
Serve flags use the reference's spellings (--model --host --port --model-name --api-key --ctx
--max-seqs --max-batched-tokens -tp -pp --expert-parallel --kv-cache-type ...).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from typing import List, Optional


def _add_engine_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", required=True, help="preset name (random weights), .gguf file or checkpoint directory")
    p.add_argument("--device", default=None, help="cuda[:i] or cpu (default: cuda when available)")
    p.add_argument("--ctx", "--max-model-len", dest="ctx", type=int, default=8192)
    p.add_argument("--max-seqs", "--max-num-seqs", dest="max_seqs", type=int, default=256)
    p.add_argument("--max-batched-tokens", "--max-num-batched-tokens", dest="max_batched_tokens", type=int, default=2048)
    p.add_argument("--gpu-memory-utilization", type=float, default=0.90)
    p.add_argument("--kv-cache-type", default="bf16")
    p.add_argument("--kv-blocks", type=int, default=0)
    p.add_argument("--no-prefix-cache", action="store_true")
    p.add_argument("--no-cuda-graphs", action="store_true")
    p.add_argument("--scheduling-policy", default="fcfs", choices=["fcfs", "priority"])
    p.add_argument("--preemption", default="recompute", choices=["recompute", "swap"])
    p.add_argument("--kv-tier-host-gb", type=float, default=0.0, help="host memory for evicted prefix-cache blocks")
    p.add_argument("--kv-tier-disk-dir", default=None, help="directory for blocks that fall out of the host tier (default $FLLM_KV_DISK_DIR)")
    p.add_argument("--kv-tier-disk-gb", type=float, default=0.0)
    p.add_argument("--state-cache-gb", type=float, default=0.0,
                   help="recurrent / hybrid models: host memory for state checkpoints on block boundaries (prefix reuse)")
    p.add_argument("--speculative", default="off", choices=["off", "ngram", "suffix", "draft"])
    p.add_argument("--draft-model", default=None)
    p.add_argument("--draft-tokens", type=int, default=4)
    p.add_argument("-tp", "--tensor-parallel", dest="tp", type=int, default=1)
    p.add_argument("-pp", "--pipeline-parallel", dest="pp", type=int, default=1)
    p.add_argument("--expert-parallel", action="store_true")
    p.add_argument("--ep-dispatch", default="alltoall", choices=["alltoall", "allreduce"])
    p.add_argument("--distributed-backend", default="fused", choices=["fused", "nccl"])
    p.add_argument("--tokenizer", default=None, help="tokenizer.json / directory / .gguf (default: embedded or byte-level)")
    p.add_argument("--seed", type=int, default=0)


def build_engine(args):
    import torch
    from .config import EngineConfig, ParallelConfig, preset
    from .runtime import LLMEngine
    from .tokenizer import load_tokenizer

    device = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    ec = EngineConfig.from_env(
        max_num_seqs=args.max_seqs, max_num_batched_tokens=args.max_batched_tokens, max_model_len=args.ctx,
        gpu_memory_utilization=args.gpu_memory_utilization, kv_cache_dtype=args.kv_cache_type,
        num_kv_blocks=args.kv_blocks, enable_prefix_caching=not args.no_prefix_cache,
        use_cuda_graphs=not args.no_cuda_graphs, scheduling_policy=args.scheduling_policy,
        preemption=args.preemption, speculative=args.speculative, draft_tokens=args.draft_tokens, seed=args.seed,
        kv_tier_host_gb=args.kv_tier_host_gb, kv_tier_disk_dir=args.kv_tier_disk_dir, kv_tier_disk_gb=args.kv_tier_disk_gb,
        state_cache_gb=getattr(args, "state_cache_gb", 0.0))
    par = ParallelConfig(tp=args.tp, pp=args.pp, expert_parallel=args.expert_parallel, ep_dispatch=args.ep_dispatch,
                         distributed_backend=args.distributed_backend)
    weights, tok_path = None, args.tokenizer
    from . import hub
    args.model = hub.resolve(args.model)          # a path, a store entry, an alias that was pulled, or a preset name
    if args.model.endswith(".gguf") or os.path.isdir(args.model):
        from .formats.loader import load_model
        cfg, weights, embedded_tok = load_model(args.model, device)
        tok_path = tok_path or embedded_tok
    else:
        cfg = preset(args.model)
    tp_rt, rank = None, 0
    if par.world > 1:
        from .comm import init_distributed
        from .parallel.tp import make_tp_runtime
        rank, world, local = init_distributed()
        if world != par.world:
            raise SystemExit(f"tp x pp = {par.world} but WORLD_SIZE = {world}; launch one process per GPU with torchrun")
        device = f"cuda:{local}" if torch.cuda.is_available() else "cpu"
        tp_rt = make_tp_runtime(par.tp, rank % par.tp, device, par.distributed_backend, hidden=cfg.hidden_size,
                                max_tokens=ec.max_num_batched_tokens)
    try:
        tokenizer = load_tokenizer(tok_path, cfg.vocab_size)
    except Exception as e:
        print(f"[fllm_b200] tokenizer unavailable ({e}); falling back to the byte tokenizer", file=sys.stderr)
        tokenizer = load_tokenizer(None, max(cfg.vocab_size, 258))
    eng = LLMEngine(cfg, ec, par, device=device, weights=weights, tp_group=tp_rt, tp_rank=rank, seed=args.seed,
                    eos_token_id=getattr(tokenizer, "eos_token_id", None))
    return eng, tokenizer


def _encoder_dir(path: str) -> bool:
    """A Hugging Face directory whose config names a BERT-family encoder."""
    cfg = os.path.join(path, "config.json")
    if not os.path.isfile(cfg):
        return False
    try:
        return json.load(open(cfg)).get("model_type") in ("bert", "roberta", "xlm-roberta")
    except (OSError, ValueError):
        return False


def cmd_serve_encoder(args, path: str) -> int:
    """`serve` on an encoder checkpoint: embeddings / pooling / classify / score / rerank routes."""
    import torch
    from .models.encoder import Encoder, load_hf_encoder
    from .ops import get_ops
    from .server.encoder_app import serve_encoder
    from .tokenizer import load_tokenizer
    dev = args.device if getattr(args, "device", None) else ("cuda:0" if torch.cuda.is_available() else "cpu")
    cfg, w = load_hf_encoder(path, dev, torch.bfloat16 if str(dev).startswith("cuda") else torch.float32)
    enc = Encoder(cfg, w, get_ops("cuda" if str(dev).startswith("cuda") else "cpu"), dev)
    tok = load_tokenizer(path if os.path.exists(os.path.join(path, "tokenizer.json")) else None, cfg.vocab_size)
    serve_encoder(enc, tok, args.host, args.port, args.model_name or os.path.basename(path.rstrip("/")), args.api_key, args.log_level,
                  ssl_certfile=args.ssl_certfile, ssl_keyfile=args.ssl_keyfile)
    return 0


def cmd_serve(args) -> int:
    from .server.app import serve
    if args.model and os.path.isdir(args.model) and _encoder_dir(args.model):
        return cmd_serve_encoder(args, args.model)
    eng, tok = build_engine(args)
    eng.warm_up(buckets=[b for b in eng.cfg.graph_buckets if b <= 64])
    controller = None
    if eng.par.world > 1:
        # One front end for the whole rank group: rank 0 serves HTTP and announces every admission, abort and
        # step; the other ranks run the worker loop (launch one process per GPU with torch.distributed.run).
        from .comm import shutdown_distributed
        from .runtime.step_control import ControlChannel, StepController
        from .server.app import make_guided_builder
        controller = StepController(eng, ControlChannel(timeout_s=args.control_timeout),
                                    guided_builder=make_guided_builder(eng, tok, args.tool_parser))
        if not controller.ch.is_leader:
            why = controller.follow()
            eng.close()
            if why == "comm":
                print("[fllm_b200] control channel lost; this rank leaves", file=sys.stderr, flush=True)
                os._exit(3)                  # a broken group cannot be torn down collectively
            shutdown_distributed()
            return 0
    serve(eng, tok, args.host, args.port, args.model_name or os.path.basename(args.model), args.api_key, args.log_level,
          tool_parser=args.tool_parser, reasoning_parser=args.reasoning_parser,
          response_cache_entries=args.response_cache_entries, otlp_endpoint=args.otlp_endpoint, controller=controller,
          cors_origins=args.cors_origin, rate_limit_rps=args.rate_limit, ssl_certfile=args.ssl_certfile,
          ssl_keyfile=args.ssl_keyfile)
    return 0


def cmd_run(args) -> int:
    from .runtime import SamplingParams
    from .tokenizer import render_chat
    eng, tok = build_engine(args)
    prof = None
    if os.environ.get("FLLM_PROFILE", "0") not in ("", "0"):
        # a CUDA-event pair around every operator call; eager steps only (events cannot sit inside a captured graph)
        from .utils.telemetry import OpProfiler
        eng.cfg.use_cuda_graphs = False
        prof = eng.ops = eng.decoder.ops = OpProfiler(eng.ops)
    text = args.prompt if args.raw else render_chat(getattr(tok, "chat_template", None), [{"role": "user", "content": args.prompt}])
    ids = tok.encode(text, add_bos=True)
    sp = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p, top_k=args.top_k,
                        seed=args.seed)
    out = eng.generate([ids], sp)[0]
    print(tok.decode(out))
    if prof is not None:
        print(prof.table(), file=sys.stderr)
    return 0


def cmd_devices(args) -> int:
    import torch
    info = {"cuda_available": torch.cuda.is_available(), "devices": []}
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        peers = [j for j in range(torch.cuda.device_count()) if j != i and torch.cuda.can_device_access_peer(i, j)]
        info["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}.{p.minor}", "sms": p.multi_processor_count,
                                "memory_gib": round(p.total_memory / 2 ** 30, 1), "p2p_peers": peers})
    from .ops import _lib
    info["native_cuda_library"] = _lib.have_cuda_lib()
    print(json.dumps(info, indent=1) if args.json else "\n".join(
        [f"cuda:{d['index']} {d['name']} sm_{d['sm']} {d['sms']} SMs {d['memory_gib']} GiB p2p->{d['p2p_peers']}"
         for d in info["devices"]] or ["no CUDA device; the CPU engine is available"]))
    return 0


def cmd_formats(args) -> int:
    from .formats.gguf import GGML_TYPES
    print("weight formats (name, values/block, bytes/block):")
    for tid, (name, bs, bb) in sorted(GGML_TYPES.items()):
        print(f"  {tid:4d} {name:8s} {bs:4d} {bb:4d}")
    print("  1001 NVFP4      16    9   (e2m1 x16 + e4m3 scale; fp32 tensor scale kept apart)")
    print("  1002 FP8_E4M3    1    1   (block-wise fp32 scales kept apart, 128x128 typical)")
    return 0


def cmd_inspect(args) -> int:
    from .formats.gguf import GgufReader
    r = GgufReader(args.file)
    print(f"{args.file}: {len(r.tensors)} tensors, {len(r.metadata)} metadata keys")
    for k, v in r.metadata.items():
        s = repr(v)
        print(f"  {k} = {s[:100] + '...' if len(s) > 100 else s}")
    if args.tensors:
        for t in r.tensors.values():
            print(f"  {t.name:40s} {t.type_name:6s} {tuple(t.shape)} @{t.offset} {t.nbytes} B")
    return 0


def cmd_quantize(args) -> int:
    """Re-quantise the 2-D tensors of a GGUF file to another packed type."""
    from .formats.convert import quantize_gguf
    print(json.dumps(quantize_gguf(args.input, args.output, args.type)))
    return 0


def cmd_convert(args) -> int:
    """Hugging Face checkpoint directory -> GGUF (optionally quantised)."""
    from .formats.convert import convert_checkpoint
    from . import hub
    print(json.dumps(convert_checkpoint(hub.resolve(args.input), args.output, args.type)))
    return 0


def cmd_gguf_tool(args) -> int:
    from .formats import convert as C
    if args.cmd == "gguf-set":
        edits = {}
        for kv in args.set or []:
            k, _, v = kv.partition("=")
            try:
                edits[k] = json.loads(v)
            except json.JSONDecodeError:
                edits[k] = v
        print(json.dumps(C.gguf_set(args.input, args.output, edits, args.remove or [])))
    elif args.cmd == "gguf-split":
        print(json.dumps(C.gguf_split(args.input, args.output_prefix, args.max_tensors)))
    elif args.cmd == "gguf-merge":
        print(json.dumps(C.gguf_merge(args.first_shard, args.output)))
    else:
        print(json.dumps(C.merge_lora_gguf(args.base, args.lora, args.output, args.type)))
    return 0


def cmd_store(args) -> int:
    """pull / list / rm / show on the local model store."""
    from . import hub
    try:
        if args.cmd == "pull":
            print(json.dumps(hub.pull(args.ref, args.name, args.link)))
        elif args.cmd == "list":
            for e in hub.list_models():
                print(f"{e['name']:40s} {e['bytes'] / 2 ** 30:8.2f} GiB  {e['source']}")
            if args.catalog:
                for k, v in sorted(hub.catalog().items()):
                    print(f"alias {k:34s} -> {v}")
        elif args.cmd == "rm":
            if not hub.remove(args.name):
                print(f"no model {args.name!r} in the store", file=sys.stderr)
                return 1
        else:
            print(json.dumps(hub.show(args.name), indent=1))
    except hub.HubError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


def cmd_ppl(args) -> int:
    """Perplexity of a text file: the file is tokenised, cut into windows of --ctx tokens, each window scored."""
    import math
    eng, tok = build_engine(args)
    text = open(args.file, encoding="utf-8", errors="replace").read()
    ids = tok.encode(text, add_bos=True)
    win = min(args.window or eng.cfg.max_model_len, eng.cfg.max_model_len)
    total, count = 0.0, 0
    for off in range(0, max(len(ids) - 1, 1), win):
        chunk = ids[off: off + win]
        if len(chunk) < 2:
            break
        lp = eng.score_tokens(chunk)
        total += -sum(lp)
        count += len(lp)
        print(f"[{off + len(chunk)}/{len(ids)}] ppl so far {math.exp(total / max(count, 1)):.4f}", file=sys.stderr, flush=True)
    print(json.dumps({"tokens": count, "nll": total / max(count, 1), "perplexity": math.exp(total / max(count, 1))}))
    return 0


def cmd_chat(args) -> int:
    """Interactive chat in the terminal (line input; /reset clears the history, /quit leaves)."""
    from .runtime import SamplingParams
    from .tokenizer import render_chat
    eng, tok = build_engine(args)
    history: list = [{"role": "system", "content": args.system}] if args.system else []
    sp = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p, top_k=args.top_k)
    while True:
        try:
            line = input("> ")
        except EOFError:
            break
        if line.strip() in ("/quit", "/exit"):
            break
        if line.strip() == "/reset":
            history = history[:1] if args.system else []
            continue
        if not line.strip():
            continue
        history.append({"role": "user", "content": line})
        ids = tok.encode(render_chat(getattr(tok, "chat_template", None), history), add_bos=True)
        rid = eng.add_request(ids, sp)
        out: list = []
        shown = 0
        while eng.has_unfinished():
            for ev in eng.step():
                if ev.request_id == rid:
                    out.extend(t for t in ev.token_ids if t != getattr(tok, "eos_token_id", None))
                    text = tok.decode(out)
                    if not text.endswith("\ufffd"):
                        print(text[shown:], end="", flush=True)
                        shown = len(text)
        print()
        history.append({"role": "assistant", "content": tok.decode(out)})
    return 0


def cmd_make_tiny(args) -> int:
    from .cpu_engine import write_tiny_llama_gguf
    cfg = write_tiny_llama_gguf(args.output, seed=args.seed)
    print(f"wrote {args.output}: {cfg.num_layers} layers, hidden {cfg.hidden_size}, vocab {cfg.vocab_size}, Q4_K")
    return 0


def cmd_plan_cluster(args) -> int:
    from .config import preset
    from .parallel.planner import GPU_PRESETS, plan_cluster
    plans = plan_cluster(preset(args.model), args.gpus, GPU_PRESETS[args.gpu], batch=args.batch, ctx=args.ctx,
                         weight_bits=args.weight_bits)
    for p in plans[: args.top]:
        print(json.dumps(p))
    return 0


def _selftest(which: str) -> int:
    from . import selftest
    return selftest.main([which])


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "bench-kernel":            # its own option set (a REMAINDER argument would refuse leading options)
        from .bench_kernel import main as bench_kernel_main
        return bench_kernel_main(argv[1:]) or 0
    ap = argparse.ArgumentParser(prog="fllm_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve", help="HTTP server (OpenAI / Anthropic / Ollama dialects on one port)")
    _add_engine_flags(s)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--model-name", default=None)
    s.add_argument("--api-key", default=os.environ.get("FLLM_API_KEY"))
    s.add_argument("--log-level", default="info")
    s.add_argument("--tool-parser", default=None, choices=["hermes", "llama3_json", "mistral"])
    s.add_argument("--reasoning-parser", default=None, choices=["think", "think_open"])
    s.add_argument("--response-cache-entries", type=int, default=256, help="0 disables the response cache")
    s.add_argument("--cors-origin", action="append", default=None, help="allowed CORS origin (repeatable; '*' allows all)")
    s.add_argument("--rate-limit", type=float, default=0.0, help="requests per second per API key / client address (0 = off)")
    s.add_argument("--ssl-certfile", default=None)
    s.add_argument("--ssl-keyfile", default=None)
    s.add_argument("--control-timeout", type=float, default=float(os.environ.get("FLLM_CONTROL_TIMEOUT", "30")),
                   help="seconds a rank waits for the step-control message of a multi-rank server before it gives up")
    s.add_argument("--otlp-endpoint", default=os.environ.get("OTEL_EXPORTER_OTLP_ENDPOINT"),
                   help="export request spans as OTLP/HTTP JSON to <endpoint>/v1/traces")
    s.set_defaults(fn=cmd_serve)
    rt = sub.add_parser("router", help="front several serve processes (data-parallel replicas) with one port")
    rt.add_argument("--replica", action="append", required=True, help="base URL of a replica, e.g. http://127.0.0.1:8001 (repeat)")
    rt.add_argument("--host", default="127.0.0.1")
    rt.add_argument("--port", type=int, default=8080)
    rt.add_argument("--policy", default="prefix", choices=["prefix", "least_loaded", "round_robin"])
    rt.add_argument("--log-level", default="info")
    rt.set_defaults(fn=lambda a: (__import__("fllm_b200.server.router", fromlist=["serve_router"]).serve_router(
        a.replica, a.host, a.port, a.policy, a.log_level), 0)[1])
    bs = sub.add_parser("bench-serve", help="load a running server over HTTP and report TTFT / ITL / throughput")
    bs.add_argument("--url", default="http://127.0.0.1:8000")
    bs.add_argument("--num-prompts", type=int, default=64)
    bs.add_argument("--concurrency", type=int, default=16)
    bs.add_argument("--prompt-len", type=int, default=256)
    bs.add_argument("--max-tokens", type=int, default=64)
    bs.add_argument("--vocab", type=int, default=1000)
    bs.set_defaults(fn=lambda a: (print(json.dumps(__import__("fllm_b200.server.bench_serve", fromlist=["main"]).main(
        a.url, num_prompts=a.num_prompts, concurrency=a.concurrency, prompt_len=a.prompt_len, max_tokens=a.max_tokens,
        vocab=a.vocab), indent=1)), 0)[1])
    r = sub.add_parser("run", help="generate once from a prompt")
    _add_engine_flags(r)
    r.add_argument("prompt")
    r.add_argument("--raw", action="store_true", help="do not apply the chat template")
    r.add_argument("--max-tokens", type=int, default=128)
    r.add_argument("--temperature", type=float, default=0.0)
    r.add_argument("--top-p", type=float, default=1.0)
    r.add_argument("--top-k", type=int, default=0)
    r.set_defaults(fn=cmd_run)
    d = sub.add_parser("devices")
    d.add_argument("--json", action="store_true")
    d.set_defaults(fn=cmd_devices)
    sub.add_parser("formats").set_defaults(fn=cmd_formats)
    i = sub.add_parser("inspect")
    i.add_argument("file")
    i.add_argument("--tensors", action="store_true")
    i.set_defaults(fn=cmd_inspect)
    q = sub.add_parser("quantize")
    q.add_argument("input")
    q.add_argument("output")
    q.add_argument("type")
    q.set_defaults(fn=cmd_quantize)
    cv = sub.add_parser("convert", help="Hugging Face checkpoint -> GGUF")
    cv.add_argument("input")
    cv.add_argument("output")
    cv.add_argument("--type", default="F16")
    cv.set_defaults(fn=cmd_convert)
    gs = sub.add_parser("gguf-set", help="copy a GGUF with metadata keys changed")
    gs.add_argument("input"); gs.add_argument("output")
    gs.add_argument("--set", action="append", metavar="KEY=JSON")
    gs.add_argument("--remove", action="append", metavar="KEY")
    gs.set_defaults(fn=cmd_gguf_tool)
    gsp = sub.add_parser("gguf-split")
    gsp.add_argument("input"); gsp.add_argument("output_prefix"); gsp.add_argument("--max-tensors", type=int, default=128)
    gsp.set_defaults(fn=cmd_gguf_tool)
    gm = sub.add_parser("gguf-merge")
    gm.add_argument("first_shard"); gm.add_argument("output")
    gm.set_defaults(fn=cmd_gguf_tool)
    ml = sub.add_parser("merge-lora", help="bake a PEFT LoRA into a GGUF")
    ml.add_argument("base"); ml.add_argument("lora"); ml.add_argument("output"); ml.add_argument("--type", default=None)
    ml.set_defaults(fn=cmd_gguf_tool)
    pl = sub.add_parser("pull", help="add a model to the local store (path or hf://org/name[@rev][:file])")
    pl.add_argument("ref"); pl.add_argument("--name", default=None); pl.add_argument("--link", action="store_true")
    pl.set_defaults(fn=cmd_store)
    ls = sub.add_parser("list"); ls.add_argument("--catalog", action="store_true"); ls.set_defaults(fn=cmd_store)
    rm = sub.add_parser("rm"); rm.add_argument("name"); rm.set_defaults(fn=cmd_store)
    sh = sub.add_parser("show"); sh.add_argument("name"); sh.set_defaults(fn=cmd_store)
    pp = sub.add_parser("ppl", help="perplexity of a text file")
    _add_engine_flags(pp)
    pp.add_argument("--file", required=True)
    pp.add_argument("--window", type=int, default=0)
    pp.set_defaults(fn=cmd_ppl)
    ch = sub.add_parser("chat", help="interactive chat in the terminal")
    _add_engine_flags(ch)
    ch.add_argument("--system", default=None)
    ch.add_argument("--max-tokens", type=int, default=512)
    ch.add_argument("--temperature", type=float, default=0.7)
    ch.add_argument("--top-p", type=float, default=0.95)
    ch.add_argument("--top-k", type=int, default=0)
    ch.set_defaults(fn=cmd_chat)
    t = sub.add_parser("make-tiny-model")
    t.add_argument("output")
    t.add_argument("--seed", type=int, default=0)
    t.set_defaults(fn=cmd_make_tiny)
    pc = sub.add_parser("plan-cluster")
    pc.add_argument("--model", default="qwen3-8b")
    pc.add_argument("--gpus", type=int, default=8)
    pc.add_argument("--gpu", default="b200")
    pc.add_argument("--batch", type=int, default=64)
    pc.add_argument("--ctx", type=int, default=2048)
    pc.add_argument("--weight-bits", type=float, default=16)
    pc.add_argument("--top", type=int, default=5)
    pc.set_defaults(fn=cmd_plan_cluster)
    bk = sub.add_parser("bench-kernel")
    bk.add_argument("rest", nargs=argparse.REMAINDER)
    bk.set_defaults(fn=lambda a: __import__("fllm_b200.bench_kernel", fromlist=["main"]).main(a.rest) or 0)
    b = sub.add_parser("bench")
    b.add_argument("rest", nargs=argparse.REMAINDER)
    b.set_defaults(fn=lambda a: subprocess.call([sys.executable, os.path.join(os.path.dirname(os.path.dirname(
        os.path.abspath(__file__))), "bench.py")] + a.rest))
    for which in ("cpu", "gpu", "comm", "parallel", "sanitize"):
        sub.add_parser(f"selftest-{which}").set_defaults(fn=lambda a, w=which: _selftest(w))
    args = ap.parse_args(argv)
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    sys.exit(main())
