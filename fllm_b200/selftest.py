"""Built-in self-tests (``python -m fllm_b200 selftest-cpu | -gpu | -comm | -parallel``).

They need nothing but the installed package: no test tree, no test runner. Each check is a
small function that raises on failure; a run prints one line per check and returns the number
of failures as the exit code. Plays the role of the reference's ``selftest-*`` sub-commands
(rust/engine/src/cpu_selftest.rs, rust/engine/src/backend/selftest*.rs,
rust/engine/src/comm/selftest.rs:20-87, rust/engine/src/parallel/selftest.rs:24-72).

``selftest-comm`` and ``selftest-parallel`` start their ranks as child processes of this same
module (``python -m fllm_b200.selftest --worker ...``) with a loop-back rendezvous; on CPU the
ranks use gloo, whose sums this package takes in rank order, so every check there is exact.
"""
from __future__ import annotations

import json
import os
import socket
import subprocess
import sys
import time
import traceback
from typing import Callable, List, Tuple

import torch


def _run(checks: List[Tuple[str, Callable[[], None]]]) -> int:
    failed = 0
    for name, fn in checks:
        t0 = time.time()
        try:
            fn()
            print(f"ok    {name} ({time.time() - t0:.2f}s)", flush=True)
        except Exception:
            failed += 1
            print(f"FAIL  {name}\n{traceback.format_exc()}", flush=True)
    print(f"{len(checks) - failed} passed, {failed} failed", flush=True)
    return failed


def _close(a, b, tol):
    err = (a.float() - b.float()).abs().max().item()
    scale = b.float().abs().max().item() + 1e-6
    if err > tol * scale:
        raise AssertionError(f"max abs err {err:.4g} against scale {scale:.4g} (tolerance {tol})")


# ------------------------------------------------------------------------------------------- CPU
def _check_codecs():
    import numpy as np
    from .formats import quant
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 512), dtype=np.float32)
    for name, qt, tol in (("Q8_0", quant.Q8_0, 0.02), ("Q4_0", quant.Q4_0, 0.2), ("Q4_K", quant.Q4_K, 0.15),
                          ("Q5_K", quant.Q5_K, 0.08), ("Q6_K", quant.Q6_K, 0.04), ("F16", quant.F16, 1e-3)):
        y = quant.dequantize(quant.quantize(x, qt), qt, 4, 512)
        rel = float(np.abs(y - x).max() / np.abs(x).max())
        if rel > tol:
            raise AssertionError(f"{name}: round-trip error {rel:.3f} above {tol}")


def _check_gguf_round_trip():
    import tempfile
    import numpy as np
    from .formats.gguf import TYPE_ID, GgufReader, GgufWriter
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "t.gguf")
        w = GgufWriter(path)
        w.add("general.architecture", "llama")
        w.add("llama.block_count", 2)
        w.add("tokenizer.ggml.tokens", ["a", "b", "c"])
        t = np.arange(24, dtype=np.float32).reshape(4, 6)
        w.add_tensor("x.weight", (4, 6), TYPE_ID["F32"], t)
        w.write()
        r = GgufReader(path)
        assert r.metadata["llama.block_count"] == 2 and r.metadata["tokenizer.ggml.tokens"] == ["a", "b", "c"]
        got = np.frombuffer(r.tensor_bytes("x.weight"), dtype=np.float32).reshape(4, 6)
        assert np.array_equal(got, t)


def _tiny_engine(device, **kw):
    from .config import EngineConfig, preset
    from .runtime import LLMEngine
    cfg = preset("qwen3-tiny")
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=kw.pop("budget", 32), max_model_len=256, num_kv_blocks=96, **kw)
    return cfg, LLMEngine(cfg, ec, device=device, seed=3)


def _prompts(vocab, lens=(3, 17, 50, 33)):
    g = torch.Generator().manual_seed(1)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def _check_engine_chunking_and_cache():
    from .runtime import SamplingParams
    cfg, small = _tiny_engine("cpu", budget=16)
    _, big = _tiny_engine("cpu", budget=256)
    p = _prompts(cfg.vocab_size)
    sp = SamplingParams(max_tokens=6)
    a, b = small.generate(p, sp), big.generate(p, sp)
    assert a == b, "chunked prefill changed the greedy text"
    assert small.generate(p, sp) == a, "a prefix-cache hit changed the greedy text"
    assert small.blocks.stats["prefix_hits"] >= 1


def _check_cpu_native_engine():
    import tempfile
    from .cpu_engine import CpuEngine, write_tiny_llama_gguf
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tiny.gguf")
        cfg = write_tiny_llama_gguf(path)
        eng = CpuEngine(path)
        out1 = eng.generate(list(range(1, 20)), 8)
        eng2 = CpuEngine(path)
        assert out1 == eng2.generate(list(range(1, 20)), 8) and len(out1) == 8
        assert all(0 <= t < cfg.vocab_size for t in out1)


def selftest_cpu() -> int:
    return _run([("packed codecs round trip", _check_codecs), ("gguf write / read", _check_gguf_round_trip),
                 ("engine: chunked prefill and prefix cache keep the text", _check_engine_chunking_and_cache),
                 ("native cpu engine on a packed tiny model", _check_cpu_native_engine)])


def selftest_sanitize() -> int:
    """The CPU self-test again in a child process against the AddressSanitizer + UBSan build of the native CPU
    library (`_build.build_cpu_sanitized`), the sanitizer runtime preloaded. Any report fails the run."""
    from . import _build
    rt = _build.sanitizer_runtime()
    if not rt:
        print("sanitize: the compiler ships no AddressSanitizer runtime; skipped")
        return 0
    lib = _build.build_cpu_sanitized()
    env = dict(os.environ, LD_PRELOAD=rt, FLLM_CPU_LIB=str(lib), OMP_NUM_THREADS="2",
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=0:exitcode=23", UBSAN_OPTIONS="print_stacktrace=1:halt_on_error=1")
    p = subprocess.run([sys.executable, "-m", "fllm_b200.selftest", "cpu"], env=env, capture_output=True, text=True, timeout=1200)
    bad = [l for l in p.stderr.splitlines() if "AddressSanitizer" in l or "runtime error:" in l]
    print(p.stdout[-2000:])
    if p.returncode != 0 or bad:
        print("\n".join(bad[:20]) or p.stderr[-2000:])
        print(f"sanitize: FAILED (exit {p.returncode})")
        return 1
    print("sanitize: clean (AddressSanitizer + UndefinedBehaviorSanitizer)")
    return 0


# ------------------------------------------------------------------------------------------- GPU
def _gpu_ops():
    from .ops.native import NativeOps
    from .ops.reference import RefOps
    return NativeOps(torch.device("cuda:0")), RefOps()


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _check_gpu_linear():
    ops, ref = _gpu_ops()
    for T, N, K in ((1, 256, 128), (64, 4096, 4096), (300, 1000, 320), (2048, 1024, 512)):
        x, w = _rand((T, K), 1), _rand((N, K), 2, 0.05)
        _close(ops.linear(x, w), ref.linear(x, w), 2e-2)
    if ops.check_status():
        raise AssertionError("kernel status word set")


def _check_gpu_norm_rope_glu():
    ops, ref = _gpu_ops()
    x, d, w = _rand((13, 4096), 1), _rand((13, 4096), 2), _rand((4096,), 3)
    xa, xb = x.clone(), x.clone()
    _close(ops.rmsnorm(xa, d, w, 1e-6), ref.rmsnorm(xb, d, w, 1e-6), 1e-2)
    assert torch.equal(xa, xb)
    gu = _rand((33, 2048), 4)
    for kind in (0, 1, 2):
        _close(ops.glu(gu, kind), ref.glu(gu, kind), 1e-2)
    T, hq, hkv, D, bs, nb = 21, 8, 2, 128, 16, 8
    qkv = _rand((T, (hq + 2 * hkv) * D), 5)
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    slots = torch.randperm(nb * bs, device="cuda")[:T].int()
    inv = (1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))).contiguous()
    kc, vc = torch.zeros(nb, hkv, bs, D, device="cuda", dtype=torch.bfloat16), torch.zeros(nb, hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    kr, vr = kc.clone(), vc.clone()
    qa = ops.rope_kv_write(qkv.clone(), pos, slots, inv, None, None, kc, vc, hq, hkv, D, D, 0, 1e-6, 1.0)
    qb = ref.rope_kv_write(qkv.clone(), pos, slots, inv, None, None, kr, vr, hq, hkv, D, D, 0, 1e-6, 1.0)
    _close(qa, qb, 2e-2)
    _close(kc, kr, 2e-2)
    assert torch.equal(vc, vr)


def _check_gpu_attention_and_argmax():
    from .models.decoder import StepBatch
    ops, ref = _gpu_ops()
    B, L, bs, hq, hkv, D = 5, 70, 16, 8, 2, 128
    nblk = -(-L // bs)
    kc, vc = _rand((B * nblk, hkv, bs, D), 1), _rand((B * nblk, hkv, bs, D), 2)
    tables = torch.arange(B * nblk, device="cuda", dtype=torch.int32).view(B, nblk)
    q = _rand((B, hq * D), 3)
    row_seq = torch.arange(B, device="cuda", dtype=torch.int32)
    pos = torch.full((B,), L - 1, device="cuda", dtype=torch.int32)
    meta = StepBatch(None, pos, None, row_seq, tables, None, num_seqs=B, num_tokens=B, max_kv_len=L, all_decode=True,
                     seq_lens=torch.full((B,), L, device="cuda", dtype=torch.int32),
                     q_starts=torch.arange(B + 1, device="cuda", dtype=torch.int32))
    want = ref.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5)
    _close(ops.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5, meta=meta), want, 2e-2)
    _close(ops.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5), want, 2e-2)
    lg = _rand((9, 50257), 4)
    assert torch.equal(ops.argmax(lg).long(), lg.float().argmax(-1))


def _check_gpu_engine_matches_cpu():
    """Greedy text of the tiny model: sm_100a kernels + CUDA graphs against the PyTorch fp32 path. A token may
    differ only where the reference's two best logits are nearly tied."""
    from .runtime import SamplingParams
    cfg, gpu = _tiny_engine("cuda:0")
    _, cpu = _tiny_engine("cpu")
    p = _prompts(cfg.vocab_size)
    sp = SamplingParams(max_tokens=8)
    a, b = gpu.generate(p, sp), cpu.generate(p, sp)
    same = sum(int(x == y) for ta, tb in zip(a, b) for x, y in zip(ta, tb))
    total = sum(len(t) for t in b)
    if same < 0.9 * total:
        raise AssertionError(f"only {same} of {total} greedy tokens agree with the fp32 reference")
    if gpu.ops.check_status():
        raise AssertionError("kernel status word set")


def selftest_gpu() -> int:
    if not torch.cuda.is_available():
        print("selftest-gpu: no CUDA device")
        return 1
    return _run([("tcgen05 GEMM vs fp32 matmul", _check_gpu_linear), ("norm / rope+kv / gated activations", _check_gpu_norm_rope_glu),
                 ("paged attention (tensor-core and generic) and argmax", _check_gpu_attention_and_argmax),
                 ("engine on the GPU vs the fp32 reference engine", _check_gpu_engine_matches_cpu)])


# ------------------------------------------------------------------------------------------- ranks
def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def spawn_ranks(world: int, worker_args: List[str], timeout: float = 300.0, extra_env=None) -> List[dict]:
    """Start `world` child processes of this module with a loop-back rendezvous; returns the JSON line each
    printed. Raises if a rank fails or prints nothing."""
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1", NCCL_NVLS_ENABLE="0")
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, "-m", "fllm_b200.selftest", "--worker"] + worker_args, env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    try:
        for p in procs:
            o, e = p.communicate(timeout=timeout)
            outs.append((p.returncode, o, e))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    res = []
    for r, (rc, o, e) in enumerate(outs):
        lines = [l for l in o.splitlines() if l.startswith("{")]
        if rc != 0 or not lines:
            raise RuntimeError(f"rank {r} failed (exit {rc}): {e[-1500:]}")
        res.append(json.loads(lines[-1]))
    return res


def _worker_comm() -> dict:
    """Exact-integer collectives on this rank's group (values chosen so that every sum is exact in fp32)."""
    from .comm import Group, init_distributed
    dev = os.environ.get("FLLM_SELFTEST_DEVICE", "cpu")
    rank, world, local = init_distributed("gloo" if dev == "cpu" else "nccl", timeout_s=60)
    device = torch.device("cpu") if dev == "cpu" else torch.device("cuda", local)
    g = Group()
    r, n = g.rank, g.size
    x = (torch.arange(6, dtype=torch.float32) + 10 * r).to(device)
    want = (torch.arange(6, dtype=torch.float32) * n + 10 * sum(range(n))).to(device)
    assert torch.equal(g.all_reduce(x.clone()), want), "all_reduce"
    ag = g.all_gather(torch.tensor([r, r * r], dtype=torch.int64, device=device))
    assert ag.tolist() == [[i, i * i] for i in range(n)], "all_gather"
    rs = g.reduce_scatter(torch.ones(2 * n, 3, device=device) * (r + 1))
    assert torch.equal(rs.cpu(), torch.full((2, 3), float(sum(range(1, n + 1))))), "reduce_scatter"
    b = torch.tensor([7.0, 8.0], device=device) if r == n - 1 else torch.zeros(2, device=device)
    assert g.broadcast(b, src=n - 1).tolist() == [7.0, 8.0], "broadcast"
    recv = g.all_to_all([torch.full((d + 1, 2), float(r * 100 + d), device=device) for d in range(n)])
    assert [t.shape[0] for t in recv] == [r + 1] * n and [float(t[0, 0]) for t in recv] == [s * 100.0 + r for s in range(n)], "all_to_all"
    if n > 1:
        if r == 0:
            g.send(torch.tensor([41.0, 42.0], device=device), dst=n - 1)
        if r == n - 1:
            assert g.recv(torch.zeros(2, device=device), src=0).tolist() == [41.0, 42.0], "send/recv"
    g.barrier()
    return {"rank": rank, "ok": True}


def _worker_parallel(model: str, pp: int) -> dict:
    """This layout's greedy text against a single-device engine of the same model built on the same rank."""
    from .comm import init_distributed, make_tp_pp_groups
    from .config import EngineConfig, ParallelConfig, preset
    from .parallel.tp import LibraryTP
    from .runtime import LLMEngine, SamplingParams
    rank, world, _ = init_distributed("gloo", timeout_s=120)
    cfg = preset(model)
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=48, max_model_len=256, num_kv_blocks=96, use_cuda_graphs=False)
    prompts = _prompts(cfg.vocab_size, (7, 40, 21))
    sp = SamplingParams(max_tokens=8)
    want = LLMEngine(cfg, ec, ParallelConfig(tp=1), device="cpu", seed=3).generate(prompts, sp)
    tp = world // pp
    grp, pp_grp, stage, tp_rank = make_tp_pp_groups(tp, pp)
    eng = LLMEngine(cfg, ec, ParallelConfig(tp=tp, pp=pp), device="cpu", tp_group=LibraryTP(grp), tp_rank=tp_rank, seed=3,
                    pp_group=pp_grp, stage=stage)
    got = eng.generate(prompts, sp)
    out = {"rank": rank, "world": world, "tp": tp, "pp": pp}
    if rank == 0:
        out["agree"] = sum(int(a == b) for x, y in zip(got, want) for a, b in zip(x, y))
        out["total"] = sum(len(w) for w in want)
    return out


def selftest_comm(worlds=(1, 2, 4), device: str = "cpu") -> int:
    def check(n):
        def fn():
            res = spawn_ranks(n, ["comm"], extra_env={"FLLM_SELFTEST_DEVICE": device})
            assert len(res) == n and all(r["ok"] for r in res)
        return fn
    return _run([(f"exact collectives on {n} {device} rank(s)", check(n)) for n in worlds])


def selftest_parallel() -> int:
    def check(world, pp):
        def fn():
            r0 = spawn_ranks(world, ["parallel", "qwen3-tiny", str(pp)])[0]
            # pipeline stages compute the same bits; tensor-parallel sums round partials to bf16, so a near-tie may flip
            need = r0["total"] if world == pp else int(0.8 * r0["total"])
            if r0["agree"] < need:
                raise AssertionError(f"{r0['agree']} of {r0['total']} greedy tokens agree with the single-device engine")
        return fn
    return _run([("tensor parallel x2 == single device (gloo)", check(2, 1)), ("pipeline x2 == single device (gloo)", check(2, 2)),
                 ("tensor x2 . pipeline x2 == single device (gloo)", check(4, 2))])


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "--worker":
        kind = argv[1]
        out = _worker_comm() if kind == "comm" else _worker_parallel(argv[2], int(argv[3]))
        print(json.dumps(out), flush=True)
        sys.stdout.flush()
        os._exit(0)               # leave without tearing the process group down rank by rank
    which = argv[0] if argv else "cpu"
    return {"cpu": selftest_cpu, "gpu": selftest_gpu, "comm": selftest_comm, "parallel": selftest_parallel,
            "sanitize": selftest_sanitize}[which]()


if __name__ == "__main__":
    sys.exit(main())
