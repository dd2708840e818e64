"""Kernel micro-benchmarks (``python -m fllm_b200.bench_kernel``): every hot op of the
decoder at the shapes of a model preset, timed with CUDA events after warm-up, with an
L2 flush between iterations, and reported against the measured machine peaks
(``MEASURED_PEAKS.json`` when present). The library GEMM (cuBLAS through torch.matmul)
is timed next to ours as the bar to clear. Plays the role of the reference's
``bench-kernel`` sub-command (rust/engine/src/bench_kernel.rs).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _peaks():
    for p in ("MEASURED_PEAKS.json", os.path.join(os.path.dirname(os.path.dirname(__file__)), "MEASURED_PEAKS.json")):
        if os.path.exists(p):
            d = json.load(open(p))
            return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, flush_mb: int = 256):
        self.flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn, iters: int = 10, warmup: int = 3) -> float:
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            self.flush.zero_()                      # evict L2
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]                     # median, ms


def run_case(case: str, reps: int = 4) -> None:
    """One kernel family, a handful of launches, inputs larger than L2 but far below a GB-scale footprint:
    a self-ending workload for a profiler capture or a quick look (``bench-kernel --case gemm_decode``).
    Cases: gemm_decode (64 tokens x gate_up of an 8B model), gemm_prefill (2048 tokens), gemm_pair_prefill (the same on
    CTA pairs, cta_group::2), attn_decode
    (64 sequences at 1152 context), attn_prefill (2 x 1024 tokens), attn_prefill_long (4 x 4096 tokens),
    fp8_prefill, gemm_fp4_decode (64 tokens x NVFP4 gate_up), gemm_mx4_decode / gemm_mx4_prefill / gemm_mx8_decode /
    gemm_nvf4_decode / gemm_nvf4_prefill (block-scaled MXFP4 / MXFP8 / NVFP4 gate_up), gemv_q4k (one token x 4-bit
    gate_up on the dp4a kernel), tp_rs_gemm / tp_norm / tp_ag_gemm (the fused
    tensor-parallel kernels with two virtual ranks on one device), mla_decode / mla_decode_cc / mla_prefill (latent
    attention on the tensor-core and the CUDA-core kernel), mamba2_decode / mamba2_prefill / gdn_decode (recurrent
    scans; these print their CUDA-event time and the state or cache bytes per second)."""
    from .ops.native import NativeOps, Fp8BlockLinear, quantize_weight_fp8_block
    ops = NativeOps(torch.device("cuda:0"))
    bf = dict(device="cuda", dtype=torch.bfloat16)
    if case in ("gemm_decode", "gemm_prefill", "gemm_pair_prefill"):
        T = 64 if case == "gemm_decode" else 2048
        x = torch.randn(T, 4096, **bf)
        w = torch.randn(24576, 4096, **bf) * 0.02
        y = torch.empty(T, 24576, **bf)
        fn = (lambda: ops.k.linear_pair(x, w, None, y, ops.status)) if case == "gemm_pair_prefill" else (lambda: ops.linear(x, w, out=y))
    elif case == "gemm_fp4_decode":
        from .ops.fp4 import Fp4Weight
        x = torch.randn(64, 4096, **bf)
        codes = torch.randint(0, 256, (24576, 2048), device="cuda", dtype=torch.uint8)
        scales = torch.full((24576, 256), 0x38, device="cuda", dtype=torch.uint8)      # e4m3 1.0
        q = Fp4Weight(codes, scales, 0, 0.01)
        y = torch.empty(64, 24576, **bf)
        fn = lambda: ops.linear(x, q, out=y)
    elif case in ("gemm_mx4_decode", "gemm_mx4_prefill", "gemm_mx8_decode", "gemm_nvf4_decode", "gemm_nvf4_prefill"):
        from .ops.mx import MxWeight, Nvfp4TcWeight
        T = 2048 if case.endswith("prefill") else 64
        x = torch.randn(T, 4096, **bf)
        a4 = "mx4" in case
        if "nvf4" in case:
            q = Nvfp4TcWeight(torch.randint(0, 256, (24576, 2048), device="cuda", dtype=torch.uint8),
                              torch.full((24576, 256), 0x38, device="cuda", dtype=torch.uint8), 0.01)       # e4m3 1.0
        else:
            q = MxWeight(torch.randint(0, 256, (24576, 2048 if a4 else 4096), device="cuda", dtype=torch.uint8).clamp_(0, 0x7E),
                         torch.full((24576, 128), 120, device="cuda", dtype=torch.uint8), a4)
        q.atoms
        y = torch.empty(T, 24576, **bf)
        fn = lambda: ops.linear(x, q, out=y)
    elif case == "gemv_q4k":
        from .ops.int4 import Int4Weight
        x = torch.randn(1, 4096, **bf)
        q = Int4Weight(torch.randint(0, 256, (24576, 2048), device="cuda", dtype=torch.uint8),
                       torch.full((24576, 128, 2), 0.01, device="cuda", dtype=torch.bfloat16))
        y = torch.empty(1, 24576, **bf)
        fn = lambda: ops.linear(x, q, out=y)
    elif case in ("tp_rs_gemm", "tp_norm", "tp_ag_gemm"):
        # the fused tensor-parallel kernels with two virtual ranks on this one device (plain pointers instead
        # of IPC mappings; the ranks' kernels run phase by phase): 2048 tokens, o_proj shard -> norm -> gate_up shard
        from .comm.symm import FusedTP
        T, H, I = 2048, 4096, 12288
        ranks = FusedTP.local_group(2, H, T)
        a = [torch.randn(T, H // 2, **bf) for _ in range(2)]
        wo = [torch.randn(H, H // 2, **bf) * 0.02 for _ in range(2)]
        wgu = torch.randn(I, H, **bf) * 0.02
        nw = torch.ones(H, **bf)
        res = [torch.zeros(T // 2, H, **bf) for _ in range(2)]

        def fn():
            for r in range(2):
                ranks[r].linear_rs(a[r], wo[r], None, False)
            for r in range(2):
                ranks[r]._rs_expected = ranks[0]._rs_expected
                ranks[r].norm(res[r], T, True, nw, 1e-6, 0.0, False)
            for r in range(2):
                ranks[r].linear_ag(T, wgu)
    elif case == "fp8_prefill":
        x = torch.randn(2048, 4096, **bf)
        wq, sw = quantize_weight_fp8_block(torch.randn(8192, 4096, **bf) * 0.02)
        lin = Fp8BlockLinear(ops, wq, sw)
        fn = lambda: lin(x)
    elif case in ("attn_decode", "attn_prefill", "attn_prefill_long"):
        from .models.decoder import StepBatch
        B, L, bs, hq, hkv, D = 64, 1152, 16, 32, 8, 128
        nb = B * (L // bs)
        kc = torch.randn(nb, hkv, bs, D, **bf)
        vc = torch.randn_like(kc)
        tables = torch.arange(nb, device="cuda", dtype=torch.int32).view(B, L // bs)
        if case == "attn_decode":
            q = torch.randn(B, hq * D, **bf)
            meta = StepBatch(None, None, None, None, tables, None, num_seqs=B, num_tokens=B, max_kv_len=L,
                             seq_lens=torch.full((B,), L, device="cuda", dtype=torch.int32),
                             q_starts=torch.arange(B + 1, device="cuda", dtype=torch.int32))
        elif case == "attn_prefill_long":
            n, Lq = 4, 4096
            tables = torch.arange(n * (Lq // bs), device="cuda", dtype=torch.int32).view(n, Lq // bs)
            q = torch.randn(n * Lq, hq * D, **bf)
            meta = StepBatch(None, None, None, None, tables, None, num_seqs=n, num_tokens=n * Lq, max_kv_len=Lq,
                             seq_lens=torch.full((n,), Lq, device="cuda", dtype=torch.int32),
                             q_starts=torch.arange(n + 1, device="cuda", dtype=torch.int32) * Lq,
                             max_q_len=Lq, min_q_len=Lq)
        else:
            q = torch.randn(2048, hq * D, **bf)
            meta = StepBatch(None, None, None, None, tables, None, num_seqs=2, num_tokens=2048, max_kv_len=1024,
                             seq_lens=torch.full((2,), 1024, device="cuda", dtype=torch.int32),
                             q_starts=torch.tensor([0, 1024, 2048], device="cuda", dtype=torch.int32),
                             max_q_len=1024, min_q_len=1024)
        fn = lambda: ops.attention(q, kc, vc, tables, None, None, hq, hkv, D, D ** -0.5, meta=meta)
    elif case in ("mla_decode", "mla_decode_cc", "mla_prefill"):
        # latent attention of DeepSeek-V2-Lite (16 heads): 64 sequences at 1152 tokens of context, or a 1024-token prefill
        # chunk of 2 sequences; the pool (64 x 1152 x 576 bf16 = 85 MB for decode) is read once per launch
        H, bs = 16, 16
        B, L, Lq = (64, 1152, 1) if case != "mla_prefill" else (2, 1024, 1024)
        nblk = B * (L // bs)
        cache = (torch.randn(nblk, bs, 576, **bf) * 0.3)
        tables = torch.arange(nblk, device="cuda", dtype=torch.int32).view(B, L // bs)
        row_seq = torch.arange(B, device="cuda", dtype=torch.int32).repeat_interleave(Lq)
        pos = (torch.arange(L - Lq, L, device="cuda", dtype=torch.int32)).repeat(B)
        q_abs, q_pe = torch.randn(H, B * Lq, 512, **bf), torch.randn(B * Lq, H, 64, **bf)
        tc = case != "mla_decode_cc"
        fn = lambda: ops.attention_mla(q_abs, q_pe, cache, tables, row_seq, pos, 576 ** -0.5, L, tensor_cores=tc)
        nbytes = cache.numel() * 2
    elif case in ("mamba2_decode", "mamba2_prefill", "gdn_decode"):
        # Mamba-2 2.7B layer (80 heads x 64 x 128 state): 64 decode rows (state 2.6 MB per sequence, read and written), or one
        # 2048-token chunk; gated delta rule of Qwen3-Next (32 value heads x 128 x 128)
        B, n = (64, 1) if case != "mamba2_prefill" else (1, 2048)
        T = B * n
        qs = torch.arange(0, T + 1, n, device="cuda", dtype=torch.int32)
        ss = torch.arange(B, device="cuda", dtype=torch.int32)
        pos = (torch.arange(n, device="cuda", dtype=torch.int32) + (0 if n > 1 else 100)).repeat(B)
        if case == "gdn_decode":
            from .ops.recurrent import GATED_DELTA
            Hv, Hk, D = 32, 16, 128
            r, k = torch.randn(T, Hk * D, **bf), torch.randn(T, Hk * D, **bf)
            v, beta = torch.randn(T, Hv * D, **bf), torch.rand(T, Hv, **bf)
            w = -torch.rand(T, Hv, device="cuda")
            st = torch.zeros(B, Hv, D, D, device="cuda")
            fn = lambda: ops.matrix_state_scan(GATED_DELTA, r, k, v, None, None, w, None, beta, st, qs, ss, pos, Hv, D, D, 2, True, D ** -0.5)
        else:
            Hh, P, N = 80, 64, 128
            x, dt = torch.randn(T, Hh * P, **bf), torch.randn(T, Hh, **bf)
            Bm, Cm = torch.randn(T, N, **bf), torch.randn(T, N, **bf)
            A, D_, dtb = -torch.rand(Hh, device="cuda"), torch.ones(Hh, device="cuda"), torch.zeros(Hh, device="cuda")
            st = torch.zeros(B, Hh, P, N, device="cuda")
            fn = lambda: ops.mamba2_scan(x, dt, Bm, Cm, A, D_, dtb, st, qs, ss, pos, Hh, P, 1, N, 0.0, 1e30, max_q_len=n)
        nbytes = st.numel() * 4 * 2
    else:
        raise SystemExit(f"unknown case {case}")
    if case.startswith(("mla_", "mamba2_", "gdn_")):
        ms = Timer()(fn)
        hbm, _, which = _peaks()
        print(json.dumps({"case": case, "us": round(ms * 1e3, 1), "bytes": nbytes, "gbs": round(nbytes / ms / 1e6, 1),
                          "frac_of_" + which + "_copy_bw": round(nbytes / (ms * 1e-3) / (hbm * 1e9), 3)}))
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    print(case, "done; kernel status", ops.check_status())


NVLINK_GBS = 770.0       # measured peer-copy bandwidth per direction per GPU on this machine class


def tp_half_layer(args) -> None:
    """Roofline of the fused tensor-parallel half-layer: row-parallel GEMM -> reduce(-scatter) + residual +
    RMSNorm (+ all-gather) -> column-parallel GEMM, against the same half-layer on library collectives.
    Launch one process per GPU:

        python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
            -m fllm_b200.bench_kernel --tp-half-layer [--model qwen3-8b] [--tokens 64,2048]

    Times are CUDA events on the launching stream, max over ranks, L2 flushed between iterations. The
    roofline of a step is the slowest of: its FLOPs at the measured GEMM peak, its bytes over NVLink at
    the measured peer-copy bandwidth, and its weight bytes from HBM at the measured copy bandwidth (the
    last one is what binds a 64-token step)."""
    import torch.distributed as dist
    from .comm import Group, init_distributed, shutdown_distributed
    from .comm.symm import FusedTP
    from .config import preset
    from .ops.native import NativeOps

    rank, world, local = init_distributed("nccl", timeout_s=120)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cfg = preset(args.model)
    H, I = cfg.hidden_size, cfg.intermediate_size
    grp = Group()
    ops = NativeOps(dev)
    tokens = [int(t) for t in args.tokens.split(",")]
    tp = FusedTP(grp, dev, H, max(tokens))
    hbm, tflops, _ = _peaks()
    bf = dict(device=dev, dtype=torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(rank)
    wo = (torch.randn(H, H // world, generator=g, **bf) * 0.02)              # row-parallel (K cut)
    wgu = (torch.randn(2 * I // world, H, generator=g, **bf) * 0.02)         # column-parallel (N cut)
    nw = torch.ones(H, **bf)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def timed(fn):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        t = torch.tensor([tot / args.iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for T in tokens:
        a = torch.randn(T, H // world, generator=g, **bf)
        bc = tp.use_bcast(T)
        lo, hi = tp.my_rows(T)
        res = torch.zeros(T if bc else max(hi - lo, 1), H, **bf)

        def fused():
            tp.linear_rs(a, wo, None, bc)
            tp.norm(res, T, True, nw, 1e-6, 0.0, bc)
            return ops.linear(tp.ag_local[:T], wgu) if bc else tp.linear_ag(T, wgu)

        resl = torch.zeros(T, H, **bf)

        def library():
            y = ops.linear(a, wo)
            dist.all_reduce(y)
            h = ops.rmsnorm(resl, y, nw, 1e-6)
            return ops.linear(h, wgu)

        ms_f, ms_l = timed(fused), timed(library)
        flops = 2.0 * T * H * (H / world) + 2.0 * T * H * (2 * I / world)
        link = T * H * 2.0 * (world - 1) if bc else 2.0 * T * H * 2.0 * (world - 1) / world   # bytes out of one GPU
        wbytes = 2.0 * (wo.numel() + wgu.numel())
        t_c, t_l, t_m = flops / (tflops * 1e12), link / (NVLINK_GBS * 1e9), wbytes / (hbm * 1e9)
        roof = max(t_c, t_l, t_m)
        row = {"tp": world, "tokens": T, "layout": "broadcast" if bc else "scatter", "fused_us": ms_f * 1e3,
               "library_us": ms_l * 1e3, "roof_us": roof * 1e6, "bound": "mma" if roof == t_c else "nvlink" if roof == t_l else "hbm",
               "compute_us": t_c * 1e6, "nvlink_us": t_l * 1e6, "hbm_us": t_m * 1e6, "fused_frac": roof / (ms_f / 1e3),
               "library_frac": roof / (ms_l / 1e3), "status": tp.check_status() | ops.check_status()}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.json:
        json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "nvlink_gbs": NVLINK_GBS}, "rows": rows},
                  open(args.json, "w"), indent=1)
    dist.barrier()
    tp.close()
    shutdown_distributed()


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--tokens", default="1,16,64,128,256,2048,8192")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--json", default="")
    ap.add_argument("--fp4", action="store_true", help="only the packed FP4 (NVFP4 / MXFP4) decode GEMMs")
    ap.add_argument("--case", default="", help="run ONE kernel family a few times and exit (see run_case)")
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--tp-half-layer", action="store_true",
                    help="fused vs library tensor-parallel half-layer (one process per GPU under torch.distributed.run)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--vs-reference", action="store_true",
                    help="time our kernels next to the reference engine's own CUDA kernels (bench_reference.py)")
    ap.add_argument("--ref-lib", default=None, help="path of the reference kernel library (libfllmcuda.so)")
    args = ap.parse_args(argv)
    if args.vs_reference:
        from .bench_reference import run as run_vs_reference
        return run_vs_reference(args.model, args.ref_lib, args.json)
    if args.case:
        return run_case(args.case, args.reps)
    if args.tp_half_layer:
        if args.tokens == ap.get_default("tokens"):
            args.tokens = "64,2048"
        return tp_half_layer(args)
    from .config import preset
    from .ops.native import NativeOps

    cfg = preset(args.model)
    ops = NativeOps(torch.device("cuda:0"))
    hbm, tflops, src = _peaks()
    timer = Timer()
    H, I = cfg.hidden_size, cfg.intermediate_size // args.tp
    qkv = (cfg.q_size + 2 * cfg.kv_size) // args.tp
    shapes = {"qkv": (qkv, H), "o": (H, cfg.q_size // args.tp), "gate_up": (2 * I, H), "down": (H, I),
              "lm_head": (cfg.vocab_size // args.tp // 8 * 8, H)}
    rows = []
    if args.fp4:
        from .ops.fp4 import Fp4Weight
        from .ops.mx import MxWeight, Nvfp4TcWeight
        print(f"# peaks ({src}): {hbm} GB/s; bytes = packed weight + scales + activations")
        print("# nvfp4 / mxfp4: packed weights expanded in the kernel, bf16 activations (W4A16);")
        print("# mx4a8 / mx8a8: block-scaled MMA on MXFP4 / MXFP8 weights and MXFP8 activations, quantiser included;")
        print("# nvf4a4: block-scaled MMA on NVFP4 weights and NVFP4 activations, quantiser included")
        for name, (N, K) in shapes.items():
            if name == "lm_head":
                continue
            w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
            for fmt in ("nvfp4", "mxfp4", "mx4a8", "mx8a8", "nvf4a4"):
                if fmt in ("nvfp4", "mxfp4"):
                    q = Fp4Weight.from_dense(w, fmt)
                elif fmt == "nvf4a4":
                    q = Nvfp4TcWeight.from_dense(w.float())
                    q.atoms
                else:
                    q = MxWeight.from_dense(w.float(), "mxfp4" if fmt == "mx4a8" else "mxfp8")
                    q.atoms                                                   # built once, at load time
                for T in (1, 16, 64, 128, 2048):
                    if T > 128 and fmt in ("nvfp4", "mxfp4"):
                        continue
                    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
                    y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
                    ms = timer(lambda: ops.linear(x, q, out=y))
                    ms16 = timer(lambda: ops.linear(x, w, out=y))
                    byts = q.nbytes() + 2.0 * (T * K + T * N)
                    print(f"{name:8s} {fmt:6s} T={T:4d} N={N:6d} K={K:6d} {ms * 1e3:8.1f} us  (bf16 {ms16 * 1e3:7.1f} us)  "
                          f"{byts / ms / 1e6:6.0f} GB/s  frac {byts / (hbm * 1e9) / (ms / 1e3):.2f}  "
                          f"{2.0 * T * N * K / ms / 1e9:7.1f} TFLOP/s")
                    rows.append({"op": name, "fmt": fmt, "T": T, "us": ms * 1e3, "bf16_us": ms16 * 1e3, "gbs": byts / ms / 1e6})
            del w
        print("kernel status word:", ops.check_status())
        if args.json:
            json.dump({"rows": rows}, open(args.json, "w"), indent=1)
        return
    print(f"# peaks ({src}): {hbm} GB/s, {tflops} TFLOP/s bf16")
    print(f"{'op':10s} {'T':>6s} {'N':>7s} {'K':>6s} {'ours ms':>9s} {'cublas ms':>9s} {'TFLOP/s':>8s} {'GB/s':>7s} {'frac':>6s} {'bound':>5s}")
    for name, (N, K) in shapes.items():
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
        for T in [int(t) for t in args.tokens.split(",")]:
            if name == "lm_head" and T > 256:
                continue
            x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
            y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            ms = timer(lambda: ops.linear(x, w, out=y))
            ms_lib = timer(lambda: torch.matmul(x, w.t(), out=y))
            if T >= 256 and N >= 256 and N % 8 == 0:                 # the CTA-pair kernel on its own, whatever the planner picks
                ms_pair = timer(lambda: ops.k.linear_pair(x, w, None, y, ops.status))
                print(f"{name + ' (pair)':10s} {T:6d} {N:7d} {K:6d} {ms_pair:9.4f} {ms_lib:9.4f} {2.0 * T * N * K / ms_pair / 1e9:8.1f}")
                rows.append({"op": name + "_pair", "T": T, "N": N, "K": K, "ms": ms_pair, "cublas_ms": ms_lib,
                             "tflops": 2.0 * T * N * K / ms_pair / 1e9})
            flops = 2.0 * T * N * K
            byts = 2.0 * (T * K + N * K + T * N)
            t_c, t_m = flops / (tflops * 1e12), byts / (hbm * 1e9)
            roof = max(t_c, t_m)
            frac = roof / (ms / 1e3)
            rows.append({"op": name, "T": T, "N": N, "K": K, "ms": ms, "cublas_ms": ms_lib,
                         "tflops": flops / ms / 1e9, "gbs": byts / ms / 1e6, "roofline_frac": frac,
                         "bound": "mem" if t_m > t_c else "mma"})
            print(f"{name:10s} {T:6d} {N:7d} {K:6d} {ms:9.4f} {ms_lib:9.4f} {flops / ms / 1e9:8.1f} "
                  f"{byts / ms / 1e6:7.0f} {frac:6.2f} {'mem' if t_m > t_c else 'mma':>5s}")
        del w
    # decode attention at the benchmark's shape
    B, L, bs = 64, 1152, 16
    hq, hkv, D = cfg.num_heads // args.tp, max(cfg.num_kv_heads // args.tp, 1), cfg.head_dim
    nb = B * (L // bs)
    kc = torch.randn(nb, hkv, bs, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.randn_like(kc)
    tables = torch.arange(nb, device="cuda", dtype=torch.int32).view(B, L // bs)
    q = torch.randn(B, hq * D, device="cuda", dtype=torch.bfloat16)
    row_seq = torch.arange(B, device="cuda", dtype=torch.int32)
    pos = torch.full((B,), L - 1, device="cuda", dtype=torch.int32)
    from .models.decoder import StepBatch
    meta = StepBatch(None, pos, None, row_seq, tables, None, num_seqs=B, num_tokens=B, max_kv_len=L, all_decode=True,
                     seq_lens=torch.full((B,), L, device="cuda", dtype=torch.int32),
                     q_starts=torch.arange(B + 1, device="cuda", dtype=torch.int32))
    byts = 2.0 * kc.numel() * 2
    for label, m in (("attn_dec_tc", meta), ("attn_dec_generic", None)):
        ms = timer(lambda: ops.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5, meta=m))
        print(f"{label:18s} {B:4d} ctx={L} {ms:9.4f} ms  {byts / ms / 1e6:7.0f} GB/s  frac {byts / (hbm * 1e9) / (ms / 1e3):.2f}")
        rows.append({"op": label, "B": B, "ctx": L, "ms": ms, "gbs": byts / ms / 1e6})
    kc8, vc8 = kc.to(torch.float8_e4m3fn), vc.to(torch.float8_e4m3fn)
    for label, m in (("attn_dec_tc_e4m3", meta), ("attn_dec_generic_e4m3", None)):
        ms = timer(lambda: ops.attention(q, kc8, vc8, tables, row_seq, pos, hq, hkv, D, D ** -0.5, meta=m))
        print(f"{label:18s} {B:4d} ctx={L} {ms:9.4f} ms  {byts / 2 / ms / 1e6:7.0f} GB/s  frac {byts / 2 / (hbm * 1e9) / (ms / 1e3):.2f}")
        rows.append({"op": label, "B": B, "ctx": L, "ms": ms, "gbs": byts / 2 / ms / 1e6})
    del kc8, vc8
    # prefill attention: one 2048-token chunk of two 1024-token prompts
    Tq = 2048
    qp = torch.randn(Tq, hq * D, device="cuda", dtype=torch.bfloat16)
    metap = StepBatch(None, None, None, None, tables, None, num_seqs=2, num_tokens=Tq, max_kv_len=1024,
                      seq_lens=torch.full((2,), 1024, device="cuda", dtype=torch.int32),
                      q_starts=torch.tensor([0, 1024, 2048], device="cuda", dtype=torch.int32),
                      max_q_len=1024, min_q_len=1024)
    rs = torch.arange(2, device="cuda", dtype=torch.int32).repeat_interleave(1024)
    ps = torch.arange(1024, device="cuda", dtype=torch.int32).repeat(2)
    ms = timer(lambda: ops.attention(qp, kc, vc, tables, rs, ps, hq, hkv, D, D ** -0.5, meta=metap))
    fl = 4.0 * 2 * (1024 * 1025 / 2) * D * hq
    print(f"{'attn_prefill_tc':18s} 2x1024 {ms:9.4f} ms  {fl / ms / 1e9:7.1f} TFLOP/s")
    rows.append({"op": "attention_prefill", "ms": ms, "tflops": fl / ms / 1e9})
    # elementwise
    for T in (64, 2048):
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        d = torch.randn_like(x)
        w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        ms = timer(lambda: ops.rmsnorm(x, d, w, 1e-6))
        print(f"{'add_rms':10s} {T:6d} {ms:9.4f} ms  {4 * 2.0 * T * H / ms / 1e6:7.0f} GB/s")
        gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
        ms = timer(lambda: ops.glu(gu))
        print(f"{'swiglu':10s} {T:6d} {ms:9.4f} ms  {3 * 2.0 * T * I / ms / 1e6:7.0f} GB/s")
    print("kernel status word:", ops.check_status())
    if args.json:
        json.dump({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "rows": rows},
                  open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
