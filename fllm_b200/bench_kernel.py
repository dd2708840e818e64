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


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--tokens", default="1,16,64,128,256,2048,8192")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--json", default="")
    ap.add_argument("--fp4", action="store_true", help="only the packed FP4 (NVFP4 / MXFP4) decode GEMMs")
    args = ap.parse_args(argv)
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
        print(f"# peaks ({src}): {hbm} GB/s; bytes = packed weight + scales + activations")
        for name, (N, K) in shapes.items():
            if name == "lm_head":
                continue
            w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
            for fmt in ("nvfp4", "mxfp4"):
                q = Fp4Weight.from_dense(w, fmt)
                for T in (1, 16, 64, 128):
                    x = torch.randn(T, K, device="cuda", dtype=torch.bfloat16)
                    y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
                    ms = timer(lambda: ops.linear(x, q, out=y))
                    ms16 = timer(lambda: ops.linear(x, w, out=y))
                    byts = q.nbytes() + 2.0 * (T * K + T * N)
                    print(f"{name:8s} {fmt:6s} T={T:4d} N={N:6d} K={K:6d} {ms * 1e3:8.1f} us  (bf16 {ms16 * 1e3:7.1f} us)  "
                          f"{byts / ms / 1e6:6.0f} GB/s  frac {byts / (hbm * 1e9) / (ms / 1e3):.2f}")
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
