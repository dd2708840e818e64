"""Roofline of the fused tensor-parallel half-layer: row-parallel GEMM -> reduce(-scatter) + residual +
RMSNorm (+ all-gather) -> column-parallel GEMM, against the same half-layer on library collectives.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m fllm_b200.bench_tp [--model qwen3-8b] [--tokens 64,2048]

Times are CUDA events on the launching stream, max over ranks, L2 flushed between iterations. The
roofline of a step is the slowest of: its FLOPs at the measured GEMM peak, its bytes over NVLink at
the measured peer-copy bandwidth (770 GB/s per direction per GPU), and its weight bytes from HBM at
the measured copy bandwidth (the last one is what binds a 64-token step).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3-8b")
    ap.add_argument("--tokens", default="64,2048")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)
    from .bench_kernel import _peaks
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


if __name__ == "__main__":
    main()
