"""Small, self-ending workloads for profiler captures: ``python -m fllm_b200.profile_case <case>``.

Each case launches ONE kernel family a handful of times on inputs larger than L2 but far below a
GB-scale footprint, so a multi-pass capture (``ncu --set full -k regex:<kernel> -c 1``) finishes
in seconds. Cases: gemm_decode (64 tokens x gate_up of an 8B model), gemm_prefill (2048 tokens),
attn_decode (64 sequences at 1152 context), attn_prefill (2 x 1024 tokens), attn_prefill_long (4 x 4096 tokens,
the tcgen05 kernel with two query tiles per CTA), fp8_prefill, gemm_fp4_decode (64 tokens x NVFP4 gate_up), tp_rs_gemm / tp_norm / tp_ag_gemm (fused tensor-parallel kernels, two virtual ranks).
"""
from __future__ import annotations

import sys

import torch


def main(argv=None) -> None:
    argv = argv if argv is not None else sys.argv[1:]
    case = argv[0] if argv else "gemm_decode"
    reps = int(argv[1]) if len(argv) > 1 else 4
    from .ops.native import NativeOps, Fp8BlockLinear, quantize_weight_fp8_block
    ops = NativeOps(torch.device("cuda:0"))
    bf = dict(device="cuda", dtype=torch.bfloat16)
    if case in ("gemm_decode", "gemm_prefill"):
        T = 64 if case == "gemm_decode" else 2048
        x = torch.randn(T, 4096, **bf)
        w = torch.randn(24576, 4096, **bf) * 0.02
        y = torch.empty(T, 24576, **bf)
        fn = lambda: ops.linear(x, w, out=y)
    elif case == "gemm_fp4_decode":
        from .ops.fp4 import Fp4Weight
        x = torch.randn(64, 4096, **bf)
        codes = torch.randint(0, 256, (24576, 2048), device="cuda", dtype=torch.uint8)
        scales = torch.full((24576, 256), 0x38, device="cuda", dtype=torch.uint8)      # e4m3 1.0
        q = Fp4Weight(codes, scales, 0, 0.01)
        y = torch.empty(64, 24576, **bf)
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
    else:
        raise SystemExit(f"unknown case {case}")
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    print(case, "done; kernel status", ops.check_status())


if __name__ == "__main__":
    main()
