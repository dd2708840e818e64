"""Kernel-for-kernel comparison with the reference engine's CUDA kernels on the same GPU
(``python -m fllm_b200 bench-kernel --vs-reference``).

The reference's kernels are built unmodified into ``libfllmcuda.so`` by
``baseline/build_ref_kernels.py`` and are called here through their own C API
(rust/engine/cuda/fllm_cuda.h), with the device layouts that API expects: fp32 activations,
row-major 16-bit or packed weights, a slot-major fp16 KV pool ``[slot][kv_heads * head_dim]`` with
64-bit block tables and lengths passed from the host. Our kernels run on the same values. Each pair
is timed with CUDA events on the stream that launches it, after warm-up, L2 flushed between
iterations, median of the iterations; outputs are compared so that a row only counts when both
sides computed the same thing. The one-shot all-reduce kernel of the reference is never called (its
wait is unbounded, rust/engine/cuda/comm_kernels.cu:188-189).

Rows: dense bf16 linear at the model's projection shapes (reference: tensor-core GEMV up to 16
tokens, cuBLASLt above, rust/engine/cuda/linear.cu:396-507, cublaslt_gemm.cu:125-152), add + RMSNorm
(fused.cu:68-192), decode attention (attention4.cu:275-495), prompt attention (attention3.cu:57-288),
Q4_K linear (mmvq.cu:50 for one token, qgemm4k.cu:105-326 above).
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Optional

import torch

KIND_F16, KIND_BF16, KIND_Q4_K = 1, 30, 12


def find_ref_lib(path: Optional[str] = None) -> Optional[str]:
    cands = [path, os.environ.get("FLLM_REF_LIB"),
             os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref", "libfllmcuda.so")]
    for c in cands:
        if c and os.path.exists(c):
            return c
    return None


class RefLib:
    def __init__(self, path: str, device: int = 0):
        self.lib = ctypes.CDLL(path)
        L = self.lib
        L.fllm_cuda_last_error.restype = ctypes.c_char_p
        L.fllm_cuda_stream_create.restype = ctypes.c_void_p
        L.fllm_cuda_stream_create.argtypes = [ctypes.c_int]
        L.fllm_cuda_stream_native.restype = ctypes.c_void_p
        L.fllm_cuda_stream_native.argtypes = [ctypes.c_void_p]
        L.fllm_cuda_stream_sync.argtypes = [ctypes.c_void_p]
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.fllm_cuda_linear.argtypes = [vp, vp, ci, vp, vp, vp, ci, ci, ci]
        L.fllm_cuda_add_rms_norm.argtypes = [vp, vp, vp, cf, vp, vp, ci, ci, cf, ci, ci, vp, ci]
        L.fllm_cuda_rms_norm.argtypes = [vp, vp, vp, vp, ci, ci, cf]
        L.fllm_cuda_attention.argtypes = [vp, vp, vp, vp, vp, vp, ctypes.c_size_t, vp, ci, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci,
                                          ci, ci, cf, cf, ci, ci]
        self.st = L.fllm_cuda_stream_create(device)
        if not self.st:
            raise RuntimeError("reference stream: " + (L.fllm_cuda_last_error() or b"").decode())
        self.stream = torch.cuda.ExternalStream(L.fllm_cuda_stream_native(self.st))

    def check(self, rc: int, what: str):
        if rc != 0:
            raise RuntimeError(f"reference {what} returned {rc}: {(self.lib.fllm_cuda_last_error() or b'').decode()}")

    def linear(self, w, kind, x32, y32, rows, cols, batch):
        self.check(self.lib.fllm_cuda_linear(self.st, w.data_ptr(), kind, x32.data_ptr(), y32.data_ptr(), None, rows, cols, batch), "linear")

    def add_rms_norm(self, x32, branch32, w32, out32, rows, cols, eps):
        return self.lib.fllm_cuda_add_rms_norm(self.st, x32.data_ptr(), branch32.data_ptr(), 1.0, w32.data_ptr(), out32.data_ptr(),
                                               rows, cols, eps, 0, KIND_BF16, None, 0)

    def attention(self, q32, kpool, vpool, out32, tables, lengths, rows, heads, kv_heads, d, stride, block_size, scale):
        self.check(self.lib.fllm_cuda_attention(self.st, q32.data_ptr(), kpool.data_ptr(), vpool.data_ptr(), out32.data_ptr(),
                                                tables.ctypes.data, tables.size, lengths.ctypes.data, rows, None, None, heads, kv_heads,
                                                d, d, stride, block_size, KIND_F16, 0, 0, 0, 0, scale, 0.0, 0, 0), "attention")

    def sync(self):
        self.lib.fllm_cuda_stream_sync(self.st)


class _Timer:
    def __init__(self, flush_mb: int = 256):
        self.flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn, stream=None, iters: int = 10, warmup: int = 3) -> float:
        stream = stream or torch.cuda.current_stream()
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            self.flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            fn()
            e1.record(stream)
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2] * 1e3           # median, microseconds


def _rel_err(a, b) -> float:
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9))


def run(model: str = "qwen3-8b", ref_lib: Optional[str] = None, json_path: str = "", tokens=(16, 64, 2048)) -> int:
    from .config import preset
    from .models.decoder import StepBatch
    from .ops.native import NativeOps
    path = find_ref_lib(ref_lib)
    if path is None:
        print("reference kernel library not found: build it with `python baseline/build_ref_kernels.py` or pass --ref-lib")
        return 2
    cfg = preset(model)
    ops = NativeOps(torch.device("cuda:0"))
    ref = RefLib(path, 0)
    timer = _Timer()
    H, I = cfg.hidden_size, cfg.intermediate_size
    shapes = {"qkv": (cfg.q_size + 2 * cfg.kv_size, H), "o": (H, cfg.q_size), "gate_up": (2 * I, H), "down": (H, I)}
    rows_out = []

    def report(op, shape, ours_us, ref_us, err, note=""):
        ratio = ref_us / ours_us if ours_us > 0 else float("nan")
        rows_out.append({"op": op, "shape": shape, "ours_us": round(ours_us, 1), "reference_us": round(ref_us, 1),
                         "speedup": round(ratio, 2), "rel_err_vs_reference": round(err, 4), "note": note})
        print(f"{op:22s} {shape:26s} ours {ours_us:9.1f} us   reference {ref_us:9.1f} us   x{ratio:5.2f}   err {err:.3g} {note}", flush=True)

    print(f"# reference kernels: {path}")
    # ---- dense bf16 linear
    for name, (N, K) in shapes.items():
        w = (torch.randn(N, K, device="cuda") * 0.02).to(torch.bfloat16)
        for T in tokens:
            x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
            x32 = x.float().contiguous()
            y = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
            y32 = torch.empty(T, N, device="cuda", dtype=torch.float32)
            ours = timer(lambda: ops.linear(x, w, out=y))
            theirs = timer(lambda: ref.linear(w, KIND_BF16, x32, y32, N, K, T), ref.stream)
            report("linear bf16 " + name, f"T={T} N={N} K={K}", ours, theirs, _rel_err(y, y32),
                   "reference: tensor-core GEMV" if T <= 16 else "reference: cuBLASLt")
        del w
    # ---- add + RMSNorm (decode rows)
    for T in (64,):
        xr = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        d = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        nw = torch.ones(H, device="cuda", dtype=torch.bfloat16)
        x32, d32, w32, o32 = xr.float().contiguous(), d.float().contiguous(), nw.float().contiguous(), torch.empty(T, H, device="cuda")
        x_keep = xr.clone()

        def ours_fn():
            xr.copy_(x_keep)                 # the op updates the residual in place: same start every time
            return ops.rmsnorm(xr, d, nw, 1e-6)
        x32_keep = x32.clone()

        def ref_fn():
            x32.copy_(x32_keep)
            return ref.add_rms_norm(x32, d32, w32, o32, T, H, 1e-6)
        rc = ref_fn()
        ref.sync()
        if rc == 0:
            torch.cuda.synchronize()
            y = ours_fn()
            ours = timer(ours_fn)
            with torch.cuda.stream(ref.stream):
                theirs = timer(ref_fn, ref.stream)
            report("add + rmsnorm", f"rows={T} hidden={H}", ours, theirs, _rel_err(y, o32), "both include a copy restoring the residual")
        else:
            print(f"add + rmsnorm: the reference declined the fused call (code {rc})")
    # ---- decode attention: 64 sequences at 1152 tokens of context, GQA
    import numpy as np
    B, L, bs = 64, 1152, 16
    hq, hkv, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    nblk = L // bs
    nb = B * nblk
    kc = torch.randn(nb, hkv, bs, D, device="cuda").to(torch.bfloat16)            # ours: [block][kv head][slot][dim]
    vc = torch.randn(nb, hkv, bs, D, device="cuda").to(torch.bfloat16)
    kref = kc.permute(0, 2, 1, 3).contiguous().to(torch.float16)                  # reference: [block * slot][kv head * dim] fp16
    vref = vc.permute(0, 2, 1, 3).contiguous().to(torch.float16)
    tables = torch.arange(nb, device="cuda", dtype=torch.int32).view(B, nblk)
    q = torch.randn(B, hq * D, device="cuda").to(torch.bfloat16)
    meta = StepBatch(None, None, None, None, tables, None, num_seqs=B, num_tokens=B, max_kv_len=L, all_decode=True,
                     seq_lens=torch.full((B,), L, device="cuda", dtype=torch.int32),
                     q_starts=torch.arange(B + 1, device="cuda", dtype=torch.int32))
    q32, o32 = q.float().contiguous(), torch.empty(B, hq * D, device="cuda")
    tab_h = np.ascontiguousarray(tables.cpu().numpy().astype(np.int64))
    len_h = np.full((B,), L, dtype=np.int64)
    y = ops.attention(q, kc, vc, tables, None, None, hq, hkv, D, D ** -0.5, meta=meta)
    ours = timer(lambda: ops.attention(q, kc, vc, tables, None, None, hq, hkv, D, D ** -0.5, meta=meta))
    theirs = timer(lambda: ref.attention(q32, kref, vref, o32, tab_h, len_h, B, hq, hkv, D, nblk, bs, D ** -0.5), ref.stream)
    report("decode attention", f"B={B} ctx={L} heads={hq}/{hkv}", ours, theirs, _rel_err(y, o32), "reference time includes its table upload")
    # ---- prompt attention: one 2048-token prompt
    Lq = 2048
    nbq = Lq // bs
    tq = torch.arange(nbq, device="cuda", dtype=torch.int32).view(1, nbq)
    qp = torch.randn(Lq, hq * D, device="cuda").to(torch.bfloat16)
    metap = StepBatch(None, None, None, None, tq, None, num_seqs=1, num_tokens=Lq, max_kv_len=Lq,
                      seq_lens=torch.full((1,), Lq, device="cuda", dtype=torch.int32),
                      q_starts=torch.tensor([0, Lq], device="cuda", dtype=torch.int32), max_q_len=Lq, min_q_len=Lq)
    qp32, op32 = qp.float().contiguous(), torch.empty(Lq, hq * D, device="cuda")
    tab_p = np.ascontiguousarray(np.tile(np.arange(nbq, dtype=np.int64), (Lq, 1)))
    len_p = np.arange(1, Lq + 1, dtype=np.int64)
    yp = ops.attention(qp, kc, vc, tq, None, None, hq, hkv, D, D ** -0.5, meta=metap)
    ours = timer(lambda: ops.attention(qp, kc, vc, tq, None, None, hq, hkv, D, D ** -0.5, meta=metap))
    theirs = timer(lambda: ref.attention(qp32, kref, vref, op32, tab_p, len_p, Lq, hq, hkv, D, nbq, bs, D ** -0.5), ref.stream, iters=5)
    report("prompt attention", f"1 x {Lq} heads={hq}/{hkv}", ours, theirs, _rel_err(yp, op32), "causal")
    # ---- Q4_K linear (packed 4-bit K-quant blocks, 144 bytes per 256 weights)
    try:
        from .formats import quant
        from .ops.int4 import Int4Weight
        N, K = shapes["gate_up"]
        wf = (torch.randn(N, K) * 0.02).numpy()
        packed = quant.quantize(wf, quant.Q4_K)
        w_ref = torch.from_numpy(packed).cuda().contiguous()
        w_ours = Int4Weight.from_gguf("Q4_K", packed, N, K, device="cuda")
        for T in (1, 64, 2048):
            x = torch.randn(T, K, device="cuda").to(torch.bfloat16)
            x32 = x.float().contiguous()
            y32 = torch.empty(T, N, device="cuda")
            theirs = timer(lambda: ref.linear(w_ref, KIND_Q4_K, x32, y32, N, K, T), ref.stream)
            if w_ours is not None:
                y = ops.linear(x, w_ours)
                ours = timer(lambda: ops.linear(x, w_ours))
                report("linear Q4_K gate_up", f"T={T} N={N} K={K}", ours, theirs, _rel_err(y, y32))
            else:
                print(f"linear Q4_K gate_up T={T}: reference {theirs:.1f} us (no packed weight constructor on this side)")
    except Exception as e:                                   # a missing codec must not lose the rows above
        print(f"Q4_K rows skipped: {type(e).__name__}: {e}")
    code = ops.check_status()
    print("kernel status word:", code)
    if json_path:
        json.dump({"reference_library": path, "rows": rows_out, "kernel_status": code}, open(json_path, "w"), indent=1)
    return 0
