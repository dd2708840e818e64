#!/usr/bin/env python
"""Build the reference engine's CUDA kernels, unmodified, into one shared library.

The reference is a Rust workspace, so its engine cannot be installed where no Rust toolchain
exists. Its GPU kernels, however, are plain CUDA sources behind a self-contained C API
(rust/engine/cuda/fllm_cuda.h) that its build script compiles with nvcc
(rust/engine/build.rs:521-660, flags :643-651). This script does the same job for one target
architecture: every source is compiled as it is, straight from the reference tree (nothing is
copied or patched), with the reference's flags, and linked into ``baseline/_ref/libfllmcuda.so``
(objects are kept under ``baseline/_ref_build``). ``fllm_b200.bench_kernel --vs-reference`` then times those
kernels next to ours on the same GPU, through that C API.

    python baseline/build_ref_kernels.py [--ref /path/to/reference] [--arch 100] [--jobs 8] [--no-marlin]

Sources that need headers the reference does not ship (CUTLASS, FlashInfer) are built the way the
reference builds them without those headers: as stubs that decline every call (-DFLLM_NO_HOPPER,
-DFLLM_NO_SM100), so the library holds what an offline build of the reference would hold.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref_build"
LIB_DIR = HERE / "_ref"

# rust/engine/build.rs:521
SOURCES = ["api.cu", "kda.cu", "sampling.cu", "attn_tree.cu", "comm_kernels.cu", "moe.cu", "linear.cu", "gemv2.cu",
           "elementwise.cu", "attention.cu", "attention2.cu", "tc_gemm.cu", "qgemm4k.cu", "attention3.cu", "qgemm6k.cu",
           "qgemm5k.cu", "qgemm8.cu", "qgemm_leg.cu", "attention4.cu", "mmvq.cu", "nvfp4.cu", "flashinfer_prefill.cu",
           "marlin_q4k.cu", "deltanet.cu", "kv_quant.cu", "arch_ops.cu", "dsa.cu", "block_sparse.cu", "inkling.cu", "hc.cu",
           "qwen4.cu", "v4.cu", "mla.cu", "mamba2.cu", "shortconv.cu", "mamba1.cu", "fused.cu", "attn_encoder.cu",
           "act_narrow.cu", "exl.cu", "mlx_affine.cu", "rwkv.cu", "scan.cu"]
# rust/engine/build.rs:405-417 (files that exist in the tree), with the define their flavor gets without its headers
EXTRA = [("nvfp4_cutlass_sm100.cu", ["-DFLLM_NO_SM100"]), ("fp8_gemm.cu", []), ("fp8_block.cu", []),
         ("fp8_cutlass_sm90.cu", ["-DFLLM_NO_HOPPER"]), ("int8_gemm.cu", []), ("cublaslt_gemm.cu", []),
         ("fa3_prefill.cu", ["-DFLLM_NO_HOPPER"]), ("fi_attn.cu", []), ("mla_latent.cu", []), ("mla_decode.cu", [])]
NO_FAST_MATH = {"kv_quant.cu", "sampling.cu"}          # rust/engine/build.rs:545


def nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def compile_one(cmd, obj: Path, key: str):
    stamp = Path(str(obj) + ".key")
    if obj.exists() and stamp.exists() and stamp.read_text() == key:
        return obj, "cached", ""
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        return obj, "failed", (r.stdout + r.stderr)[-3000:]
    stamp.write_text(key)
    return obj, "built", ""


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("FLLM_REFERENCE_DIR", "/root/reference"))
    ap.add_argument("--arch", default="100")
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    ap.add_argument("--no-marlin", action="store_true", help="skip the generated Marlin instances (AWQ / GPTQ / FP8 / FP4 W4A16)")
    args = ap.parse_args()
    cuda_dir = Path(args.ref) / "rust" / "engine" / "cuda"
    if not cuda_dir.is_dir():
        print(f"no reference CUDA sources under {cuda_dir}", file=sys.stderr)
        return 2
    OUT.mkdir(parents=True, exist_ok=True)
    gencode = ["-gencode", f"arch=compute_{args.arch},code=sm_{args.arch}"]
    base = [nvcc(), "-c", "-O3", "--std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]
    jobs = []

    def add(src: Path, obj_name: str, extra):
        obj = OUT / obj_name
        cmd = base + list(extra) + gencode + ["-o", str(obj), str(src)]
        h = hashlib.sha256(src.read_bytes() + repr(cmd).encode()).hexdigest()
        jobs.append((cmd, obj, h))

    for s in SOURCES:
        extra = [] if s in NO_FAST_MATH else ["--use_fast_math"]
        if s == "nvfp4.cu":
            extra.append("-DFLLM_NO_FP4")          # no sm_120a target in this build (rust/engine/build.rs:537-541)
        add(cuda_dir / s, s[:-3] + ".o", extra)
    for s, defs in EXTRA:
        if (cuda_dir / s).exists():
            add(cuda_dir / s, s[:-3] + ".o", ["--use_fast_math", "--expt-relaxed-constexpr"] + defs)
    if not args.no_marlin:
        mdir = cuda_dir / "marlin_vllm"
        for src in sorted(mdir.glob("*.cu")) + [cuda_dir / "marlin_vllm_glue.cu"]:
            add(src, "marlin_" + src.stem + ".o", ["--use_fast_math", "--expt-relaxed-constexpr", f"-I{mdir}"])
    failed = []
    objs = []
    with cf.ThreadPoolExecutor(args.jobs) as ex:
        futs = [ex.submit(compile_one, *j) for j in jobs]
        for f in cf.as_completed(futs):
            obj, state, log = f.result()
            print(f"{state:7s} {obj.name}", flush=True)
            if state == "failed":
                failed.append((obj.name, log))
            else:
                objs.append(str(obj))
    for name, log in failed:
        print(f"---- {name}\n{log}", file=sys.stderr)
    if failed:
        return 1
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    lib = LIB_DIR / "libfllmcuda.so"
    r = subprocess.run([nvcc(), "-shared", "-o", str(lib)] + sorted(objs) + ["-lcudart", "-ldl"], capture_output=True, text=True)
    if r.returncode != 0:
        print(r.stdout + r.stderr, file=sys.stderr)
        return 1
    print("built", lib)
    return 0


if __name__ == "__main__":
    sys.exit(main())
