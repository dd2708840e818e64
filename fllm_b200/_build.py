"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``_C.so``    every sm_100a CUDA kernel plus the ``torch.ops.fllm_b200`` bindings
               (``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo``);
* ``_cpu.so``  the CPU reference engine (quantizers, Q4_K x Q8_K dots, paged
               attention, sampler) behind a C ABI used through ``ctypes``.

Objects are cached under ``fllm_b200/build`` keyed by a hash of the source, the
headers and the flags, so an unchanged file is never recompiled. nvcc
cross-compiles without a GPU, so this also serves as the "does it build" check.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
CPU_SRC = ROOT / "csrc_cpu"
BUILD = ROOT / "build"
LIB_CUDA = ROOT / "_C.so"
LIB_CPU = ROOT / "_cpu.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-DFLLM_SM100A=1",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-fopenmp", "-march=native"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"


def _nvcc() -> str:
    cand = os.path.join(_cuda_home(), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def _torch_paths():
    import torch
    from torch.utils.cpp_extension import include_paths

    lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(bool(torch._C._GLIBCXX_USE_CXX11_ABI))
    return include_paths(), lib, abi


def _hash(paths, extra) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(Path(p).read_bytes())
    h.update(repr(extra).encode())
    return h.hexdigest()


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    r = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("build step failed: " + " ".join(map(str, cmd[:3])) + " ...")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)
    return r.stdout + r.stderr


def _compile_many(jobs, verbose):
    """jobs: list of (src, obj, cmd, deps). Returns True if anything was rebuilt."""
    todo = []
    for src, obj, cmd, deps in jobs:
        stamp = Path(str(obj) + ".hash")
        key = _hash([src] + deps, cmd)
        if obj.exists() and stamp.exists() and stamp.read_text() == key:
            continue
        todo.append((obj, cmd, stamp, key))
    if not todo:
        return False
    workers = min(len(todo), max(1, (os.cpu_count() or 4)))
    with cf.ThreadPoolExecutor(workers) as ex:
        futs = {ex.submit(_run, cmd, verbose): (obj, stamp, key) for obj, cmd, stamp, key in todo}
        for f in cf.as_completed(futs):
            obj, stamp, key = futs[f]
            f.result()
            stamp.write_text(key)
    return True


def build_cuda(verbose: bool = False, ptxas_info: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    inc, torch_lib, abi = _torch_paths()
    cuda_inc = os.path.join(_cuda_home(), "include")
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    jobs = []
    objs = []
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_info else [])
    for src in sorted(CSRC.glob("*.cu")):
        obj = BUILD / (src.stem + ".o")
        objs.append(obj)
        jobs.append((src, obj, [_nvcc(), *flags, "-I", CSRC, "-c", src, "-o", obj], headers))
    for src in sorted(CSRC.glob("*.cpp")):
        obj = BUILD / (src.stem + ".cpp.o")
        objs.append(obj)
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
               "-DTORCH_API_INCLUDE_EXTENSION_H", "-I", CSRC, "-I", cuda_inc]
        for i in inc:
            cmd += ["-isystem", i]
        cmd += ["-c", src, "-o", obj]
        jobs.append((src, obj, cmd, headers))
    changed = _compile_many(jobs, verbose)
    if changed or not LIB_CUDA.exists():
        tmp = LIB_CUDA.with_suffix(".so.tmp")
        cmd = [_nvcc(), "-shared", "-o", tmp, *objs, "-L", torch_lib, "-lc10", "-lc10_cuda",
               "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart",
               "-Xlinker", f"-rpath={torch_lib}"]
        _run(cmd, verbose)
        os.replace(tmp, LIB_CUDA)
    return LIB_CUDA


def build_cpu(verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    headers = sorted(CPU_SRC.glob("*.h"))
    jobs, objs = [], []
    for src in sorted(CPU_SRC.glob("*.cpp")):
        obj = BUILD / ("cpu_" + src.stem + ".o")
        objs.append(obj)
        jobs.append((src, obj, ["g++", *CXX_FLAGS, "-I", CPU_SRC, "-c", src, "-o", obj], headers))
    if not objs:
        return LIB_CPU
    changed = _compile_many(jobs, verbose)
    if changed or not LIB_CPU.exists():
        tmp = LIB_CPU.with_suffix(".so.tmp")
        _run(["g++", "-shared", "-fopenmp", "-o", tmp, *objs], verbose)
        os.replace(tmp, LIB_CPU)
    return LIB_CPU


SAN_FLAGS = ["-O1", "-g", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-fopenmp", "-fno-omit-frame-pointer",
             "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"]
LIB_CPU_SAN = BUILD / "_cpu_sanitized.so"


def build_cpu_sanitized(verbose: bool = False) -> Path:
    """The CPU engine and codecs with AddressSanitizer + UndefinedBehaviorSanitizer (a separate library under
    build/, loaded by `python -m fllm_b200 selftest-cpu --sanitize` in a child process with the ASan runtime
    preloaded). Plays the role of the reference's sanitizer builds of its host code."""
    BUILD.mkdir(exist_ok=True)
    headers = sorted(CPU_SRC.glob("*.h"))
    jobs, objs = [], []
    for src in sorted(CPU_SRC.glob("*.cpp")):
        obj = BUILD / ("cpusan_" + src.stem + ".o")
        objs.append(obj)
        jobs.append((src, obj, ["g++", *SAN_FLAGS, "-I", CPU_SRC, "-c", src, "-o", obj], headers))
    changed = _compile_many(jobs, verbose)
    if changed or not LIB_CPU_SAN.exists():
        tmp = LIB_CPU_SAN.with_suffix(".so.tmp")
        _run(["g++", "-shared", "-fopenmp", "-fsanitize=address,undefined", "-o", tmp, *objs], verbose)
        os.replace(tmp, LIB_CPU_SAN)
    return LIB_CPU_SAN


def sanitizer_runtime() -> str:
    """Path of the AddressSanitizer runtime to preload into a Python child process ('' when the compiler has none)."""
    import subprocess
    try:
        p = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True, check=True).stdout.strip()
    except (OSError, subprocess.CalledProcessError):
        return ""
    return os.path.realpath(p) if os.path.sep in p and os.path.exists(p) else ""


def build_all(verbose: bool = False) -> None:
    build_cpu(verbose)
    build_cuda(verbose)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv)
    print("built", LIB_CUDA, LIB_CPU)
