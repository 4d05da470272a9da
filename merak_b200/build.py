"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``_mrk_kernels.so``  every ``csrc/*.cu`` compiled by nvcc for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``); plain C ABI, loaded with ctypes.
* ``_mrk_native.so``   host-only C++ (``csrc/*.cpp``): the AutoPipe partitioner and the
  pipeline-schedule simulator.

nvcc cross-compiles without a GPU, so ``python -m merak_b200.build`` works on a CPU-only
machine.  Objects are cached under ``build/`` and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(os.path.dirname(HERE), "build", "obj")
KERNEL_LIB = os.path.join(HERE, "_mrk_kernels.so")
NATIVE_LIB = os.path.join(HERE, "_mrk_native.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
# Approximate division / exp / flush-to-zero only where the instruction count of an inner loop or
# an epilogue depends on it (tensor-core kernels); norms, cross entropy, AdamW and the reductions
# are memory-bound and keep IEEE division, sqrt and exp.
FAST_MATH_SOURCES = {"gemm_tcgen05.cu", "gemm_tcgen05_pair.cu", "attention_fwd.cu", "attention_bwd.cu"}
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _newest_header_mtime() -> float:
    hdrs = (glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) +
            glob.glob(os.path.join(CSRC, "*.inc")))
    return max([os.path.getmtime(h) for h in hdrs] + [0.0])


def _stale(target: str, sources: list[str], hdr_mtime: float) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources) or hdr_mtime > t


def _run(cmd: list[str], verbose: bool) -> str:
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), res.stdout, res.stderr))
    return res.stdout + res.stderr


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> dict:
    """Builds both libraries if they are out of date. Returns {"kernels": path, "native": path}."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdr_mtime = _newest_header_mtime()
    cu_sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    cpp_sources = sorted(glob.glob(os.path.join(CSRC, "*.cpp")))
    nvcc = _nvcc()
    log = []

    jobs = []
    objs = []
    for src in cu_sources:
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src], hdr_mtime):
            flags = list(NVCC_FLAGS)
            if os.path.basename(src) in FAST_MATH_SOURCES:
                flags.append("--use_fast_math")
            if ptxas_info:
                flags += ["-Xptxas", "-v"]
            jobs.append([nvcc] + flags + ["-I", CSRC, "-c", src, "-o", obj])
    cpp_objs = []
    for src in cpp_sources:
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        cpp_objs.append(obj)
        if force or _stale(obj, [src], hdr_mtime):
            jobs.append(["g++"] + CXX_FLAGS + ["-I", CSRC, "-c", src, "-o", obj])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(lambda c: _run(c, verbose), jobs):
                if out.strip():
                    log.append(out)
    if objs and (force or _stale(KERNEL_LIB, objs, 0.0)):
        _run([nvcc, "-shared", "-o", KERNEL_LIB] + objs + ["-lcudart"], verbose)
    if cpp_objs and (force or _stale(NATIVE_LIB, cpp_objs, 0.0)):
        _run(["g++", "-shared", "-o", NATIVE_LIB] + cpp_objs, verbose)
    if verbose or ptxas_info:
        for entry in log:
            print(entry)
    return {"kernels": KERNEL_LIB, "native": NATIVE_LIB, "log": "\n".join(log)}


if __name__ == "__main__":
    build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
