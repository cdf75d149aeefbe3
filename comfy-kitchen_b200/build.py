"""Builds ``libck_b200.so`` in-tree with nvcc for sm_100a (no other architecture, no fast-math)."""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libck_b200.so")
SOURCES = ["abi.cu", "quantize_nvfp4.cu", "gemm_nvfp4_sm100.cu", "mxfp8.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
    # bit-exact parity with the reference eager backend needs IEEE division, no flush-to-zero, no implicit FMA
    "-prec-div=true", "-prec-sqrt=true", "-ftz=false", "-fmad=false",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libck_b200.so cannot be built")
    return exe


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "ck_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources into ``libck_b200.so`` next to this file; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    objs = []
    build_dir = os.path.join(HERE, "build")
    os.makedirs(build_dir, exist_ok=True)
    env = dict(os.environ)
    env.pop("CC", None)
    def compile_one(src: str):
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        cmd = [_nvcc(), *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        return src, obj, subprocess.run(cmd, capture_output=True, text=True, env=env)

    # the translation units are independent: compile them side by side
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    for src, obj, r in results:
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stderr}")
        if verbose:
            print(r.stderr)
        objs.append(obj)
    # link beside the target and rename: a reader never sees a half-written library
    tmp = os.path.join(build_dir, "libck_b200.so.new")
    cmd = [_nvcc(), "-shared", "-o", tmp, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError(f"linking libck_b200.so failed:\n{r.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
