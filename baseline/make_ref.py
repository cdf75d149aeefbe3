#!/usr/bin/env python
"""Puts the comparators of the NVFP4 path under ``baseline/_ref/`` (git-ignored; it travels to the GPU box with the
working tree, where no reference checkout exists).

    python baseline/make_ref.py [/path/to/comfy-kitchen checkout]

What it makes, all from an unmodified reference checkout and none of it product source:

* ``_ref/comfy_kitchen/``  the reference's Python package (``*.py`` only: registry, custom ops, eager and Triton
  backends, ``QuantizedTensor`` and the NVFP4 layout).  The GPU tests register this library's backend with that
  registry and compare with its eager backend on the same CUDA tensors; ``bench.py`` times its Triton quantizer.
* ``_ref/tests/``  the reference's own tests of this path (``test_qdq.py``, ``test_tensor.py``,
  ``test_integration.py`` with their ``conftest.py``), which ``tests/test_gpu_registry.py`` runs against this backend.
* ``_ref/libref_quantize_nvfp4.so``  the reference CUDA quantizer (``comfy_kitchen/backends/cuda/ops/quantize_nvfp4.cu``
  with the three headers it includes) compiled by itself for sm_100a with the flags of the reference's CMakeLists
  (``--use_fast_math`` among them); it exports the reference's own ``launch_quantize_nvfp4_kernel``.  ``bench.py`` times it
  beside this library's quantizer and counts the bytes on which it differs from eager.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
# the reference checkout: $COMFY_KITCHEN_REFERENCE, else a directory named "reference" beside this repository
DEFAULT_CHECKOUT = os.environ.get("COMFY_KITCHEN_REFERENCE",
                                  os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
REF_TESTS = ["__init__.py", "conftest.py", "test_qdq.py", "test_tensor.py", "test_integration.py"]


def copy_python_package(checkout: str) -> str:
    src = os.path.join(checkout, "comfy_kitchen")
    dst = os.path.join(DEST, "comfy_kitchen")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    for dirpath, dirnames, files in os.walk(src):
        dirnames[:] = [d for d in dirnames if d != "__pycache__"]
        rel = os.path.relpath(dirpath, src)
        for f in files:
            if f.endswith(".py"):
                os.makedirs(os.path.join(dst, rel), exist_ok=True)
                shutil.copyfile(os.path.join(dirpath, f), os.path.join(dst, rel, f))
    return dst


def copy_reference_tests(checkout: str) -> str:
    dst = os.path.join(DEST, "tests")
    os.makedirs(dst, exist_ok=True)
    for f in REF_TESTS:
        shutil.copyfile(os.path.join(checkout, "tests", f), os.path.join(dst, f))
    return dst


def build_cuda_quantizer(checkout: str) -> str | None:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return None
    cuda_dir = os.path.join(checkout, "comfy_kitchen", "backends", "cuda")
    out = os.path.join(DEST, "libref_quantize_nvfp4.so")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "--use_fast_math",
           "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC", "-shared", "-I", cuda_dir,
           "-o", out, os.path.join(cuda_dir, "ops", "quantize_nvfp4.cu")]
    env = dict(os.environ)
    env.pop("CC", None)
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed on the reference quantizer:\n" + r.stderr)
    return out


def make(checkout: str = DEFAULT_CHECKOUT) -> dict:
    """Returns what was made; an absent checkout leaves an existing ``_ref`` untouched and returns {}."""
    if not os.path.isdir(os.path.join(checkout, "comfy_kitchen")):
        return {}
    os.makedirs(DEST, exist_ok=True)
    return {"package": copy_python_package(checkout), "tests": copy_reference_tests(checkout),
            "cuda_quantizer": build_cuda_quantizer(checkout)}


if __name__ == "__main__":
    made = make(sys.argv[1] if len(sys.argv) > 1 else DEFAULT_CHECKOUT)
    if not made:
        print("no reference checkout found: nothing made")
    for k, v in made.items():
        print(f"{k}: {v}")
