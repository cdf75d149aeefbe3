"""CPU checks of the drop-in boundary: the C-ABI library loads and exports what include/ck_b200.h declares, the
host wrappers mirror the reference operator signatures, and the backend registers with the reference registry."""
from __future__ import annotations

import ctypes
import inspect
import os
import re
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.environ.get("COMFY_KITCHEN_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))


@pytest.fixture(scope="module")
def ckb():
    import comfy_kitchen_b200 as m
    m.build_library()
    return m


def test_library_exports_every_declared_symbol(ckb):
    header = open(os.path.join(ROOT, "include", "ck_b200.h")).read()
    declared = set(re.findall(r"\b(ck_b200_[a-z0-9_]+)\s*\(", header))
    from comfy_kitchen_b200 import _lib
    assert declared == set(_lib.EXPORTED_SYMBOLS), "header and loader disagree on the exported symbols"
    L = ctypes.CDLL(os.path.join(ROOT, "comfy-kitchen_b200", "libck_b200.so"))
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in ck_b200.h but not exported"


def test_host_only_entry_points(ckb):
    """Entry points that need no GPU: error text, tuning switches, ABI version."""
    from comfy_kitchen_b200 import _lib
    L = _lib.load()
    assert L.ck_b200_query(_lib.QUERY_ABI_VERSION) == 2
    assert L.ck_b200_query(12345) == -1
    prev = L.ck_b200_set_tuning(_lib.TUNE_QUANT_VARIANT, 0)
    assert L.ck_b200_set_tuning(_lib.TUNE_QUANT_VARIANT, prev) == 0
    assert L.ck_b200_set_tuning(99, 1) == -1
    assert isinstance(_lib.last_error(), str)


def test_signatures_mirror_reference_operators(ckb):
    want = {
        "quantize_nvfp4": ["x", "per_tensor_scale", "epsilon", "pad_16x", "hi_first"],
        "dequantize_nvfp4": ["qx", "per_tensor_scale", "block_scales", "output_type", "hi_first"],
        "scaled_mm_nvfp4": ["a", "b", "tensor_scale_a", "tensor_scale_b", "block_scale_a", "block_scale_b", "bias",
                            "out_dtype", "alpha"],
    }
    for name, params in want.items():
        sig = inspect.signature(getattr(ckb, name))
        assert list(sig.parameters) == params
    assert inspect.signature(ckb.quantize_nvfp4).parameters["hi_first"].default is True
    assert inspect.signature(ckb.quantize_nvfp4).parameters["pad_16x"].default is False
    assert inspect.signature(ckb.dequantize_nvfp4).parameters["output_type"].default is torch.bfloat16
    if os.path.isdir(REFERENCE):
        sys.path.insert(0, REFERENCE)
        try:
            from comfy_kitchen.backends.eager import quantization as ref
            for name in want:
                assert list(inspect.signature(getattr(ref, name)).parameters) == want[name]
        finally:
            sys.path.remove(REFERENCE)


def test_no_cpu_fallback(ckb):
    x = torch.randn(16, 16, dtype=torch.bfloat16)
    with pytest.raises(TypeError, match="no CPU path"):
        ckb.quantize_nvfp4(x, torch.tensor(0.01))
    with pytest.raises(TypeError):
        ckb.dequantize_nvfp4(torch.zeros(16, 8, dtype=torch.uint8), torch.tensor(0.01),
                             torch.zeros(128, 4, dtype=torch.uint8))
    with pytest.raises(TypeError):
        ckb.scaled_mm_nvfp4(torch.zeros(16, 16, dtype=torch.uint8), torch.zeros(16, 16, dtype=torch.uint8),
                            torch.tensor(1.0), torch.tensor(1.0), torch.zeros(128, 4, dtype=torch.uint8),
                            torch.zeros(128, 4, dtype=torch.uint8))


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "comfy-kitchen_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


@pytest.mark.skipif(not os.path.isdir(REFERENCE), reason="reference checkout not present")
def test_registers_with_reference_registry(ckb):
    sys.path.insert(0, REFERENCE)
    sys.dont_write_bytecode = True
    try:
        import comfy_kitchen as ck
        from comfy_kitchen.registry import registry
        old_priority = list(registry._priority)
        mod = ckb.install()
        try:
            info = ck.list_backends()["sm100"]
            assert info["available"] and not info["disabled"]
            assert info["capabilities"] == ["dequantize_mxfp8", "dequantize_nvfp4", "quantize_mxfp8", "quantize_nvfp4",
                                            "scaled_mm_mxfp8", "scaled_mm_nvfp4"]
            assert registry._priority[0] == "sm100"
            assert registry.get_implementation("quantize_nvfp4", backend="sm100") is mod.quantize_nvfp4
            # CPU tensors: our constraints reject them and the registry falls through to eager
            x = torch.randn(32, 64, dtype=torch.bfloat16)
            kwargs = dict(x=x, per_tensor_scale=torch.tensor(0.01), epsilon=0.0, pad_16x=False, hi_first=True)
            res = registry.validate_backend_for_call("sm100", "quantize_nvfp4", kwargs)
            assert not res.success
            assert registry.get_capable_backend("quantize_nvfp4", kwargs) == "eager"
            q, sf = ck.quantize_nvfp4(x, torch.tensor(0.01))
            assert q.shape == (32, 32) and sf.shape == (128, 4)
            # the layout goes through the registry as well
            from comfy_kitchen.tensor import QuantizedTensor
            qt = QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout")
            assert qt._qdata.shape == (32, 32)
            # constraint rules: non-contiguous input and bad shapes are rejected, not raised
            c = registry.get_constraints("sm100", "scaled_mm_nvfp4")
            assert c.min_compute_capability == (10, 0) and c.default_devices == frozenset({"cuda"})
        finally:
            ckb.uninstall()
            registry.set_priority(old_priority)
            registry.enable("sm100")
    finally:
        sys.path.remove(REFERENCE)
