"""The drop-in boundary on a GPU: this library registered with the reference's own registry, reached through the
reference's public operators, its ``QuantizedTensor`` / ``TensorCoreNVFP4Layout`` and its own tests.

Needs the copy of the reference's Python package that ``baseline/make_ref.py`` puts under ``baseline/_ref/`` (the GPU
box has no reference checkout); skipped when it is absent.  Pattern of every comparison: the reference eager backend
and this backend on the same CUDA tensors (``tests/test_qdq.py:152-190`` of the reference).

Tolerances: quantized bytes, block scales and dequantized values bit-equal to eager; GEMM relative RMS error <= 1e-2
against the eager ``scaled_mm_nvfp4`` (cuBLASLt through torch) on the same quantized operands.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys

import pytest
import torch

from helpers import seeded_randn

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
REL_RMS_TOL = 1e-2

if not os.path.isdir(os.path.join(REF, "comfy_kitchen")):
    pytest.skip("baseline/_ref/comfy_kitchen is absent (python baseline/make_ref.py makes it from a reference checkout)",
                allow_module_level=True)


@pytest.fixture(scope="module")
def env():
    """(ck, ckb, registry) with this backend installed first in the reference registry's priority list."""
    sys.path.insert(0, REF)
    sys.dont_write_bytecode = True
    import comfy_kitchen as ck
    from comfy_kitchen.registry import registry

    import comfy_kitchen_b200 as ckb
    old = list(registry._priority)
    ckb.install()
    yield ck, ckb, registry
    ckb.uninstall()
    registry.set_priority(old)
    registry.enable("sm100")
    sys.path.remove(REF)
    assert ckb.read_device_status() == 0


def rel_rms(y, ref):
    y, ref = y.double(), ref.double()
    return float((y - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt().clamp_min(1e-30))


def layout_scale(x):
    """The per-tensor scale of the reference tests (tests/test_qdq.py:157-159 of the reference)."""
    return (torch.max(torch.abs(x)) / (448.0 * 6.0)).to(torch.float32)


CASES = [("config1_256x1024", 256, 1024, 0), ("flux_activation_4608x3072", 4608, 3072, 3), ("ragged_129x200", 129, 200, 0)]


@pytest.mark.parametrize("name,m,k,outliers", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "fp16"])
def test_public_quantize_dispatches_here_and_equals_eager(env, name, m, k, outliers, dtype):
    ck, ckb, registry = env
    x = seeded_randn((m, k), seed=m + k, dtype=dtype, outlier_cols=outliers).cuda()
    ts = layout_scale(x)
    pad = m % 16 != 0 or k % 16 != 0
    kwargs = dict(x=x, per_tensor_scale=ts, epsilon=0.0, pad_16x=pad, hi_first=True)
    assert registry.get_capable_backend("quantize_nvfp4", kwargs) == "sm100"
    n0 = ckb.launches()
    q, sf = ck.quantize_nvfp4(x, ts, pad_16x=pad)            # the reference's public operator (its custom op)
    assert ckb.launches() == n0 + 1, "ck.quantize_nvfp4 on a CUDA tensor did not reach this library's kernel"
    with ck.use_backend("eager"):
        q_ref, sf_ref = ck.quantize_nvfp4(x, ts, pad_16x=pad)
    assert ckb.launches() == n0 + 1
    assert q.dtype == torch.uint8 and sf.dtype == torch.float8_e4m3fn
    assert torch.equal(q, q_ref), f"{int((q != q_ref).sum())} packed bytes differ from eager"
    assert torch.equal(sf.view(torch.uint8), sf_ref.view(torch.uint8)), "block scales differ from eager"
    # and back: the dequantizer through the same route, bit-equal too
    n1 = ckb.launches()
    d = ck.dequantize_nvfp4(q, ts, sf, output_type=dtype)
    assert ckb.launches() == n1 + 1
    with ck.use_backend("eager"):
        d_ref = ck.dequantize_nvfp4(q_ref, ts, sf_ref, output_type=dtype)
    assert torch.equal(d.view(torch.int16), d_ref.view(torch.int16))


def test_public_quantize_low_nibble_first(env):
    ck, ckb, _ = env
    x = seeded_randn((64, 256), seed=7).cuda() * 4
    ts = layout_scale(x)
    q, sf = ck.quantize_nvfp4(x, ts, hi_first=False)
    with ck.use_backend("eager"):
        q_ref, sf_ref = ck.quantize_nvfp4(x, ts, hi_first=False)
    assert torch.equal(q, q_ref) and torch.equal(sf.view(torch.uint8), sf_ref.view(torch.uint8))


def test_rejected_calls_fall_through_to_eager(env):
    """A call this backend's rules reject (non-contiguous input) is served by the next backend, not raised."""
    ck, ckb, registry = env
    x = seeded_randn((64, 512), seed=3).cuda()[:, ::2]
    assert not x.is_contiguous()
    ts = layout_scale(x)
    kwargs = dict(x=x, per_tensor_scale=ts, epsilon=0.0, pad_16x=False, hi_first=True)
    assert not registry.validate_backend_for_call("sm100", "quantize_nvfp4", kwargs).success
    n0 = ckb.launches()
    q, _ = ck.quantize_nvfp4(x, ts)
    assert ckb.launches() == n0 and tuple(q.shape) == (64, 128)


@pytest.mark.parametrize("shape", [(256, 1024, 1024), (4608, 3072, 3072), (49, 81, 113)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("with_bias", [False, True], ids=["nobias", "bias"])
def test_layout_linear_reaches_this_gemm(env, shape, with_bias):
    """F.linear on two NVFP4 QuantizedTensors (comfy_kitchen/tensor/nvfp4.py:212-260) runs this library's quantizer
    and GEMM and agrees with the eager scaled_mm_nvfp4 on the same quantized operands."""
    ck, ckb, _ = env
    from comfy_kitchen.tensor import QuantizedTensor
    m, k, n = shape
    if with_bias and n % 16:
        pytest.skip("the reference hands the unpadded bias to the padded GEMM: no backend takes that call")
    x = seeded_randn((m, k), seed=m).cuda()
    w = seeded_randn((n, k), seed=n + 1, std=0.02).cuda()
    bias = seeded_randn((1, n), seed=5, std=0.5).reshape(n).cuda() if with_bias else None
    n0 = ckb.launches()
    qt_x = QuantizedTensor.from_float(x, "TensorCoreNVFP4Layout")      # dynamic scale computed by the layout
    qt_w = QuantizedTensor.from_float(w, "TensorCoreNVFP4Layout")
    assert ckb.launches() == n0 + 2
    y = torch.nn.functional.linear(qt_x, qt_w, bias)
    assert ckb.launches() >= n0 + 3, "the layout's linear handler did not reach this library's GEMM"
    assert tuple(y.shape) == (m, n) and y.dtype == torch.bfloat16
    with ck.use_backend("eager"):
        y_ref = torch.nn.functional.linear(qt_x, qt_w, bias)           # cuBLASLt through torch, same operands
    assert rel_rms(y.float(), y_ref.float()) <= REL_RMS_TOL
    # the reference's own check (tests/test_tensor.py:891-909 of the reference): close to the dequantized product
    expected = torch.nn.functional.linear(qt_x.dequantize(), qt_w.dequantize(), bias)
    assert rel_rms(y.float(), expected.float()) <= REL_RMS_TOL


def test_mm_with_transposed_weight(env):
    ck, ckb, _ = env
    from comfy_kitchen.tensor import QuantizedTensor
    a = seeded_randn((32, 64), seed=1).cuda()
    b = seeded_randn((128, 64), seed=2).cuda()
    qa = QuantizedTensor.from_float(a, "TensorCoreNVFP4Layout")
    qb = QuantizedTensor.from_float(b, "TensorCoreNVFP4Layout")
    n0 = ckb.launches()
    y = torch.mm(qa, qb.t())
    assert ckb.launches() > n0
    with ck.use_backend("eager"):
        y_ref = torch.mm(qa, qb.t())
    assert rel_rms(y.float(), y_ref.float()) <= REL_RMS_TOL


def test_cuda_graph_capture_and_replay(env):
    """Quantize -> linear -> GELU -> quantize -> linear captured on a side stream and replayed
    (tests/test_integration.py:85-168 of the reference): replays are bit-identical and follow a changed input."""
    ck, ckb, _ = env
    from comfy_kitchen.tensor import QuantizedTensor
    layout = "TensorCoreNVFP4Layout"
    w1 = QuantizedTensor.from_float(seeded_randn((128, 64), seed=11).cuda(), layout)
    w2 = QuantizedTensor.from_float(seeded_randn((32, 128), seed=12).cuda(), layout)
    s_in = torch.tensor(48.0 / 2688.0, device="cuda")
    s_hid = torch.tensor(96.0 / 2688.0, device="cuda")

    def model(x):
        h = torch.nn.functional.linear(QuantizedTensor.from_float(x, layout, scale=s_in), w1)
        h = torch.nn.functional.gelu(h)
        return torch.nn.functional.linear(QuantizedTensor.from_float(h, layout, scale=s_hid), w2)

    static_in = seeded_randn((16, 64), seed=13).cuda()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        eager_out = model(static_in).clone()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    n0 = ckb.launches()
    with torch.cuda.stream(stream), torch.cuda.graph(graph):
        static_out = model(static_in)
    stream.synchronize()
    assert ckb.launches() - n0 >= 4, "the captured model did not launch this library's kernels"
    outs = []
    for _ in range(3):
        with torch.cuda.stream(stream):
            graph.replay()
        stream.synchronize()
        outs.append(static_out.clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert torch.equal(outs[0], eager_out), "a replay differs from the eager launch on the same input"
    static_in.copy_(seeded_randn((16, 64), seed=14).cuda() * 10)
    with torch.cuda.stream(stream):
        graph.replay()
    stream.synchronize()
    assert not torch.equal(static_out, outs[0])


def _run_reference_tests(extra_args, with_this_backend=True, timeout=900):
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([os.path.join(ROOT, "tests"), REF, ROOT, env.get("PYTHONPATH", "")])
    env["PYTHONDONTWRITEBYTECODE"] = "1"
    cmd = [sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider"]
    if with_this_backend:
        cmd += ["-p", "ref_alias_plugin"]
    return subprocess.run(cmd + extra_args, cwd=REF, env=env, capture_output=True, text=True, timeout=timeout)


COMPILE_TESTS = "tests/test_integration.py::TestQuantizedCompile"


def test_reference_own_nvfp4_tests_pass_on_this_backend():
    """The reference's NVFP4 tests (quantize / dequantize / nibble order / scaled_mm in test_qdq.py, the layout and
    linear tests in test_tensor.py, CUDA graph capture and replay in test_integration.py), unmodified, in a child
    process with this library registered as the reference's "cuda" backend (tests/ref_alias_plugin.py).  The two
    torch.compile tests are compared separately below."""
    res = _run_reference_tests(["tests/test_qdq.py", "tests/test_tensor.py", "tests/test_integration.py", "-k", "nvfp4",
                                "--deselect", COMPILE_TESTS])
    tail = res.stdout[-4000:] + res.stderr[-2000:]
    assert res.returncode == 0, tail
    passed = re.search(r"(\d+) passed", res.stdout)
    assert passed and int(passed.group(1)) >= 50, tail
    launches = re.search(r"CKB_KERNEL_LAUNCHES=(\d+) CKB_DEVICE_STATUS=(\d+)", res.stdout)
    assert launches and int(launches.group(1)) > 50 and int(launches.group(2)) == 0, tail


def test_reference_compile_tests_behave_as_without_this_backend():
    """torch.compile over the reference's QuantizedTensor model (tests/test_integration.py:171-231 of the reference).
    With torch 2.11 dynamo fails inside its own symbolic-shape code while tracing the reference's tensor subclass, before
    any backend is asked for a kernel; so the contract checked here is that each of those tests ends the same way with
    this backend registered as without it (stock registry: Triton / eager) - pass and pass, or the same failure."""
    outcomes = []
    for with_backend in (False, True):
        res = _run_reference_tests([COMPILE_TESTS, "-k", "nvfp4", "-rA"], with_this_backend=with_backend)
        per_test = {name: kind for kind, name in re.findall(r"^(PASSED|FAILED|ERROR) (\S+)", res.stdout, flags=re.M)}
        assert per_test, res.stdout[-3000:] + res.stderr[-1000:]
        outcomes.append(per_test)
    assert outcomes[0] == outcomes[1], f"stock registry: {outcomes[0]}; with this backend: {outcomes[1]}"
