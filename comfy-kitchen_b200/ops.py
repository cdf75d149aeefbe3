"""Host side of the NVFP4 linear path: the three operators of the reference backend interface.

Names, parameters, defaults, returned shapes and error behaviour mirror the reference CUDA backend
(``comfy_kitchen/backends/cuda/__init__.py:582-667`` and ``:1725-1849``); results are bit-identical to the
reference *eager* backend for quantize/dequantize.  PyTorch is used for allocation, device and stream
handling only; the arithmetic runs in the kernels of ``libck_b200.so``.
"""
from __future__ import annotations

import contextlib
import ctypes

import torch

from . import _lib

DTYPE_TO_CODE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}  # eager/quantization.py:34-42


_WORKSPACES: dict[tuple[int, int], torch.Tensor] = {}
_WORKSPACE_BYTES = 32 << 20   # the reference keeps a 32 MiB cuBLAS workspace per device (backends/cuda/__init__.py:444-462)


def _stream_key(device: torch.device) -> tuple[int, int]:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    return idx, int(torch.cuda.current_stream(device).cuda_stream)


def _workspace(device: torch.device) -> torch.Tensor | None:
    """Scratch for split-K partial sums (problems with M <= 128): one buffer per (device, stream), so that calls on
    different streams never share partial sums, allocated once through torch's caching allocator so that calls stay
    allocation-free afterwards.  Returns None while the stream is being captured and has no buffer yet (nothing is
    allocated inside a capture: the GEMM then runs unsplit); one call on that stream before the capture avoids that."""
    key = _stream_key(device)
    ws = _WORKSPACES.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        ws = torch.empty(_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


_NO_SWITCH = contextlib.nullcontext()


def _on_device(device: torch.device):
    """Device guard for the calls below; free when ``device`` already is the current device (the usual case), where
    torch's guard object would cost several microseconds per operator call."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


def roundup(x: int, multiple: int) -> int:
    return ((x + multiple - 1) // multiple) * multiple


def _plain(t):
    return t.data if isinstance(t, torch.nn.Parameter) else t


def _ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _scale_on(device: torch.device, s: torch.Tensor) -> torch.Tensor:
    s = _plain(s)
    if s.dtype != torch.float32:
        raise TypeError(f"per-tensor scale must be float32, got {s.dtype}")
    if s.numel() != 1:
        raise ValueError("per-tensor scale must have exactly one element")
    if s.device != device:
        s = s.to(device, non_blocking=True)
    return s      # one element: any view of it is contiguous, and only its address is used


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor (comfy_kitchen_b200 has no CPU path), got {t.device}")


def quantize_nvfp4(x: torch.Tensor, per_tensor_scale: torch.Tensor, epsilon: float = 0.0, pad_16x: bool = False,
                   hi_first: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """bf16/fp16/fp32 [R, C] -> (packed e2m1 uint8 [R', C'/2], e4m3 block scales [roundup(R',128), roundup(C'/16,4)]
    in the 128x4 tiled layout).  ``epsilon`` is accepted and unused, as in every reference backend."""
    x = _plain(x)
    _require_cuda(x, "x")
    if x.dim() != 2:
        raise ValueError(f"quantize_nvfp4 needs a 2D tensor, got {x.dim()}D")
    if x.dtype not in DTYPE_TO_CODE:
        raise TypeError(f"quantize_nvfp4: unsupported dtype {x.dtype}")
    assert x.is_contiguous(), "Input tensor must be contiguous"
    orig_rows, orig_cols = x.shape
    if pad_16x:
        num_rows, num_cols = roundup(orig_rows, 16), roundup(orig_cols, 16)
    else:
        num_rows, num_cols = orig_rows, orig_cols
        assert num_rows % 16 == 0, f"num_rows must be divisible by 16, got {num_rows}"
        assert num_cols % 16 == 0, f"num_cols must be divisible by 16, got {num_cols}"
    with _on_device(x.device):
        pts = _scale_on(x.device, per_tensor_scale)
        qx = torch.empty((num_rows, num_cols // 2), device=x.device, dtype=torch.uint8)
        # the kernel writes every byte of the scale tensor, zero padding included: no memset pass
        sx = torch.empty((roundup(num_rows, 128), roundup(num_cols // 16, 4)), device=x.device, dtype=torch.uint8)
        if qx.numel() == 0:
            return qx, sx.view(torch.float8_e4m3fn)
        rc = _lib.load().ck_b200_quantize_nvfp4(_ptr(x), DTYPE_TO_CODE[x.dtype], _ptr(pts), _ptr(qx), _ptr(sx), orig_rows,
                                                orig_cols, int(bool(pad_16x)), int(bool(hi_first)), _stream(x.device))
    _lib.check(rc, "quantize_nvfp4")
    return qx, sx.view(torch.float8_e4m3fn)


_DYN_SYNC: dict[tuple[int, int], torch.Tensor] = {}


def _dynamic_sync(device: torch.device) -> torch.Tensor | None:
    """The 16 zeroed bytes the one-launch dynamic quantizer meets at, one set per (device, stream).  None while the
    stream is being captured and has none yet (the call then takes the separate kernels: same bits)."""
    key = _stream_key(device)
    t = _DYN_SYNC.get(key)
    if t is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        t = torch.zeros(64, dtype=torch.uint8, device=device)
        _DYN_SYNC[key] = t
    return t


def quantize_nvfp4_dynamic(x: torch.Tensor, pad_16x: bool = False, hi_first: bool = True,
                           _sync: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """quantize_nvfp4 with the per-tensor scale ``TensorCoreNVFP4Layout.quantize`` derives when none is given
    (``comfy_kitchen/tensor/nvfp4.py:53-84``: amax(|x|)/(448*6) in x's dtype), without a separate pass over x where x
    fits the L2: returns (packed bytes, tiled block scales, the float32 scale), bit-identical to
    ``dynamic_scale_nvfp4`` followed by ``quantize_nvfp4``."""
    x = _plain(x)
    _require_cuda(x, "x")
    if x.dim() != 2:
        raise ValueError(f"quantize_nvfp4_dynamic needs a 2D tensor, got {x.dim()}D")
    if x.dtype not in DTYPE_TO_CODE:
        raise TypeError(f"quantize_nvfp4_dynamic: unsupported dtype {x.dtype}")
    assert x.is_contiguous(), "Input tensor must be contiguous"
    orig_rows, orig_cols = x.shape
    if pad_16x:
        num_rows, num_cols = roundup(orig_rows, 16), roundup(orig_cols, 16)
    else:
        num_rows, num_cols = orig_rows, orig_cols
        assert num_rows % 16 == 0, f"num_rows must be divisible by 16, got {num_rows}"
        assert num_cols % 16 == 0, f"num_cols must be divisible by 16, got {num_cols}"
    with _on_device(x.device):
        scale = torch.empty((), device=x.device, dtype=torch.float32)
        qx = torch.empty((num_rows, num_cols // 2), device=x.device, dtype=torch.uint8)
        sx = torch.empty((roundup(num_rows, 128), roundup(num_cols // 16, 4)), device=x.device, dtype=torch.uint8)
        sync = _sync if _sync is not None else _dynamic_sync(x.device)
        rc = _lib.load().ck_b200_quantize_nvfp4_dynamic(_ptr(x), DTYPE_TO_CODE[x.dtype], _ptr(scale), _ptr(qx), _ptr(sx),
                                                        orig_rows, orig_cols, int(bool(pad_16x)), int(bool(hi_first)),
                                                        _ptr(sync), _stream(x.device))
    _lib.check(rc, "quantize_nvfp4_dynamic")
    return qx, sx.view(torch.float8_e4m3fn), scale


def dequantize_nvfp4(qx: torch.Tensor, per_tensor_scale: torch.Tensor, block_scales: torch.Tensor,
                     output_type: torch.dtype = torch.bfloat16, hi_first: bool = True) -> torch.Tensor:
    """packed uint8 [R, C/2] + tiled e4m3 scales -> [R, C] in ``output_type``."""
    qx = _plain(qx)
    block_scales = _plain(block_scales)
    _require_cuda(qx, "qx")
    if qx.dim() != 2 or qx.dtype != torch.uint8:
        raise TypeError("dequantize_nvfp4 needs a 2D uint8 tensor")
    if output_type not in DTYPE_TO_CODE:
        raise TypeError(f"dequantize_nvfp4: unsupported output dtype {output_type}")
    assert qx.is_contiguous(), "Input tensor must be contiguous"
    num_rows, packed = qx.shape
    want = (roundup(num_rows, 128), roundup(packed * 2 // 16, 4))
    if block_scales.numel() != want[0] * want[1] or block_scales.element_size() != 1:
        raise ValueError(f"block_scales must hold {want[0]}x{want[1]} one-byte scales, got {tuple(block_scales.shape)}")
    assert block_scales.is_contiguous() and block_scales.device == qx.device
    with _on_device(qx.device):
        pts = _scale_on(qx.device, per_tensor_scale)
        out = torch.empty((num_rows, packed * 2), device=qx.device, dtype=output_type)
        if out.numel() == 0:
            return out
        rc = _lib.load().ck_b200_dequantize_nvfp4(_ptr(qx), _ptr(pts), _ptr(block_scales), _ptr(out),
                                                  DTYPE_TO_CODE[output_type], num_rows, packed, int(bool(hi_first)),
                                                  _stream(qx.device))
    _lib.check(rc, "dequantize_nvfp4")
    return out


def scaled_mm_nvfp4(a: torch.Tensor, b: torch.Tensor, tensor_scale_a: torch.Tensor, tensor_scale_b: torch.Tensor,
                    block_scale_a: torch.Tensor, block_scale_b: torch.Tensor, bias: torch.Tensor | None = None,
                    out_dtype: torch.dtype | None = None, alpha: torch.Tensor | None = None) -> torch.Tensor:
    """[M, K/2] x [N, K/2]^T packed e2m1 with per-16 e4m3 block scales -> [M, N] in ``out_dtype`` (default bf16).
    ``alpha``, when given, replaces tensor_scale_a * tensor_scale_b."""
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    _require_cuda(a, "a")
    if out_dtype is None:
        out_dtype = torch.bfloat16
    if out_dtype not in DTYPE_TO_CODE:
        raise TypeError(f"scaled_mm_nvfp4: unsupported out_dtype {out_dtype}")
    if a.dim() != 2 or b.dim() != 2 or a.dtype != torch.uint8 or b.dtype != torch.uint8:
        raise TypeError("scaled_mm_nvfp4 needs 2D uint8 operands")
    m, k_a = a.shape
    n, k_b = b.shape
    assert k_a == k_b, "Matrix dimensions do not match"
    k = 2 * k_a
    assert a.is_contiguous() and b.is_contiguous(), "operands must be contiguous"
    assert n % 8 == 0, "B tensor must have 8 alignment in N dimension"
    assert block_scale_a.dtype == block_scale_b.dtype, "A and B scale dtype must match"
    if block_scale_a.dtype not in (torch.float8_e4m3fn, torch.uint8):
        raise ValueError(f"Unsupported scale dtype: {block_scale_a.dtype}")
    sk = roundup(k // 16, 4)
    assert block_scale_a.dim() == 2 and tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    assert block_scale_b.dim() == 2 and tuple(block_scale_b.shape) == (roundup(n, 128), sk), "Invalid B scale shape"
    assert block_scale_a.is_contiguous() and block_scale_b.is_contiguous(), "scales must be contiguous"
    for t, nm in ((b, "b"), (block_scale_a, "block_scale_a"), (block_scale_b, "block_scale_b")):
        if t.device != a.device:
            raise TypeError(f"{nm} must be on {a.device}, got {t.device}")
    bias_code = 2
    if bias is not None and bias.numel() > 0:
        bias = _plain(bias)
        assert bias.dtype in (torch.float16, torch.bfloat16), "Only fp16 and bfloat16 bias are supported."
        assert bias.numel() == n and bias.is_contiguous() and bias.device == a.device, "bias must be a contiguous [N] tensor"
        bias_code = DTYPE_TO_CODE[bias.dtype]
    else:
        bias = None
    with _on_device(a.device):
        alpha_t = None
        tsa = tsb = None
        if alpha is not None:
            alpha_t = _plain(alpha)
            if alpha_t.dtype != torch.float32:
                alpha_t = alpha_t.to(torch.float32)
            alpha_t = _scale_on(a.device, alpha_t)
        else:
            tsa = _scale_on(a.device, tensor_scale_a)
            tsb = _scale_on(a.device, tensor_scale_b)
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
        if out.numel() == 0:
            return out
        ws = _workspace(a.device) if m <= 128 else None
        rc = _lib.load().ck_b200_scaled_mm_nvfp4(_ptr(a), _ptr(block_scale_a), _ptr(b), _ptr(block_scale_b), _ptr(tsa),
                                                 _ptr(tsb), _ptr(alpha_t), _ptr(bias), bias_code, _ptr(out),
                                                 DTYPE_TO_CODE[out_dtype], m, n, k, _ptr(ws),
                                                 0 if ws is None else ws.numel(), _stream(a.device))
    _lib.check(rc, "scaled_mm_nvfp4")
    return out


def scaled_mm_nvfp4_all_gather(a: torch.Tensor, b: torch.Tensor, tensor_scale_a: torch.Tensor,
                               tensor_scale_b: torch.Tensor, block_scale_a: torch.Tensor, block_scale_b: torch.Tensor,
                               out_ptrs: list[int], rank: int, out_dtype: torch.dtype = torch.bfloat16,
                               bias: torch.Tensor | None = None, rows: int | None = None) -> None:
    """scaled_mm_nvfp4 of this rank's weight shard ``b`` [N_local, K/2], written into columns
    [rank*N_local, (rank+1)*N_local) of every rank's [M, world*N_local] matrix (``out_ptrs``: device addresses by rank,
    peers' matrices as mapped by ``peer_open``).  Returns nothing: the matrices are complete after the next
    ``peer_barrier`` on every rank.  ``rows``: number of rows of ``a`` to use (the output matrices have that many)."""
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    _require_cuda(a, "a")
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("scaled_mm_nvfp4_all_gather writes float16 or bfloat16")
    m, k_half = a.shape
    n_local = b.shape[0]
    assert b.shape[1] == k_half and a.is_contiguous() and b.is_contiguous()
    sk = roundup(2 * k_half // 16, 4)
    assert tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    if rows is not None:     # `a` was padded to 16 rows by the quantizer: only the first `rows` are multiplied and stored
        assert 0 < rows <= m and roundup(rows, 128) == roundup(m, 128)
        m = rows
    assert tuple(block_scale_b.shape) == (roundup(n_local, 128), sk), "Invalid B scale shape"
    bias_code = 2
    if bias is not None:
        bias = _plain(bias)
        assert bias.numel() == n_local and bias.is_contiguous() and bias.dtype in (torch.float16, torch.bfloat16)
        bias_code = DTYPE_TO_CODE[bias.dtype]
    world = len(out_ptrs)
    arr = (ctypes.c_void_p * world)(*out_ptrs)
    with _on_device(a.device):
        tsa = _scale_on(a.device, tensor_scale_a)
        tsb = _scale_on(a.device, tensor_scale_b)
        rc = _lib.load().ck_b200_scaled_mm_nvfp4_all_gather(_ptr(a), _ptr(block_scale_a), _ptr(b), _ptr(block_scale_b),
                                                            _ptr(tsa), _ptr(tsb), None, _ptr(bias), bias_code, arr, world,
                                                            rank, DTYPE_TO_CODE[out_dtype], m, n_local, 2 * k_half,
                                                            _stream(a.device))
    _lib.check(rc, "scaled_mm_nvfp4_all_gather")


def peer_barrier(flag_ptrs: list[int], rank: int, epoch: torch.Tensor) -> None:
    """Enqueue a barrier between the ranks of the node on the current stream (``flag_ptrs``: every rank's flag array
    as mapped here; ``epoch``: this rank's zero-initialised int32 counter)."""
    world = len(flag_ptrs)
    arr = (ctypes.c_void_p * world)(*flag_ptrs)
    with _on_device(epoch.device):
        rc = _lib.load().ck_b200_peer_barrier(arr, world, rank, _ptr(epoch), _stream(epoch.device))
    _lib.check(rc, "peer_barrier")


def peer_alloc(nbytes: int, device: torch.device) -> tuple[int, bytes]:
    """Zeroed device memory other processes of the node can map: (address, 64-byte handle)."""
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    with _on_device(device):
        _lib.check(_lib.load().ck_b200_peer_alloc(nbytes, ctypes.byref(ptr), handle), "peer_alloc")
    return int(ptr.value), handle.raw


def peer_open(handle: bytes, device: torch.device) -> int:
    ptr = ctypes.c_void_p()
    with _on_device(device):
        _lib.check(_lib.load().ck_b200_peer_open(ctypes.create_string_buffer(handle, 64), ctypes.byref(ptr)), "peer_open")
    return int(ptr.value)


def peer_close(ptr: int, device: torch.device) -> None:
    with _on_device(device):
        _lib.check(_lib.load().ck_b200_peer_close(ptr), "peer_close")


def peer_free(ptr: int, device: torch.device) -> None:
    with _on_device(device):
        _lib.check(_lib.load().ck_b200_peer_free(ptr), "peer_free")


# ---- MXFP8: same interface as the reference operators (comfy_kitchen/backends/cuda/__init__.py:1689-1722,
# comfy_kitchen/backends/eager/quantization.py:319-405) ----------------------------------------------------------

def quantize_mxfp8(x: torch.Tensor, pad_32x: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
    """x [M, K] -> (float8_e4m3fn [Mp, Kp], float8_e8m0fnu block scales [roundup(Mp,128), roundup(Kp/32,4)] tiled)."""
    x = _plain(x)
    _require_cuda(x, "x")
    if x.dim() != 2 or x.dtype not in DTYPE_TO_CODE:
        raise TypeError("quantize_mxfp8 needs a 2D float32/float16/bfloat16 tensor")
    assert x.is_contiguous(), "Input tensor must be contiguous"
    rows, cols = x.shape
    if pad_32x:
        prow, pcol = roundup(rows, 32), roundup(cols, 32)
    else:
        prow, pcol = rows, cols
        assert rows % 32 == 0, f"num_rows must be divisible by 32, got {rows}"
        assert cols % 32 == 0, f"num_cols must be divisible by 32, got {cols}"
    with _on_device(x.device):
        q = torch.empty((prow, pcol), dtype=torch.uint8, device=x.device)
        sf = torch.empty((roundup(prow, 128), roundup(pcol // 32, 4)), dtype=torch.uint8, device=x.device)
        rc = _lib.load().ck_b200_quantize_mxfp8(_ptr(x), DTYPE_TO_CODE[x.dtype], _ptr(q), _ptr(sf), rows, cols,
                                                int(pad_32x), _stream(x.device))
    _lib.check(rc, "quantize_mxfp8")
    return q.view(torch.float8_e4m3fn), sf.view(torch.float8_e8m0fnu)


def dequantize_mxfp8(qx: torch.Tensor, block_scales: torch.Tensor, output_type: torch.dtype = torch.bfloat16) -> torch.Tensor:
    qx, block_scales = _plain(qx), _plain(block_scales)
    _require_cuda(qx, "qx")
    if output_type not in DTYPE_TO_CODE:
        raise TypeError(f"dequantize_mxfp8: unsupported output type {output_type}")
    assert qx.dim() == 2 and qx.is_contiguous() and block_scales.is_contiguous()
    rows, cols = qx.shape
    assert tuple(block_scales.shape) == (roundup(rows, 128), roundup(cols // 32, 4)), "Invalid scale shape"
    with _on_device(qx.device):
        out = torch.empty((rows, cols), dtype=output_type, device=qx.device)
        rc = _lib.load().ck_b200_dequantize_mxfp8(_ptr(qx), _ptr(block_scales), _ptr(out), DTYPE_TO_CODE[output_type],
                                                  rows, cols, _stream(qx.device))
    _lib.check(rc, "dequantize_mxfp8")
    return out


def scaled_mm_mxfp8(a: torch.Tensor, b: torch.Tensor, block_scale_a: torch.Tensor, block_scale_b: torch.Tensor,
                    bias: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """[M, K] x [N, K]^T e4m3 with e8m0 scales per 32 elements -> [M, N] in ``out_dtype`` (default bf16)."""
    a, b = _plain(a), _plain(b)
    block_scale_a, block_scale_b = _plain(block_scale_a), _plain(block_scale_b)
    _require_cuda(a, "a")
    if out_dtype is None:
        out_dtype = torch.bfloat16
    if out_dtype not in DTYPE_TO_CODE:
        raise TypeError(f"scaled_mm_mxfp8: unsupported out_dtype {out_dtype}")
    assert a.dim() == 2 and b.dim() == 2 and a.shape[1] == b.shape[1], "Matrix dimensions do not match"
    assert a.element_size() == 1 and b.element_size() == 1 and a.is_contiguous() and b.is_contiguous()
    m, k = a.shape
    n = b.shape[0]
    assert k % 32 == 0 and n % 8 == 0, "K must be a multiple of 32 and N of 8"
    sk = roundup(k // 32, 4)
    assert tuple(block_scale_a.shape) == (roundup(m, 128), sk), "Invalid A scale shape"
    assert tuple(block_scale_b.shape) == (roundup(n, 128), sk), "Invalid B scale shape"
    bias_code = 2
    if bias is not None and bias.numel() > 0:
        bias = _plain(bias)
        assert bias.numel() == n and bias.is_contiguous() and bias.dtype in (torch.float16, torch.bfloat16)
        bias_code = DTYPE_TO_CODE[bias.dtype]
    else:
        bias = None
    with _on_device(a.device):
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
        if out.numel() == 0:
            return out
        ws = _workspace(a.device) if m <= 128 else None
        rc = _lib.load().ck_b200_scaled_mm_mxfp8(_ptr(a), _ptr(block_scale_a), _ptr(b), _ptr(block_scale_b), _ptr(bias),
                                                 bias_code, _ptr(out), DTYPE_TO_CODE[out_dtype], m, n, k, _ptr(ws),
                                                 0 if ws is None else ws.numel(), _stream(a.device))
    _lib.check(rc, "scaled_mm_mxfp8")
    return out


_LINEAR_WS: dict[tuple[int, int], torch.Tensor] = {}
_LINEAR_NEED: dict[tuple[int, int], int] = {}     # workspace bytes by (M, K)


def linear_nvfp4(x: torch.Tensor, qweight: torch.Tensor, weight_block_scale: torch.Tensor, weight_scale: torch.Tensor,
                 input_scale: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """y[M, N] = x[M, K] @ W^T + bias with W resident in NVFP4: the activation scale (``input_scale`` or the layout's
    dynamic one), the quantization of x and the GEMM are enqueued by one library call, with the quantized activation
    in a per-device workspace that grows on demand.  Same arithmetic as dynamic_scale_nvfp4 -> quantize_nvfp4(pad_16x)
    -> scaled_mm_nvfp4, so results are bit-identical to calling those three.  The workspace (quantized activation,
    its scales, split-K partial sums) is kept per (device, stream): calls on one stream are ordered, calls on different
    streams use different buffers.  It cannot grow while the stream is being captured: call once with the largest
    shape before capturing."""
    x = _plain(x)
    _require_cuda(x, "x")
    if x.dim() != 2 or x.dtype not in DTYPE_TO_CODE:
        raise TypeError("linear_nvfp4 needs a 2D float32/float16/bfloat16 activation")
    assert x.is_contiguous(), "Input tensor must be contiguous"
    qweight, weight_block_scale = _plain(qweight), _plain(weight_block_scale)
    m, k = x.shape
    n = qweight.shape[0]
    assert qweight.dtype == torch.uint8 and qweight.shape[1] * 2 == k and qweight.is_contiguous()
    assert tuple(weight_block_scale.shape) == (roundup(n, 128), roundup(k // 16, 4)), "Invalid weight scale shape"
    if out_dtype is None:
        out_dtype = x.dtype if x.dtype in (torch.float16, torch.bfloat16) else torch.bfloat16
    bias_code = 2
    if bias is not None:
        bias = _plain(bias)
        assert bias.numel() == n and bias.is_contiguous() and bias.dtype in (torch.float16, torch.bfloat16)
        bias_code = DTYPE_TO_CODE[bias.dtype]
    L = _lib.load()
    need = _LINEAR_NEED.get((m, k))
    if need is None:
        need = L.ck_b200_linear_nvfp4_workspace_bytes(m, k)
        if need < 0:
            raise RuntimeError(f"linear_nvfp4: K = {k} must be a multiple of 32")
        need += _WORKSPACE_BYTES if m <= 128 else 0
        if len(_LINEAR_NEED) < 4096:
            _LINEAR_NEED[(m, k)] = need
    dev_index = x.device.index if x.device.index is not None else torch.cuda.current_device()
    stream = int(torch.cuda.current_stream(x.device).cuda_stream)
    key = (dev_index, stream)
    ws = _LINEAR_WS.get(key)
    with _on_device(x.device):
        if ws is None or ws.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("linear_nvfp4: the workspace of this stream must grow, which cannot happen inside a "
                                   "stream capture; call once with this shape on this stream before capturing")
            old = ws
            ws = torch.empty(max(need, 64 << 20), dtype=torch.uint8, device=x.device)
            ws[: 1 << 16].zero_()      # the fused kernel's progress words start from zero
            _LINEAR_WS[key] = ws
            if old is not None:
                old.record_stream(torch.cuda.current_stream(x.device))   # earlier calls on this stream may still read it
        w_ts = _scale_on(x.device, weight_scale)
        in_ts = None if input_scale is None else _scale_on(x.device, input_scale)
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
        rc = L.ck_b200_linear_nvfp4(_ptr(x), DTYPE_TO_CODE[x.dtype], m, k, _ptr(in_ts), _ptr(qweight),
                                    _ptr(weight_block_scale), _ptr(w_ts), n, _ptr(bias), bias_code, _ptr(out),
                                    DTYPE_TO_CODE[out_dtype], _ptr(ws), ws.numel(), ctypes.c_void_p(stream))
    if rc:
        _lib.check(rc, "linear_nvfp4")
    return out


def dynamic_scale_nvfp4(x: torch.Tensor) -> torch.Tensor:
    """amax(|x|)/(448*6) evaluated in x's dtype and returned as a float32 scalar tensor on x's device: the
    per-tensor scale ``TensorCoreNVFP4Layout.quantize`` computes when none is given
    (``comfy_kitchen/tensor/nvfp4.py:66-71``), without the host round trip."""
    x = _plain(x)
    _require_cuda(x, "x")
    if x.dtype not in DTYPE_TO_CODE:
        raise TypeError(f"dynamic_scale_nvfp4: unsupported dtype {x.dtype}")
    assert x.is_contiguous(), "Input tensor must be contiguous"
    with _on_device(x.device):
        out = torch.empty((), device=x.device, dtype=torch.float32)
        rc = _lib.load().ck_b200_dynamic_scale_nvfp4(_ptr(x), DTYPE_TO_CODE[x.dtype], x.numel(), _ptr(out),
                                                     _stream(x.device))
    _lib.check(rc, "dynamic_scale_nvfp4")
    return out


def set_tuning(key: int, value: int) -> int:
    return int(_lib.load().ck_b200_set_tuning(key, value))


def promise_resident_weights(resident: bool = True) -> bool:
    """The caller's promise that, whenever a GEMM with M <= 128 is enqueued, nothing still in flight on the GPU writes
    its weight operand or weight scales (weights quantized when the model was loaded and synchronised since).  The GEMM
    then asks for the first stages of its weight before it waits for the preceding kernel of the stream, so a stack of
    small-M layers streams the next layer's weight under the current layer's tail.  Everything a preceding kernel may
    have produced (activations, their scales, tensor scales, bias) and every store still waits.  Returns the previous
    setting; off by default."""
    return bool(set_tuning(_lib.TUNE_WEIGHTS_RESIDENT, 1 if resident else 0))


def launches() -> int:
    """Kernels this library has launched in this process."""
    return int(_lib.load().ck_b200_query(_lib.QUERY_LAUNCHES))


def read_gemm_counters() -> dict:
    """Cycle counters of the most recent launch of the counting GEMM build (``set_tuning(2, 1)``), CTA pair 0."""
    buf = (ctypes.c_longlong * 5)()
    _lib.check(_lib.load().ck_b200_read_gemm_counters(buf), "read_gemm_counters")
    cyc, ns, wait_full, wait_acc, mma = (int(v) for v in buf)
    return {"epilogue_cycles": cyc, "epilogue_ns": ns, "sm_clock_mhz": (cyc / ns * 1e3) if ns > 0 else None,
            "mma_cycles": mma, "mma_wait_loaded_stages_frac": (wait_full / mma) if mma > 0 else None,
            "mma_wait_accumulator_frac": (wait_acc / mma) if mma > 0 else None}


def read_device_status() -> int:
    """Synchronises and returns the device status word (0 = no bounded wait ran out), clearing it."""
    v = ctypes.c_int(0)
    rc = _lib.load().ck_b200_read_device_status(ctypes.byref(v))
    if rc not in (0, 4):      # 4 = CK_B200_ERR_DEVICE_STATUS: the word itself says which wait ran out
        _lib.check(rc, "read_device_status")
    if v.value != 0:
        # a kernel that gave up on a wait may have left its counters (the dynamic quantizer's meeting point, the
        # in-GEMM quantizer's progress words) part-way: the device is idle now (the call above synchronised), so
        # put them back to zero for the calls that follow
        for t in _DYN_SYNC.values():
            t.zero_()
        for ws in _LINEAR_WS.values():
            ws[: 1 << 16].zero_()
    return int(v.value)
