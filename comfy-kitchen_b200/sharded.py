"""N-sharded (column-parallel) NVFP4 linear over ``torch.distributed``: one process per GPU.

The reference is single-GPU; this is the multi-GPU form of its NVFP4 linear
(``samples/nvfp4_linear.py:39-80``: quantize the activation, ``F.linear`` on two NVFP4 tensors).  Each
rank keeps rows ``[n0, n1)`` of the weight resident as packed e2m1 bytes with its own tiled scale tensor;
the per-tensor weight scale is computed once from the whole weight so that every rank's columns equal the
columns of the unsharded result.  The activation is replicated; every rank quantizes it and multiplies by its
shard.  The bf16 column blocks reach the other ranks in one of two ways: ``fused`` - the GEMM's epilogue stores
each finished tile into every rank's output matrix over NVLink (``PeerGroup`` maps the matrices between the
processes), so there is no collective after the GEMM - or ``gather`` / ``gather_async``, one all-gather through
``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests of the host logic).
"""
from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_rows(n: int, world: int, rank: int, unit: int = 8) -> tuple[int, int]:
    """Rows [n0, n1) of an N-row weight owned by ``rank``: contiguous, in units of 8 rows (the N % 8 rule of
    scaled_mm_nvfp4), sizes differing by at most one unit."""
    if n % unit:
        raise ValueError(f"N = {n} must be a multiple of {unit}")
    u = n // unit
    return (rank * u // world) * unit, ((rank + 1) * u // world) * unit


def scale_offsets(rows: int, kblocks: int, device=None) -> torch.Tensor:
    """Byte offset of logical block scale (r, c) inside the 128x4 tiled scale tensor of a [rows, 16*kblocks] operand
    (``comfy_kitchen/float_utils.py:292-326``), as an int64 [rows, kblocks] tensor."""
    cbg = (kblocks + 3) // 4
    r = torch.arange(rows, device=device, dtype=torch.int64).unsqueeze(1)
    c = torch.arange(kblocks, device=device, dtype=torch.int64).unsqueeze(0)
    return (((r // 128) * cbg + c // 4) * 32 + r % 32) * 16 + (r % 128) // 32 * 4 + c % 4


def untile_scales(sf: torch.Tensor, rows: int, kblocks: int) -> torch.Tensor:
    """Tiled scale tensor (any shape, uint8 or float8_e4m3fn) -> logical uint8 [rows, kblocks]."""
    flat = sf.contiguous().view(torch.uint8).reshape(-1)
    return flat[scale_offsets(rows, kblocks, flat.device)]


def tile_scales(logical: torch.Tensor) -> torch.Tensor:
    """Logical uint8 [rows, kblocks] -> tiled uint8 [roundup(rows,128), roundup(kblocks,4)] with zero padding."""
    rows, kblocks = logical.shape
    rp, cp = (rows + 127) // 128 * 128, (kblocks + 3) // 4 * 4
    out = torch.zeros(rp * cp, dtype=torch.uint8, device=logical.device)
    out[scale_offsets(rows, kblocks, logical.device).reshape(-1)] = logical.reshape(-1)
    return out.view(rp, cp)


class _DeviceBytes:
    """Lets torch view raw device memory (the CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerMemory:
    """``nbytes`` of zeroed device memory on every rank, each rank's block mapped into all the others.
    ``ptrs[r]`` is rank r's block as addressable from this process."""

    def __init__(self, nbytes: int, device: torch.device, group=None, ops=None):
        if ops is None:
            from . import ops as _ops
            ops = _ops
        self.ops, self.device, self.nbytes = ops, torch.device(device), int(nbytes)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.own, handle = ops.peer_alloc(self.nbytes, self.device)
        handles = [handle]
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
        self.ptrs = [self.own if r == self.rank else ops.peer_open(handles[r], self.device) for r in range(self.world)]
        self._closed = False

    def tensor(self, shape, dtype: torch.dtype, offset: int = 0) -> torch.Tensor:
        """A tensor over this rank's own block (no copy)."""
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        assert offset + nbytes <= self.nbytes
        raw = torch.as_tensor(_DeviceBytes(self.own + offset, nbytes), device=self.device)
        return raw.view(dtype).view(*shape)

    def close(self) -> None:
        """Unmap the peers' blocks and free this rank's; collective in spirit: no rank may still be writing."""
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.ops.peer_close(p, self.device)
        if dist.is_initialized() and self.world > 1:
            dist.barrier()
        self.ops.peer_free(self.own, self.device)


class PeerGroup:
    """The ranks of one node as seen by the fused kernels: mapped memory plus a stream-ordered barrier.

    ``map_limit_bytes`` bounds the other ranks' memory that layers bound to this group map into this process.  The
    fused all-gather stores into those mappings, which the GPU translates in 2 MiB pages through a cache of limited
    reach: measured on B200s, 7.7 GiB mapped per rank (4 GPUs) takes the stores at 584 GB/s per rank, 16.8 GiB (8 GPUs)
    at 202 GB/s - five times slower than the NCCL all-gather of the same blocks.  ``ShardedNVFP4Linear.bind`` therefore
    declines (with a warning) what would pass the limit, and such a layer's ``fused`` takes the NCCL form."""

    DEFAULT_MAP_LIMIT_BYTES = 12 << 30

    def __init__(self, device: torch.device, group=None, ops=None, map_limit_bytes: int | None = None):
        self.device, self.group = torch.device(device), group
        self.flags = PeerMemory(256, self.device, group, ops)
        self.ops, self.world, self.rank = self.flags.ops, self.flags.world, self.flags.rank
        self.epoch = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.blocks: list[PeerMemory] = [self.flags]
        self.map_limit_bytes = self.DEFAULT_MAP_LIMIT_BYTES if map_limit_bytes is None else int(map_limit_bytes)
        self.mapped_bytes = 0      # bytes of the other ranks' blocks mapped into this process through this group

    def fits(self, nbytes_per_rank: int) -> bool:
        """Whether blocks of ``nbytes_per_rank`` more on every rank keep this process's peer mappings within the limit
        (the same answer on every rank: it depends on sizes only)."""
        return self.mapped_bytes + (self.world - 1) * int(nbytes_per_rank) <= self.map_limit_bytes

    def alloc(self, nbytes: int) -> PeerMemory:
        m = PeerMemory(nbytes, self.device, self.group, self.ops)
        self.blocks.append(m)
        self.mapped_bytes += (self.world - 1) * int(nbytes)
        return m

    def barrier(self) -> None:
        """Enqueue a barrier of all ranks on the current stream."""
        self.ops.peer_barrier(self.flags.ptrs, self.rank, self.epoch)

    def close(self) -> None:
        for m in reversed(self.blocks):
            m.close()
        self.blocks = []


class ShardedNVFP4Linear:
    """y = x @ W^T + bias with W quantized to NVFP4 and sharded along N.

    ``ops`` is a namespace with ``quantize_nvfp4``, ``scaled_mm_nvfp4`` and ``dynamic_scale_nvfp4`` (this package's
    operators on GPUs; the CPU tests pass a stand-in so that the sharding and gather logic runs under gloo).
    """

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, *, group=None, ops=None,
                 input_scale: torch.Tensor | None = None, weight_scale: torch.Tensor | None = None,
                 world: int | None = None, rank: int | None = None):
        if ops is None:
            from . import ops as _ops
            ops = _ops
        self.ops = ops
        self.group = group
        self._set_ranks(group, world, rank)
        self.out_features, self.in_features = weight.shape
        self.n0, self.n1 = shard_rows(self.out_features, self.world, self.rank)
        # global per-tensor scale, evaluated in the weight's dtype like TensorCoreNVFP4Layout.quantize does
        if weight_scale is None:
            weight_scale = ops.dynamic_scale_nvfp4(weight)
        self.weight_scale = weight_scale.to(torch.float32).reshape(())
        shard = weight[self.n0:self.n1].contiguous()
        pad = shard.shape[0] % 16 != 0 or shard.shape[1] % 16 != 0
        self.qweight, self.weight_block_scale = ops.quantize_nvfp4(shard, self.weight_scale, pad_16x=pad)
        self.local_rows = shard.shape[0]
        # pad_16x may have added rows; the GEMM takes N = local_rows (a multiple of 8) and the scale tensor is
        # padded to 128 rows either way
        self.qweight = self.qweight[: self.local_rows].contiguous()
        self.bias = None if bias is None else bias[self.n0:self.n1].contiguous()
        self.input_scale = input_scale

    def _set_ranks(self, group, world, rank) -> None:
        # world / rank given explicitly: a shard prepared outside a process group (tests, offline conversion)
        if world is not None:
            self.world, self.rank = int(world), int(rank or 0)
        else:
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    @classmethod
    def from_state_dict(cls, state_dict: dict, prefix: str = "", *, group=None, ops=None, world: int | None = None,
                        rank: int | None = None, device=None) -> "ShardedNVFP4Linear":
        """This rank's shard of an already quantized linear in the reference's checkpoint format
        (``samples/nvfp4_linear.py:39-68``: ``weight`` packed uint8 [N, K/2], ``weight_scale`` e4m3 block scales in
        the 128x4 tiled layout as uint8 or float8, possibly flat, ``weight_scale_2`` the fp32 per-tensor scale,
        optional ``input_scale`` and ``bias``).  Rows [n0, n1) of the packed weight are sliced; the block scales are
        per row, so the shard's tiled scale tensor is rebuilt from the rows of the full one (a shard boundary need not
        be a multiple of 128).  Nothing is re-quantized: the shard is bit-identical to quantizing those rows of the
        original weight with the global per-tensor scale."""
        if ops is None:
            from . import ops as _ops
            ops = _ops
        self = cls.__new__(cls)
        self.ops, self.group = ops, group
        self._set_ranks(group, world, rank)
        qweight = state_dict[prefix + "weight"]
        if qweight.dtype != torch.uint8 or qweight.dim() != 2:
            raise TypeError("weight must be the packed uint8 [N, K/2] tensor")
        self.out_features, self.in_features = qweight.shape[0], 2 * qweight.shape[1]
        if self.in_features % 16:
            raise ValueError("in_features must be a multiple of 16")
        self.n0, self.n1 = shard_rows(self.out_features, self.world, self.rank)
        self.local_rows = self.n1 - self.n0
        dev = qweight.device if device is None else torch.device(device)
        kblocks = self.in_features // 16
        logical = untile_scales(state_dict[prefix + "weight_scale"], self.out_features, kblocks)
        self.qweight = qweight[self.n0:self.n1].contiguous().to(dev)
        self.weight_block_scale = tile_scales(logical[self.n0:self.n1].contiguous()).to(dev).view(torch.float8_e4m3fn)
        self.weight_scale = state_dict[prefix + "weight_scale_2"].to(device=dev, dtype=torch.float32).reshape(())
        bias = state_dict.get(prefix + "bias")
        self.bias = None if bias is None else bias[self.n0:self.n1].contiguous().to(dev)
        inp = state_dict.get(prefix + "input_scale")
        self.input_scale = None if inp is None else inp.to(device=dev, dtype=torch.float32).reshape(())
        return self

    def quantize_input(self, x: torch.Tensor):
        """The activation as the GEMM wants it: (packed bytes, tiled block scales, per-tensor scale), rows padded to 16.
        Split from the GEMM so that a caller can put the two on different streams."""
        pad = x.shape[0] % 16 != 0 or x.shape[1] % 16 != 0
        if self.input_scale is None and hasattr(self.ops, "quantize_nvfp4_dynamic"):
            return self.ops.quantize_nvfp4_dynamic(x, pad_16x=pad)     # scale and quantization in one launch
        ts_x = self.input_scale if self.input_scale is not None else self.ops.dynamic_scale_nvfp4(x)
        qx, sfx = self.ops.quantize_nvfp4(x, ts_x, pad_16x=pad)
        return qx, sfx, ts_x

    def local_from_quantized(self, qx: torch.Tensor, sfx: torch.Tensor, ts_x: torch.Tensor, rows: int,
                             out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        y = self.ops.scaled_mm_nvfp4(qx, self.qweight, ts_x, self.weight_scale, sfx, self.weight_block_scale,
                                     bias=self.bias, out_dtype=out_dtype)
        return y[:rows, : self.local_rows]

    def local(self, x: torch.Tensor, one_call: bool = False) -> torch.Tensor:
        """This rank's [M, n1-n0] block of the output.  ``one_call``: through the library's whole-linear entry point
        (same bits; for more than 128 rows and columns the GEMM kernel then quantizes x itself)."""
        if one_call and hasattr(self.ops, "linear_nvfp4") and x.dtype in (torch.float16, torch.bfloat16):
            y = self.ops.linear_nvfp4(x, self.qweight, self.weight_block_scale, self.weight_scale,
                                      input_scale=self.input_scale, bias=self.bias)
            return y[:, : self.local_rows]
        qx, sfx, ts_x = self.quantize_input(x)
        return self.local_from_quantized(qx, sfx, ts_x, x.shape[0],
                                         out_dtype=x.dtype if x.dtype != torch.float32 else torch.bfloat16)

    def bind(self, peers: PeerGroup, m: int, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """Set up the fused path for activations of ``m`` rows: allocates this layer's [m, N] output matrix on every
        rank (mapped everywhere) and returns this rank's, which ``fused`` fills.  Needs equal shards."""
        sizes = {b - a for a, b in (shard_rows(self.out_features, self.world, r) for r in range(self.world))}
        if len(sizes) != 1:
            raise ValueError("the fused all-gather needs equal shards")
        self._out_rows, self._out_dtype = m, dtype
        nbytes = m * self.out_features * 2
        if not peers.fits(nbytes):
            # beyond the reach of the GPU's translation cache for peer memory the stores collapse (PeerGroup): this
            # layer keeps the library collective, and fused() says so once
            import warnings
            warnings.warn(f"ShardedNVFP4Linear.bind: {(peers.mapped_bytes + (peers.world - 1) * nbytes) / 2**30:.1f} GiB of peer "
                          f"mappings would pass the limit of {peers.map_limit_bytes / 2**30:.1f} GiB; this layer uses the "
                          "NCCL all-gather instead of the fused epilogue", RuntimeWarning, stacklevel=2)
            self.peers, self._out_mem, self.out_full = None, None, None
            return None
        self.peers = peers
        self._out_mem = peers.alloc(nbytes)
        self.out_full = self._out_mem.tensor((m, self.out_features), dtype)
        return self.out_full

    def fused_from_quantized(self, qx: torch.Tensor, sfx: torch.Tensor, ts_x: torch.Tensor, rows: int) -> torch.Tensor:
        assert rows == self._out_rows, "bind() fixed the number of rows"
        if getattr(self, "out_full", None) is None:      # bind() declined: the same matrix through the library collective
            return self.gather(self.local_from_quantized(qx, sfx, ts_x, rows))
        self.ops.scaled_mm_nvfp4_all_gather(qx, self.qweight, ts_x, self.weight_scale, sfx, self.weight_block_scale,
                                            self._out_mem.ptrs, self.rank, out_dtype=self._out_dtype, bias=self.bias,
                                            rows=rows)
        return self.out_full

    def fused(self, x: torch.Tensor) -> torch.Tensor:
        """Quantize, multiply by this rank's shard and store the column block into every rank's output matrix from
        the GEMM's epilogue.  Returns this rank's matrix, complete after the next ``peers.barrier()`` on all ranks;
        a barrier must also separate a consumer of the matrix from the next call that overwrites it."""
        qx, sfx, ts_x = self.quantize_input(x)
        return self.fused_from_quantized(qx, sfx, ts_x, x.shape[0])

    def gather_async(self, y_local: torch.Tensor):
        """Start the all-gather of equal column blocks and return ``(work, buffer)``: the collective runs on the
        process group's own stream, so kernels enqueued afterwards overlap it; ``work.wait()`` orders the current
        stream after it.  The buffer is rank-major [G, M, N/G]."""
        m = y_local.shape[0]
        sizes = {b - a for a, b in (shard_rows(self.out_features, self.world, r) for r in range(self.world))}
        if len(sizes) != 1:
            raise ValueError("gather_async needs equal shards")
        y_local = y_local.contiguous()
        flat = torch.empty((self.world * m, y_local.shape[1]), dtype=y_local.dtype, device=y_local.device)
        work = dist.all_gather_into_tensor(flat, y_local, group=self.group, async_op=True)
        return work, flat.view(self.world, m, y_local.shape[1])

    def gather(self, y_local: torch.Tensor, row_major: bool = True) -> torch.Tensor:
        """All-gather the column blocks.  ``row_major=False`` returns the rank-major [G, M, N/G] buffer the
        collective produces (equal shards only) and skips the re-layout pass."""
        if self.world == 1:
            return y_local
        m = y_local.shape[0]
        sizes = [b - a for a, b in (shard_rows(self.out_features, self.world, r) for r in range(self.world))]
        y_local = y_local.contiguous()
        if len(set(sizes)) == 1:
            flat = torch.empty((self.world * m, sizes[0]), dtype=y_local.dtype, device=y_local.device)
            dist.all_gather_into_tensor(flat, y_local, group=self.group)
            buf = flat.view(self.world, m, sizes[0])
            if not row_major:
                return buf
            return buf.permute(1, 0, 2).reshape(m, self.out_features)
        # unequal shards (e.g. 13824 columns over 8 ranks): pad every block to the widest, gather, drop the padding
        widest = max(sizes)
        padded = torch.zeros((m, widest), dtype=y_local.dtype, device=y_local.device)
        padded[:, : y_local.shape[1]] = y_local
        flat = torch.empty((self.world * m, widest), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(flat, padded, group=self.group)
        buf = flat.view(self.world, m, widest)
        return torch.cat([buf[r, :, : sizes[r]] for r in range(self.world)], dim=1)

    def __call__(self, x: torch.Tensor, row_major: bool = True) -> torch.Tensor:
        return self.gather(self.local(x), row_major=row_major)


def replicated_from_seed(shape: tuple[int, int], seed: int, std: float, dtype: torch.dtype, device,
                         transform: Callable[[torch.Tensor], torch.Tensor] | None = None) -> torch.Tensor:
    """Same tensor on every rank: generated on the CPU from a seeded generator, then moved."""
    g = torch.Generator().manual_seed(seed)
    t = torch.randn(shape, generator=g, dtype=torch.float32) * std
    if transform is not None:
        t = transform(t)
    return t.to(dtype).to(device)
