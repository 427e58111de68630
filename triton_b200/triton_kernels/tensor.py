"""Routing data structures: ``Bitmatrix``, ``BitmatrixMetadata``, ``RaggedTensorMetadata``,
``SparseMatrix`` and their builders. Counterparts of ``triton_kernels/tensor.py:203-210``,
``tensor_details/bitmatrix.py:8-25,110-150`` and ``tensor_details/ragged_tensor.py:12-94,183-210``
in the reference; field names and dtypes are the reference's (all index tensors int32)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import _lib


@dataclass
class Bitmatrix:
    """(rows x cols) bit mask packed into 32-bit words; ``data[r, w]`` holds columns 32w..32w+31
    of row r. The reference stores it transposed in memory (``data.stride(0) == 1``)."""
    data: torch.Tensor
    shape: list
    shape_max: list | None = None

    @property
    def device(self):
        return self.data.device


@dataclass
class BitmatrixMetadata:
    col_sum: torch.Tensor          # entries per column (tokens per expert)
    col_sorted_indx: torch.Tensor  # row-major entry ids grouped by column ("combine" order)
    row_sorted_indx: torch.Tensor  # position of each row-major entry in column order ("dispatch")


def make_bitmatrix_metadata(nonzero_indx: torch.Tensor, bitmatrix: Bitmatrix) -> BitmatrixMetadata:
    assert nonzero_indx.ndim == 2
    assert nonzero_indx.dtype in (torch.int16, torch.int32)
    nonzero_indx = nonzero_indx.contiguous()
    dev = nonzero_indx.device
    n = nonzero_indx.numel()
    n_cols = int(bitmatrix.shape[1])
    col_sum = torch.empty(n_cols, dtype=torch.int32, device=dev)
    combined = torch.empty(2 * n, dtype=torch.int32, device=dev)
    col_sorted, row_sorted = combined[:n], combined[n:]
    l = _lib.lib()
    need = l.tb200_bitmatrix_metadata_workspace_bytes(n, n_cols)
    ws = torch.empty(max(need, 4), dtype=torch.uint8, device=dev)
    args = _lib.BitmatrixMetadataArgs()
    args.indx = nonzero_indx.data_ptr()
    args.col_sum, args.col_sorted_indx, args.row_sorted_indx = col_sum.data_ptr(), col_sorted.data_ptr(), row_sorted.data_ptr()
    args.workspace, args.workspace_bytes = ws.data_ptr(), need
    args.n_entries, args.n_cols = n, n_cols
    args.indx_is_int16 = 1 if nonzero_indx.dtype == torch.int16 else 0
    with _lib.device_guard(dev):
        rc = l.tb200_bitmatrix_metadata(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
    _lib.check(rc, "tb200_bitmatrix_metadata")
    return BitmatrixMetadata(col_sum=col_sum, col_sorted_indx=col_sorted, row_sorted_indx=row_sorted)


@dataclass
class RaggedTensorMetadata:
    slice_sizes: torch.Tensor
    slice_offs: torch.Tensor
    block_offs_data: torch.Tensor
    block_schedule_data: torch.Tensor
    expected_slice_size: int | None = None
    slice_sizes_divisibility: int = None

    def __post_init__(self):
        assert self.block_offs_data.shape[0] == len(RaggedTensorMetadata.block_sizes())
        assert self.block_schedule_data.shape[0] == len(RaggedTensorMetadata.block_sizes())
        assert self.block_offs_data.dtype == torch.int32
        assert self.block_schedule_data.dtype == torch.int32
        if self.slice_sizes is not None:
            assert self.slice_sizes.dtype == torch.int32
        if self.slice_offs is not None:
            assert self.slice_offs.dtype == torch.int32

    @property
    def n_slices(self):
        return self.slice_sizes.shape[0]

    def block_offs(self, block_size):
        return self.block_offs_data[RaggedTensorMetadata.block_sizes().index(block_size)]

    def block_schedule(self, block_size):
        return self.block_schedule_data[RaggedTensorMetadata.block_sizes().index(block_size)]

    @staticmethod
    def n_blocks(n_slices, n_total_rows, block_size):
        if n_total_rows <= n_slices:
            return n_total_rows
        return n_slices - 1 - ((n_slices - n_total_rows - 1) // block_size)

    @staticmethod
    def max_n_blocks(n_slices, n_total_rows):
        return RaggedTensorMetadata.n_blocks(n_slices, n_total_rows, min(RaggedTensorMetadata.block_sizes()))

    @staticmethod
    def block_sizes_log2():
        return range(4, 8)

    @staticmethod
    def block_sizes():
        return [2**x for x in RaggedTensorMetadata.block_sizes_log2()]


def make_ragged_tensor_metadata(slice_sizes: torch.Tensor, n_total_rows: int) -> RaggedTensorMetadata:
    assert slice_sizes.ndim == 1
    slice_sizes = slice_sizes.to(torch.int32).contiguous()
    dev = slice_sizes.device
    n_slices = slice_sizes.shape[0]
    nbs = len(RaggedTensorMetadata.block_sizes())
    max_n_blocks = RaggedTensorMetadata.max_n_blocks(n_slices, n_total_rows)
    slice_offs = torch.empty(n_slices + 1, dtype=torch.int32, device=dev)
    block_offs = torch.empty((nbs, n_slices + 1), dtype=torch.int32, device=dev)
    block_schedule = torch.empty((nbs, max_n_blocks), dtype=torch.int32, device=dev)
    args = _lib.RaggedMetadataArgs()
    args.slice_sizes, args.slice_offs = slice_sizes.data_ptr(), slice_offs.data_ptr()
    args.block_offs, args.block_schedule = block_offs.data_ptr(), block_schedule.data_ptr()
    args.n_slices, args.max_n_blocks = n_slices, max_n_blocks
    with _lib.device_guard(dev):
        rc = _lib.lib().tb200_ragged_metadata(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
    _lib.check(rc, "tb200_ragged_metadata")
    return RaggedTensorMetadata(slice_sizes, slice_offs, block_offs, block_schedule)


def remap_ragged_tensor_metadata(md: RaggedTensorMetadata, slice_map: torch.Tensor) -> RaggedTensorMetadata:
    """Metadata of the ragged tensor that keeps slice i iff ``slice_map[i] != -1`` (renumbered to
    ``slice_map[i]``); dropped entries are compacted to the end as -1
    (``tensor_details/ragged_tensor.py:348-381``). One kernel, no host synchronisation
    (``tb200_remap_ragged_metadata``)."""
    assert slice_map.ndim == 1 and slice_map.shape[0] == md.slice_sizes.shape[0]
    dev = md.slice_sizes.device
    if not md.slice_sizes.is_cuda:
        raise RuntimeError("triton_b200 remap_ragged_tensor_metadata needs CUDA tensors (there is no CPU path)")
    sm = slice_map.to(torch.int32).contiguous()
    n_slices = md.slice_sizes.shape[0]
    bo, bs = md.block_offs_data.contiguous(), md.block_schedule_data.contiguous()
    ss, so = md.slice_sizes.contiguous(), md.slice_offs.contiguous()
    o_ss, o_so = torch.empty_like(ss), torch.empty_like(so)
    o_bo, o_bs = torch.empty_like(bo), torch.empty_like(bs)
    args = _lib.RemapRaggedMetadataArgs()
    args.slice_sizes, args.slice_offs, args.block_offs, args.block_schedule = (ss.data_ptr(), so.data_ptr(), bo.data_ptr(),
                                                                               bs.data_ptr())
    args.slice_map = sm.data_ptr()
    args.out_slice_sizes, args.out_slice_offs = o_ss.data_ptr(), o_so.data_ptr()
    args.out_block_offs, args.out_block_schedule = o_bo.data_ptr(), o_bs.data_ptr()
    args.n_slices, args.max_n_blocks = n_slices, bs.shape[1]
    with _lib.device_guard(dev):
        rc = _lib.lib().tb200_remap_ragged_metadata(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
    _lib.check(rc, "tb200_remap_ragged_metadata")
    return RaggedTensorMetadata(o_ss, o_so, o_bo, o_bs)


@dataclass
class SparseMatrix:
    indx: torch.Tensor
    vals: torch.Tensor
    mask: Bitmatrix

    def __post_init__(self):
        self.mask_metadata = make_bitmatrix_metadata(self.indx, self.mask)


# ----------------------------------------------------------------------------------------------
# Wrapped tensors and layouts for MXFP4 weights (reference: triton_kernels/tensor.py ``Tensor``,
# ``wrap_torch_tensor``, ``convert_layout``, ``FP4``; weight preparation bench/bench_mlp.py:36-57)
# ----------------------------------------------------------------------------------------------
class _FP4Type:
    """Marker for packed e2m1 values (two per byte)."""
    bitwidth = 4

    def __repr__(self):
        return "FP4"


FP4 = _FP4Type()


@dataclass
class Tensor:
    """A torch tensor plus what it means: element type (``FP4`` for packed 4-bit values, else the torch
    dtype), logical shape and the layout its bytes are in."""
    data: torch.Tensor
    dtype: object
    shape: tuple
    layout: object = None


def wrap_torch_tensor(t: torch.Tensor, dtype=None) -> Tensor:
    from .tensor_details.layout import StridedLayout
    if dtype is FP4:
        # packed along the last-but-one axis (the mx axis of a [.., K, N] weight): K/2 bytes hold K values
        shape = (*t.shape[:-2], t.shape[-2] * 2, t.shape[-1])
    else:
        dtype, shape = t.dtype, tuple(t.shape)
    return Tensor(t, dtype, tuple(shape), StridedLayout())


def convert_layout(t: Tensor, layout) -> Tensor:
    """Re-lays an MXFP4 weight (values or scales, quantised along axis -2 of ``[E, K, N]``) into the order
    the kernel reads: values blocked as ``[E][N/256][K/128][256][64 bytes]``, scales in 512-byte atoms. Done once per weight."""
    from .tensor_details.layout import BlackwellMX4ValueLayout, BlackwellMXScaleLayout, StridedLayout
    if isinstance(layout, StridedLayout):
        assert isinstance(t.layout, StridedLayout), "only strided -> kernel layout conversions are built"
        return t
    d = t.data
    if d.ndim == 2:
        d = d.unsqueeze(0)
    assert d.ndim == 3, "expected a [E, K(/2 or /32), N] weight"
    if isinstance(layout, BlackwellMX4ValueLayout):
        assert t.dtype is FP4 and d.dtype == torch.uint8
        E, K2, N = d.shape
        assert (2 * K2) % 32 == 0, "K must be a multiple of the 32-value scale block"
        nk = d.transpose(1, 2)                                   # [E, N, K/2]
        tiles, ksteps = (N + 255) // 256, (K2 + 63) // 64
        if tiles * 256 != N or ksteps * 64 != K2:                # zero rows past N, zero codes (+0.0) past K
            nk = torch.nn.functional.pad(nk, (0, ksteps * 64 - K2, 0, tiles * 256 - N))
        # blocked: [E][N/256][K/128][256 rows][64 bytes] - one tile step is one contiguous 16 KB run
        out = nk.reshape(E, tiles, 256, ksteps, 64).permute(0, 1, 3, 2, 4).contiguous()
        return Tensor(out, FP4, (E, 2 * K2, N), layout)
    if isinstance(layout, BlackwellMXScaleLayout):
        assert d.dtype == torch.uint8
        E, KB, N = d.shape  # KB = K / 32
        nb, ksteps = (N + 127) // 128, (KB + 3) // 4
        if nb * 128 != N or ksteps * 4 != KB:                          # scale 1.0 past N and K
            d = torch.nn.functional.pad(d, (0, nb * 128 - N, 0, ksteps * 4 - KB), value=127)
        s = d.transpose(1, 2).reshape(E, nb, 4, 32, ksteps, 4)          # e, n/128, n/32%4, n%32, k/128, k/32%4
        out = s.permute(0, 1, 4, 3, 2, 5).contiguous()                 # e, n/128, k/128, n%32, n/32%4, k/32%4
        return Tensor(out, torch.uint8, (E, KB, N), layout)
    raise NotImplementedError(f"convert_layout: {layout!r}")
