"""``topk(x, k, apply_softmax=True, dim=1, y_indx=None, n_rows=None, all_gather=False,
symm_mem_pool=None) -> SparseMatrix`` — counterpart of ``triton_kernels/topk.py:106`` in the
reference: per-row top-k with ties to the smaller column, values in descending order, optional
softmax over the k selected values, int16 indices and the transposed-in-memory bitmatrix.
``all_gather=True`` with a ``symm_mem_pool`` (a ``SymmetricMemoryPool`` or ``EpGroup`` of
``triton_kernels.distributed``) is the expert-parallel path (``topk.py:41-69`` in the reference): every rank
gets the values and indices of all ranks' rows, rank-major; the exchange is one NCCL all-gather and the
bitmatrix words of the gathered result are not materialised (its metadata is built from the indices)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib
from .tensor import Bitmatrix, SparseMatrix

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def topk_forward(x, k, apply_softmax=True, dim=1, y_indx=None, n_rows=None, all_gather=False, symm_mem_pool=None):
    assert x.ndim == 2 and dim == 1
    assert x.shape[-1] < 32768
    if all_gather:
        raise NotImplementedError("topk_forward is the local kernel; call topk(..., all_gather=True, symm_mem_pool=...)")
    if not x.is_cuda:
        raise RuntimeError("triton_b200 topk needs CUDA tensors (there is no CPU path)")
    assert x.dtype in _DT and x.stride(1) == 1
    rows, n_cols = x.shape
    n_valid = rows if n_rows is None else int(n_rows)
    dev = x.device
    y_vals = torch.empty((rows, k), dtype=x.dtype, device=dev)
    use_provided = y_indx is not None
    if use_provided:
        assert y_indx.dtype == torch.int16 and y_indx.shape == (rows, k) and y_indx.is_contiguous()
    else:
        y_indx = torch.empty((rows, k), dtype=torch.int16, device=dev)
    n_words = (n_cols + 31) // 32
    rows_pad = (rows + 31) // 32 * 32
    bits_t = torch.empty((n_words, rows_pad), dtype=torch.int32, device=dev)
    bits = bits_t.transpose(0, 1)[:rows]
    args = _lib.TopkArgs()
    args.x, args.y_vals, args.y_indx, args.bitmatrix = x.data_ptr(), y_vals.data_ptr(), y_indx.data_ptr(), bits_t.data_ptr()
    args.rows_alloc, args.n_rows, args.n_cols = rows, n_valid, n_cols
    args.stride_x, args.stride_y = x.stride(0), k
    args.bits_stride_row, args.bits_stride_word = 1, rows_pad
    args.k, args.dtype = k, _DT[x.dtype]
    args.apply_softmax = 1 if apply_softmax else 0
    args.use_provided_indx = 1 if use_provided else 0
    with _lib.device_guard(dev):
        rc = _lib.lib().tb200_topk(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
    _lib.check(rc, "tb200_topk")
    bitmatrix = Bitmatrix(bits, shape=[n_valid, n_cols], shape_max=[rows, None])
    return y_vals, y_indx, bitmatrix


def topk(x: torch.Tensor, k: int, apply_softmax: bool = True, dim: int = 1, y_indx: Optional[torch.Tensor] = None,
         n_rows: Optional[int] = None, all_gather: bool = False, symm_mem_pool=None) -> SparseMatrix:
    if all_gather:
        if symm_mem_pool is None or y_indx is not None or n_rows is not None:
            raise NotImplementedError("topk(all_gather=True) needs symm_mem_pool and takes neither y_indx nor n_rows")
        from .distributed import all_gather_topk
        assert dim == 1
        return all_gather_topk(x, k, symm_mem_pool, apply_softmax)
    y_vals, y_indx, bitmatrix = topk_forward(x, k, apply_softmax, dim, y_indx, n_rows, all_gather, symm_mem_pool)
    return SparseMatrix(vals=y_vals, indx=y_indx, mask=bitmatrix)
