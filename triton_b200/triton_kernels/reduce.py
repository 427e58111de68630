"""``reduce(x, dim, mask=None, scale=None) -> (y, None)`` — counterpart of
``triton_kernels/reduce.py:1135`` in the reference for the MoE combine
``reduce(y.view(-1, k, d), dim=1)``: sum over the k expert slots of each token in fp32, optionally
masked / scaled per (token, slot). MX and flexpoint arguments raise ``NotImplementedError``."""
from __future__ import annotations

import ctypes

import torch

from .. import _lib

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def reduce(x: torch.Tensor, dim: int, mask=None, scale=None, x_mxscale=None, x_flex=None, y_flex=None,
           y_flex_saturate_inf=False, postprocess_fn1=None, unpadded_batch_size=None, row_indx=None):
    if x_mxscale is not None or postprocess_fn1 is not None or y_flex is not None:
        raise NotImplementedError("reduce: MX, flexpoint and post-processing arguments are not implemented")
    if not x.is_cuda:
        raise RuntimeError("triton_b200 reduce needs CUDA tensors (there is no CPU path)")
    assert x.ndim == 3 and dim in (1, -2), "reduce is built for [tokens, k, d] summed over dim 1"
    assert x.dtype in _DT
    x = x.contiguous()
    T, k, d = x.shape
    ri = None
    if row_indx is not None:  # extension: slot (t, j) reads row row_indx[t*k + j] of x.view(-1, d)
        ri = row_indx.to(torch.int32).contiguous()
        assert ri.numel() == T * k
    assert d % 8 == 0
    y = torch.empty((T, d), dtype=x.dtype, device=x.device)
    m = None
    if mask is not None:
        m = mask.expand(T, k, -1)[..., 0].to(torch.uint8).contiguous() if mask.ndim == 3 else mask.to(torch.uint8).contiguous()
    s = None
    if scale is not None:
        s = scale.expand(T, k, -1)[..., 0].float().contiguous() if scale.ndim == 3 else scale.float().contiguous()
    args = _lib.ReduceKArgs()
    args.x, args.y = x.data_ptr(), y.data_ptr()
    args.mask = m.data_ptr() if m is not None else None
    args.scale = s.data_ptr() if s is not None else None
    args.row_indx = ri.data_ptr() if ri is not None else None
    args.n_tokens, args.d, args.k, args.dtype = T, d, k, _DT[x.dtype]
    with _lib.device_guard(x.device):
        rc = _lib.lib().tb200_reduce_k(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(x.device)))
    _lib.check(rc, "tb200_reduce_k")
    return y, None
