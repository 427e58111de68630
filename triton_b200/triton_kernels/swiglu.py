"""``swiglu(a, alpha, precision_config)`` — counterpart of ``triton_kernels/swiglu.py`` in the
reference: ``out = g * sigmoid(alpha * g) * (l + 1)`` with g the even and l the odd columns of
``a`` (g clamped to ``<= limit``, l to ``[-limit, limit]`` when ``precision_config.limit`` is set).
``swiglu_fn`` is the marker passed as ``FusedActivation(FnSpecs("swiglu", swiglu_fn, ...))`` to
``matmul`` to fuse it into the GEMM epilogue."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from .. import _lib

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


@dataclass(frozen=True)
class PrecisionConfig:
    limit: float | None = None


def swiglu_fn(*args, **kwargs):  # marker: the computation is fused into the CUDA epilogue
    raise RuntimeError("swiglu_fn is a marker for matmul(fused_activation=...); call swiglu() instead")


def swiglu(a: torch.Tensor, alpha: float, precision_config: PrecisionConfig = PrecisionConfig(), routing_data=None):
    if not a.is_cuda:
        raise RuntimeError("triton_b200 swiglu needs CUDA tensors (there is no CPU path)")
    assert a.shape[-1] % 2 == 0 and a.dtype in _DT
    a2 = a.reshape(-1, a.shape[-1]).contiguous()
    out = torch.empty((a2.shape[0], a2.shape[1] // 2), dtype=a.dtype, device=a.device)
    args = _lib.SwigluArgs()
    args.a, args.out = a2.data_ptr(), out.data_ptr()
    args.rows, args.n_in, args.lda, args.ldo = a2.shape[0], a2.shape[1], a2.stride(0), out.stride(0)
    args.alpha = float(alpha)
    limit = precision_config.limit if precision_config is not None else None
    args.limit = float(limit) if limit is not None else 0.0
    args.has_limit = 1 if limit is not None else 0
    args.dtype = _DT[a.dtype]
    with _lib.device_guard(a.device):
        rc = _lib.lib().tb200_swiglu(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(a.device)))
    _lib.check(rc, "tb200_swiglu")
    return out.view(a.shape[:-1] + out.shape[-1:])
