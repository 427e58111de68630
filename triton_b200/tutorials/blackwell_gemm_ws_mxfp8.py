"""``matmul(a, b, a_scale, b_scale, config=None)`` — counterpart of the reference's MXFP8
block-scaled GEMM, ``third_party/tlx/tutorials/blackwell_gemm_ws_mxfp8.py:1135``.

Computes ``A @ B.T`` from pre-quantised operands: ``a`` [M, K] and ``b`` [N, K] contiguous
``float8_e4m3fn``; ``a_scale`` / ``b_scale`` ``float8_e8m0fnu`` with one scale per 32 K values in
the swizzled 512-byte-atom order (``rows*K/32`` elements, any shape). Returns bf16 [M, N].
The same assertions as the reference apply (dtypes, contiguity, same device, M, N, K % 128 == 0,
``:1155-1168``). ``config``: ``BLOCK_SIZE_N`` / ``BLOCK_N`` (128 or 256) is honoured, the other keys
describe choices this kernel makes itself and are ignored.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib

VEC_SIZE = 32


def matmul(a: torch.Tensor, b: torch.Tensor, a_scale: torch.Tensor, b_scale: torch.Tensor,
           config: dict | None = None) -> torch.Tensor:
    assert a.ndim == 2 and b.ndim == 2, "A and B must be matrices"
    assert a.dtype == torch.float8_e4m3fn, "A must use E4M3 data"
    assert b.dtype == torch.float8_e4m3fn, "B must use E4M3 data"
    assert a.is_contiguous() and b.is_contiguous(), "A and B must be contiguous"
    assert a.device == b.device, "A and B must be on the same device"
    assert a_scale.device == a.device and b_scale.device == a.device, "Data and scales must be on the same device"
    assert a_scale.dtype == torch.float8_e8m0fnu
    assert b_scale.dtype == torch.float8_e8m0fnu
    if not a.is_cuda:
        raise RuntimeError("triton_b200 MXFP8 matmul needs CUDA tensors (there is no CPU path)")
    M, K = a.shape
    N, b_k = b.shape
    assert K == b_k, "A and B must have the same K dimension"
    assert M % 128 == 0 and N % 128 == 0, "M and N must be multiples of 128"
    assert K % 128 == 0, "K must be a multiple of 128"
    assert a_scale.numel() == M * K // VEC_SIZE, f"Expected {M * K // VEC_SIZE} E8M0 scales, got {a_scale.numel()}"
    assert b_scale.numel() == N * K // VEC_SIZE, f"Expected {N * K // VEC_SIZE} E8M0 scales, got {b_scale.numel()}"
    a_scale = a_scale.contiguous()
    b_scale = b_scale.contiguous()
    out = torch.empty((M, N), device=a.device, dtype=torch.bfloat16)
    if M == 0 or N == 0:
        return out
    args = _lib.GemmMxfp8Args()
    args.a, args.b = a.data_ptr(), b.data_ptr()
    args.a_scale, args.b_scale = a_scale.data_ptr(), b_scale.data_ptr()
    args.c = out.data_ptr()
    args.m, args.n, args.k, args.ldc = M, N, K, out.stride(0)
    bn = 0
    if config:
        bn = int(config.get("BLOCK_SIZE_N", config.get("BLOCK_N", 0)) or 0)
    args.block_n = bn if bn in (128, 256, 512) else 0
    if config and int(config.get("NUM_CTAS", 1) or 1) == 2:
        args.block_n = 512  # CTA pair, 256 x 256 tile per cluster
    with _lib.device_guard(a.device):
        rc = _lib.lib().tb200_gemm_mxfp8(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(a.device)))
    _lib.check(rc, "tb200_gemm_mxfp8")
    return out
