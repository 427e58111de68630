"""``blackwell_scaled_mm_ws(a, b, scale_a, scale_b, ...)`` — counterpart of the reference's FP8
scaled matmul, ``third_party/tlx/tutorials/blackwell_scaled_mm_ws.py:392``.

``a`` [M, K] and ``b`` [N, K] are ``float8_e4m3fn`` (row-major; computes ``A @ B^T``), the result is
``out_dtype`` (bf16 by default). ``scale_mode="tensorwise"`` (one fp32 scalar per operand) and
``"rowwise"`` (``scale_a`` [M] per row of A, ``scale_b`` [N] per row of B) are applied once after the
K loop; ``"blockwise"`` (the default, as in the reference: ``scale_a`` [M, K//128] M-major, ``scale_b``
[N//128, K//128], every 128-wide K group scaled and promoted into an fp32 running sum) runs its own
kernel. The tiling arguments (``BLOCK_M``, ``BLOCK_N``, ``NUM_CTAS``, ``USE_CLC``,
``EPI_SUB``, ``persistent``) are accepted for call compatibility; the kernel picks its own tiling
(``NUM_CTAS=2`` forces the CTA-pair tiling). Same shape assertions as the reference (``:408``).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib

_OUT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}
_IN = {torch.float8_e4m3fn: _lib.E4M3, torch.float8_e5m2: _lib.E5M2}


def blackwell_scaled_mm_ws(a, b, scale_a, scale_b, out_dtype=torch.bfloat16, BLOCK_M=None, BLOCK_N=128, NUM_CTAS=1,
                           USE_CLC=False, EPI_SUB=2, persistent=True, scale_mode="blockwise"):
    if scale_mode not in ("blockwise", "rowwise", "tensorwise"):
        raise KeyError(scale_mode)
    if not a.is_cuda:
        raise RuntimeError("blackwell_scaled_mm_ws needs CUDA tensors (there is no CPU path)")
    M, K = a.shape
    N, Kb = b.shape
    assert K == Kb and K % 128 == 0 and N % 128 == 0
    assert a.dtype in _IN and b.dtype == a.dtype, "fp8 operands of the same dtype"
    assert out_dtype in _OUT
    a = a.contiguous()
    b = b.contiguous()
    if scale_mode == "blockwise":
        assert 128 % BLOCK_N == 0, "blockwise requires BLOCK_N to divide 128"
        G = K // 128
        assert tuple(scale_a.shape) == (M, G) and tuple(scale_b.shape) == (N // 128, G), (
            f"blockwise expects scale_a [M, K//128]=({M}, {G}) and scale_b [N//128, K//128]=({N // 128}, {G}); "
            f"got {tuple(scale_a.shape)}, {tuple(scale_b.shape)}")
        sa = scale_a.to(torch.float32).t().contiguous()  # [K//128, M]: no copy when scale_a is M-major already
        sb = scale_b.to(torch.float32).contiguous()
        c = torch.empty((M, N), dtype=out_dtype, device=a.device)
        if M == 0:
            return c
        bargs = _lib.GemmFp8BlockwiseArgs()
        bargs.a, bargs.b, bargs.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
        bargs.scale_a, bargs.scale_b = sa.data_ptr(), sb.data_ptr()
        bargs.m, bargs.n, bargs.k, bargs.ldc = M, N, K, c.stride(0)
        bargs.in_dtype, bargs.out_dtype = _IN[a.dtype], _OUT[out_dtype]
        with _lib.device_guard(a.device):
            rc = _lib.lib().tb200_gemm_fp8_blockwise(ctypes.byref(bargs),
                                                     ctypes.c_void_p(_lib.current_stream_ptr(a.device)))
        _lib.check(rc, "tb200_gemm_fp8_blockwise")
        return c
    scale_a = scale_a.reshape(-1).contiguous().to(torch.float32)
    scale_b = scale_b.reshape(-1).contiguous().to(torch.float32)
    if scale_mode == "rowwise":
        assert scale_a.numel() == M and scale_b.numel() == N, (
            f"rowwise expects scale_a [M]={M}, scale_b [N]={N}; got {scale_a.numel()}, {scale_b.numel()}")
    else:
        assert scale_a.numel() == 1 and scale_b.numel() == 1, (
            f"tensorwise expects scalar scale_a/scale_b; got {scale_a.numel()}, {scale_b.numel()}")
    c = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if M == 0:
        return c
    args = _lib.GemmArgs()
    args.a, args.b, args.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    args.m, args.n, args.k = M, N, K
    args.lda, args.ldb, args.ldc = K, K, c.stride(0)
    args.in_dtype = _IN[a.dtype]
    args.out_dtype = _OUT[out_dtype]
    args.a_k_major = args.b_k_major = 1
    args.split_k = 1
    # NUM_CTAS=2 forces a CTA pair: 256 x 256 tile, or 256 x 512 when BLOCK_N asks for 512
    args.block_n = (1024 if BLOCK_N == 512 else 512) if NUM_CTAS == 2 else 0
    args.scale_a, args.scale_b = scale_a.data_ptr(), scale_b.data_ptr()
    args.scale_mode = 1 if scale_mode == "rowwise" else 0
    with _lib.device_guard(a.device):
        rc = _lib.lib().tb200_gemm(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(a.device)))
    _lib.check(rc, "tb200_gemm")
    return c
