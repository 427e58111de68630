"""``matmul(a, b, config=None)`` — counterpart of the reference's Blackwell warp-specialised
persistent GEMM, ``third_party/tlx/tutorials/blackwell_gemm_ws.py:1486``.

Same contract: ``a`` is (M, K), ``b`` is (K, N), fp16 or bf16, each either contiguous or the
transpose of a contiguous matrix (the reference detects this with ``is_contiguous()``,
``:1508-1522``); the result is a new (M, N) tensor of ``a.dtype`` on ``a.device``, computed
with fp32 accumulation on the current CUDA stream. ``config`` takes the reference's dict
keys; ``SPLIT_K`` and ``BLOCK_SIZE_N`` are honoured, the others describe scheduling choices
that this kernel makes itself and are accepted and ignored.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def _operand(t: torch.Tensor):
    """Returns (tensor, k_major_for_A_convention, leading_dim): how a 2-D operand lies in memory."""
    if t.stride(1) == 1 and t.stride(0) >= t.shape[1]:
        return t, True, t.stride(0)
    if t.stride(0) == 1 and t.stride(1) >= t.shape[0]:
        return t, False, t.stride(1)
    t = t.contiguous()
    return t, True, t.stride(0)


def get_heuristic_config(M, N, K, num_sms=148, dtype=torch.bfloat16, b_k_major=True):
    """The tiling the library takes for a shape, in the reference's vocabulary
    (``blackwell_gemm_ws.py:25-335``), read from the C side (``tb200_gemm_plan``): ``BLOCK_SIZE_M`` x
    ``BLOCK_SIZE_N`` is the tile one CTA (``NUM_CTAS`` = 1) or one CTA pair (2) computes."""
    args = _lib.GemmArgs()
    args.a = args.b = args.c = 16
    args.m, args.n, args.k = M, N, K
    args.lda, args.ldb, args.ldc = K, (K if b_k_major else N), N
    args.in_dtype = args.out_dtype = _DT[dtype]
    args.a_k_major, args.b_k_major = 1, int(b_k_major)
    out = (ctypes.c_int32 * 6)()
    _lib.check(_lib.lib().tb200_gemm_plan(ctypes.byref(args), out), "tb200_gemm_plan")
    return {"BLOCK_SIZE_M": out[0], "BLOCK_SIZE_N": out[1], "BLOCK_SIZE_K": out[5], "NUM_CTAS": out[2],
            "SPLIT_K": out[3], "NUM_SMEM_BUFFERS": out[4]}


def matmul(a: torch.Tensor, b: torch.Tensor, config=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out`` (extension): an (M, N) tensor of ``a.dtype`` with unit column stride that receives the product."""
    assert a.dim() == 2 and b.dim() == 2, "matmul expects 2-D operands"
    assert a.shape[1] == b.shape[0], "Incompatible dimensions"
    if not a.is_cuda or not b.is_cuda:
        raise RuntimeError("triton_b200.matmul needs CUDA tensors (there is no CPU path)")
    assert a.dtype == b.dtype and a.dtype in _DT, "fp16 or bf16 operands of the same dtype"
    assert a.device == b.device
    M, K = a.shape
    _, N = b.shape
    if out is not None:
        assert out.shape == (M, N) and out.dtype == a.dtype and out.device == a.device and out.stride(1) == 1
        c = out
    else:
        c = torch.empty((M, N), device=a.device, dtype=a.dtype)
    if M == 0 or N == 0:
        return c
    if K == 0:
        return c.zero_()

    a, a_k_major, lda = _operand(a)
    # For B (K, N): contiguous rows mean N is the fast axis, i.e. not K-major.
    b, b_n_fast, ldb = _operand(b)
    b_k_major = not b_n_fast

    args = _lib.GemmArgs()
    args.a, args.b, args.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    args.m, args.n, args.k = M, N, K
    args.lda, args.ldb, args.ldc = lda, ldb, c.stride(0)
    args.in_dtype = args.out_dtype = _DT[a.dtype]
    args.a_k_major = int(a_k_major)
    args.b_k_major = int(b_k_major)
    args.split_k = 0
    args.block_n = 0
    if config:
        args.split_k = int(config.get("SPLIT_K", 0) or 0)
        bn = int(config.get("BLOCK_SIZE_N", 0) or 0)
        args.block_n = bn if bn in (64, 128, 256, 512, 1024) else 0  # 512 / 1024: CTA pair, 256 x 256 / 256 x 512 tile
        if int(config.get("NUM_CTAS", 1) or 1) == 2:
            args.block_n = 512  # CTA pair: 256 x 256 tile per 2-CTA cluster
    l = _lib.lib()
    with _lib.device_guard(a.device):
        need = l.tb200_gemm_workspace_bytes(ctypes.byref(args))
        ws = None
        if need:
            ws = torch.empty(need, dtype=torch.uint8, device=a.device)
            args.workspace, args.workspace_bytes = ws.data_ptr(), need
        rc = l.tb200_gemm(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(a.device)))
    _lib.check(rc, "tb200_gemm")
    return c
