"""Microscaling (MX) quantisation utilities — counterpart of the reference's
``python/triton_kernels/triton_kernels/numerics_details/mxfp.py`` (``downcast_to_mxfp`` :24,
``upcast_from_mxfp`` :89 and their torch twins :212 / :384).

Weight preparation, not a hot path: plain torch ops on whatever device the input lives on.

``downcast_to_mxfp(x, out_dtype, axis)`` quantises along ``axis`` in blocks of 32: the block's
dequantisation scale is ``max|x| / max_q`` rounded **up** to a power of two (so the block maximum never
clips; ``ROUND_DOWN`` is the OCP variant) and stored as its biased exponent byte (e8m0); the values are
``x / scale`` rounded to nearest-even in the target format and saturated. ``out_dtype=torch.uint8``
means FP4 (e2m1), two values per byte along ``axis`` (even index in the low nibble), so that dimension
halves; ``torch.float8_e4m3fn`` / ``torch.float8_e5m2`` give MXFP8.
"""
from __future__ import annotations

import math
from enum import Enum

import torch

MXFP_BLOCK_SIZE = 32


class DequantScaleRoundingMode(Enum):
    ROUND_UP = 0    # 2^ceil(log2(max / max_q)): the block maximum is never clipped
    ROUND_DOWN = 1  # 2^floor(log2(max / 2^floor(log2(max_q)))): OCP, may clip the maximum


_MAX_Q = {torch.uint8: 6.0, torch.float8_e5m2: 57344.0, torch.float8_e4m3fn: 448.0}
_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def get_max_quant_val(dtype: torch.dtype) -> float:
    return _MAX_Q[dtype]


def _to_e2m1_codes(mag: torch.Tensor) -> torch.Tensor:
    """Magnitude -> 3-bit e2m1 code, round-to-nearest-even, saturating at 6."""
    code = torch.zeros_like(mag, dtype=torch.int32)
    for i in range(7):
        mid = 0.5 * (_E2M1_VALUES[i] + _E2M1_VALUES[i + 1])
        # a tie goes to the even code: up when the lower code i is odd, down when it is even
        code += ((mag >= mid) if (i & 1) else (mag > mid)).to(torch.int32)
    return code


def downcast_to_mxfp(x: torch.Tensor, out_dtype: torch.dtype, axis: int, scale_dtype: torch.dtype = torch.uint8,
                     microblock_size: int = MXFP_BLOCK_SIZE,
                     DEQUANT_SCALE_ROUNDING_MODE: DequantScaleRoundingMode = DequantScaleRoundingMode.ROUND_UP):
    """Returns ``(values, scales)``; shapes as the reference: FP4 halves ``axis``, the scale tensor has
    ``ceil(L / 32)`` entries along ``axis``."""
    assert out_dtype in _MAX_Q, f"Invalid output dtype {out_dtype=}"
    if scale_dtype != torch.uint8:
        raise NotImplementedError("only e8m0 (uint8) block scales are built (NVFP4's e4m3 scales are not)")
    assert x.dtype in (torch.float32, torch.bfloat16, torch.float16), f"Invalid input tensor dtype {x.dtype}"
    assert -x.ndim <= axis < x.ndim, f"Invalid axis {axis=}"
    axis = axis % x.ndim
    is_fp4 = out_dtype == torch.uint8
    L = x.shape[axis]
    if is_fp4:
        assert L % 2 == 0, "For mxfp4 conversion the contiguous axis length must be even."
    src = x.transpose(axis, -1).to(torch.float32)
    pad = (-L) % microblock_size
    blocks = torch.nn.functional.pad(src, (0, pad)).reshape(*src.shape[:-1], (L + pad) // microblock_size, microblock_size)
    amax = blocks.abs().amax(dim=-1, keepdim=True)
    max_q = _MAX_Q[out_dtype]
    if DEQUANT_SCALE_ROUNDING_MODE == DequantScaleRoundingMode.ROUND_UP:
        bits = (amax / max_q).view(torch.int32)
        bits = (bits + 0x007FFFFF) & 0x7F800000  # next power of two at or above
    else:
        bits = (amax / (2.0 ** math.floor(math.log2(max_q)))).view(torch.int32) & 0x7F800000
    scale = bits.view(torch.float32)
    inv = torch.where(scale == 0, torch.zeros_like(scale), 1.0 / scale)
    q = (blocks * inv).reshape(*src.shape[:-1], L + pad)[..., :L]
    if is_fp4:
        codes = _to_e2m1_codes(q.abs()) | ((q.view(torch.int32) >> 28) & 0x8)  # sign bit of the float into bit 3
        codes = codes.to(torch.uint8).reshape(*q.shape[:-1], L // 2, 2)
        values = codes[..., 0] | (codes[..., 1] << 4)
    else:
        values = q.clamp(-max_q, max_q).to(out_dtype)
    scales = (bits >> 23).to(torch.uint8).squeeze(-1)
    return values.transpose(axis, -1), scales.transpose(axis, -1)


def upcast_from_mxfp(tensor: torch.Tensor, scale: torch.Tensor, target_dtype: torch.dtype, axis: int,
                     tensor_scale: torch.Tensor | None = None):
    """Inverse of ``downcast_to_mxfp``: values (FP4 packed in uint8, or fp8) times 2^(scale - 127)."""
    assert tensor.ndim == scale.ndim, "Weight and scale must have the same number of dimensions."
    assert tensor.dtype in (torch.uint8, torch.float8_e5m2, torch.float8_e4m3fn), f"Invalid tensor dtype {tensor.dtype=}"
    assert scale.dtype == torch.uint8, f"Invalid scale dtype {scale.dtype=}"
    assert target_dtype in (torch.float16, torch.bfloat16, torch.float32), f"Invalid output dtype {target_dtype=}"
    axis = axis % tensor.ndim
    t = tensor.transpose(axis, -1)
    s = scale.transpose(axis, -1)
    if tensor.dtype == torch.uint8:
        table = torch.tensor(_E2M1_VALUES + tuple(-v for v in _E2M1_VALUES), dtype=torch.float32, device=tensor.device)
        codes = t.to(torch.int64)
        vals = torch.stack([table[codes & 0xF], table[codes >> 4]], dim=-1).reshape(*t.shape[:-1], t.shape[-1] * 2)
    else:
        vals = t.to(torch.float32)
    L = vals.shape[-1]
    if L == 0:
        return vals.to(target_dtype).transpose(axis, -1).contiguous()
    dq = (s.to(torch.int32) << 23).view(torch.float32)
    pad = (-L) % MXFP_BLOCK_SIZE
    blocks = torch.nn.functional.pad(vals, (0, pad)).reshape(*vals.shape[:-1], (L + pad) // MXFP_BLOCK_SIZE, MXFP_BLOCK_SIZE)
    finfo = torch.finfo(target_dtype)
    out = (blocks * dq.unsqueeze(-1)).clamp(finfo.min, finfo.max)
    if tensor.dtype == torch.float8_e5m2:
        out = out.where(~blocks.isinf(), blocks)
    out = out.reshape(*vals.shape[:-1], L + pad)[..., :L].to(target_dtype).contiguous().transpose(axis, -1)
    if tensor_scale is not None:
        shape = (1,) * out.ndim if tensor_scale.numel() == 1 else (*tensor_scale.shape[:axis], 1, *tensor_scale.shape[axis:])
        out = out * tensor_scale.to(device=out.device).reshape(shape)
    return out.contiguous() if tensor_scale is None else out


# the reference exposes the torch implementations under these names as well
downcast_to_mxfp_torch = downcast_to_mxfp
upcast_from_mxfp_torch = upcast_from_mxfp


def _epilogue_marker(name):
    def fn(*_args, **_kwargs):
        raise RuntimeError(f"{name} names the quantising epilogue of triton_kernels.matmul.matmul (it runs inside the "
                           "GEMM kernel's epilogue); it is not callable on its own")
    fn.__name__ = name
    return fn


# What the reference passes as ``FnSpecs(FnName.QUANTIZE_MXFP8.name, quantize_mxfp8_fn, (), ())`` (jitted device
# functions there, numerics_details/mxfp.py:452-454). Here the name selects the epilogue; the objects are markers.
quantize_mxfp8_fn = _epilogue_marker("quantize_mxfp8_fn")
quantize_mxfp4_fn = _epilogue_marker("quantize_mxfp4_fn")
quantize_nvfp4_fn = _epilogue_marker("quantize_nvfp4_fn")
