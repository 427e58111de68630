"""Oracle for the MXFP8 block-scaled GEMM (test infrastructure only).

Reference check (``third_party/tlx/tutorials/testing/test_correctness.py:487-498``):
``matmul(dequantize(a), dequantize(b).T)`` rounded to bf16, where dequantisation multiplies every
1x32 block along K by ``2**(e - 127)`` (e8m0 scale byte e). The scale tensors the kernel takes
are stored in the Blackwell 512-byte-atom layout; (un)swizzling follows
``python/triton_kernels/triton_kernels/tensor_details/layout_details/blackwell_scale.py:104-133``:
[rows, K/32] -> [rows/128, 4, 32, K/128, 4] -> transpose -> [rows/128, K/128, 32, 4, 4].
"""
import numpy as np
import torch


def swizzle_scales(s: torch.Tensor) -> torch.Tensor:
    """[rows, ks] uint8 (rows % 128 == 0, ks % 4 == 0) -> flat swizzled uint8 of the same size."""
    rows, ks = s.shape
    assert rows % 128 == 0 and ks % 4 == 0
    x = s.reshape(rows // 128, 4, 32, ks // 4, 4).permute(0, 3, 2, 1, 4).contiguous()
    return x.reshape(-1)


def unswizzle_scales(flat: torch.Tensor, rows: int, ks: int) -> torch.Tensor:
    x = flat.reshape(rows // 128, ks // 4, 32, 4, 4).permute(0, 3, 2, 1, 4).contiguous()
    return x.reshape(rows, ks)


def e8m0_to_float(e: torch.Tensor) -> torch.Tensor:
    """uint8 exponent bytes -> fp32 2**(e-127) (255 = NaN as in the OCP MX spec)."""
    e = e.to(torch.int32)
    out = torch.pow(torch.tensor(2.0, dtype=torch.float64), (e - 127).double()).float()
    return torch.where(e == 255, torch.full_like(out, float("nan")), out)


def dequantize(q: torch.Tensor, scale_swizzled: torch.Tensor) -> torch.Tensor:
    """q: [rows, K] float8_e4m3fn, scale_swizzled: flat uint8/e8m0 of rows*K/32 bytes -> fp32."""
    q = q.detach().cpu()
    rows, K = q.shape
    sc = scale_swizzled.detach().cpu().view(torch.uint8).reshape(-1)
    s = unswizzle_scales(sc, rows, K // 32)
    f = e8m0_to_float(s)
    return q.float() * f.repeat_interleave(32, dim=1)


def mxfp8_gemm_ref(a, b, a_scale, b_scale, out_dtype=torch.bfloat16):
    """a [M, K], b [N, K] e4m3; scales flat swizzled e8m0. Returns dq(a) @ dq(b).T."""
    return (dequantize(a, a_scale) @ dequantize(b, b_scale).t()).to(out_dtype)


def make_mxfp8_operand(rows: int, K: int, gen: torch.Generator):
    """Synthetic operand of the MXFP8 benchmark configuration: per 1x32 block a scale 2**u with u an
    integer uniform in [-4, 4], elements N(0,1) clipped into the e4m3 range and rounded to e4m3.
    Returns (q float8_e4m3fn [rows, K], swizzled scale bytes uint8 [rows*K/32])."""
    x = torch.randn(rows, K, generator=gen)
    x = x.clamp_(-448.0, 448.0)
    q = x.to(torch.float8_e4m3fn)
    u = torch.randint(-4, 5, (rows, K // 32), generator=gen)
    s = (u + 127).to(torch.uint8)
    return q, swizzle_scales(s)
