"""Weight layouts for MXFP4 matmuls — counterpart of the reference's
``triton_kernels/tensor_details/layout.py`` (``make_default_matmul_mxfp4_w_layout``,
``make_default_matmul_mxfp4_w_scale_layout``) and ``layout_details/blackwell_{value,scale}.py``.

The reference picks, per GPU generation, how packed FP4 values and their e8m0 scales are laid out for
its kernel. Here there is one target and one kernel (``tb200_moe_gemm_mx4``):

* values: two e2m1 values per byte along K (even index in the low nibble), blocked as
  ``[E][N/256][K/128][256 rows][64 bytes]`` so that a tile's K step is one contiguous 16 KB run of HBM;
* scales: per expert, 512-byte atoms ``[N/128][K/128][n % 32][n / 32 % 4][k / 32 % 4]`` — the order in
  which ``tcgen05.cp.32x128b.warpx4`` wants them (``layout_details/blackwell_scale.py:100-122``).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class StridedLayout:
    name: str = "strided"


@dataclass(frozen=True)
class BlackwellMX4ValueLayout:
    mx_axis: int = 1
    name: str = "tb200_mx4_value"


@dataclass(frozen=True)
class BlackwellMXScaleLayout:
    mx_axis: int = 1
    name: str = "tb200_mx_scale"


def make_default_matmul_mxfp4_w_layout(mx_axis: int = 1, **_ignored):
    return BlackwellMX4ValueLayout(mx_axis=mx_axis)


def make_default_matmul_mxfp4_w_scale_layout(mx_axis: int = 1, num_warps: int = 8, **_ignored):
    return BlackwellMXScaleLayout(mx_axis=mx_axis)
