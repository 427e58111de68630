"""Per-tensor ("flexpoint") scale holders - counterpart of ``triton_kernels/numerics.py:1-48`` in the reference.

An fp8 tensor ``t`` with ``InFlexData(scale=s)`` stands for the real values ``t * s`` (``s`` a one-element fp32
CUDA tensor). ``OutFlexData``: the kernel divides its result by ``expected_scale`` before the conversion to the
output type and folds ``max |result| / max_finite(output type)`` into ``actual_scale`` with an atomic max (the
caller zeroes it first), so that the next step can pick its scale. ``checksum_scale`` is not implemented."""
from __future__ import annotations

from dataclasses import dataclass

import torch

MAX_FINITE_FLOAT8E5 = 57344.0
MAX_FINITE_FLOAT8E4NV = 448.0
MAX_FINITE_FLOAT8E4B8 = 240.0


@dataclass(frozen=True)
class BaseFlexData:
    dtype: torch.dtype | None = None

    def view(self, x: torch.Tensor):
        return x if self.dtype is None else x.view(self.dtype)

    def reinterpret(self, x):
        if self.dtype is None or x.dtype.itemsize > 1:
            return x
        return x.view(self.dtype)


@dataclass(frozen=True)
class InFlexData(BaseFlexData):
    scale: torch.Tensor | None = None

    @property
    def is_per_batch(self):
        return False if self.scale is None else len(self.scale) > 1


@dataclass(frozen=True)
class OutFlexData(BaseFlexData):
    expected_scale: torch.Tensor | None = None
    actual_scale: torch.Tensor | None = None
    checksum_scale: torch.Tensor | None = None

    @property
    def is_per_batch(self):
        return False if self.expected_scale is None else len(self.expected_scale) > 1

    def __iter__(self):
        yield self.expected_scale
        yield self.actual_scale
        yield self.checksum_scale
