"""MX quantisation utilities against golden vectors produced by the reference's own torch implementations
(tests/golden/make_mxfp_fixture.py -> mxfp_cases.npz): bit-exact values and scales for FP4 and MXFP8, both scale
rounding modes, every e2m1 rounding tie, zeros, a non-last axis; and the upcast."""
import os

import numpy as np
import pytest
import torch

from triton_b200.triton_kernels.numerics_details.mxfp import (DequantScaleRoundingMode, downcast_to_mxfp,
                                                              upcast_from_mxfp)

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "mxfp_cases.npz"))
CASES = ["normal", "wide", "ties", "zeros", "axis0"]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("mode", list(DequantScaleRoundingMode))
@pytest.mark.parametrize("q", ["fp4", "e4m3"])
def test_downcast_and_upcast_match_reference_vectors(case, mode, q):
    x = torch.from_numpy(GOLD[f"{case}_x"])
    axis = 0 if case == "axis0" else -1
    qt = torch.uint8 if q == "fp4" else torch.float8_e4m3fn
    v, s = downcast_to_mxfp(x, qt, axis, DEQUANT_SCALE_ROUNDING_MODE=mode)
    key = f"{case}_{q}_{mode.name}"
    assert np.array_equal(s.contiguous().numpy(), GOLD[key + "_s"]), "scales"
    assert np.array_equal(v.contiguous().view(torch.uint8).numpy(), GOLD[key + "_v"]), "values"
    up = upcast_from_mxfp(v, s, torch.float32, axis)
    assert np.array_equal(up.numpy(), GOLD[key + "_up"]), "upcast"


def test_round_trip_error_bound():
    """FP4 with a round-up scale never clips: |x - up(down(x))| <= half a grid step of the block."""
    torch.manual_seed(0)
    x = torch.randn(16, 256)
    v, s = downcast_to_mxfp(x, torch.uint8, -1)
    assert v.shape == (16, 128) and s.shape == (16, 8) and v.dtype == torch.uint8 and s.dtype == torch.uint8
    up = upcast_from_mxfp(v, s, torch.float32, -1)
    step = torch.pow(2.0, s.float() - 127).repeat_interleave(32, dim=-1)  # the coarsest grid step is 2 * scale
    assert torch.all((x - up).abs() <= step + 1e-12)


def test_argument_checks():
    with pytest.raises(AssertionError):
        downcast_to_mxfp(torch.zeros(4, 33), torch.uint8, -1)  # odd length cannot be packed
    with pytest.raises(AssertionError):
        downcast_to_mxfp(torch.zeros(4, 32, dtype=torch.int32), torch.uint8, -1)
    with pytest.raises(NotImplementedError):
        downcast_to_mxfp(torch.zeros(4, 32), torch.uint8, -1, scale_dtype=torch.float8_e4m3fn)
