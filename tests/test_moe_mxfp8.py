"""MX-scaled activations (``precision_config.a_mx_scale``: MXFP8 x MXFP4) and the MX-quantising epilogue
(``precision_config.c_mx_scale`` + ``Epilogue(FnSpecs(FnName.QUANTIZE_MXFP8.name, quantize_mxfp8_fn, ...))``) of
``triton_kernels.matmul.matmul`` against the CPU oracle (``oracle.moe.quantize_mxfp8_ref`` /
``dequantize_mxfp8_ref``, pinned bit-exact to the reference's ``downcast_to_mxfp_torch`` vectors).

Where the arithmetic is exact in fp32 (small integers, power-of-two scales) values and scales must match bit for
bit; with SwiGLU or random data the comparison is the reference's own for this feature (tests/test_matmul.py:
604-625: dequantise both sides, ``maxtol 4e-1, rmstol 4e-2``) plus a bound on how many block scales differ."""
import pytest
import torch

from oracle import moe as o
from triton_b200.triton_kernels.numerics_details.mxfp import (downcast_to_mxfp, quantize_mxfp8_fn,
                                                              upcast_from_mxfp)

pytestmark = pytest.mark.gpu


def _epilogue():
    from triton_b200.triton_kernels.matmul import Epilogue, FnName, FnSpecs
    return Epilogue(FnSpecs(FnName.QUANTIZE_MXFP8.name, quantize_mxfp8_fn, (), ()), tuple(), tuple(), 6.0)


def _exact_operands(M, K, N, E, g):
    """fp8 integers in [-2, 2] with block scales 2^-2..2^2, random FP4 codes with scales 2^-2..2^2: every
    product and every partial sum is exact in fp32."""
    x = torch.randint(-2, 3, (M, K), generator=g).float().to(torch.float8_e4m3fn)
    xs = torch.randint(125, 130, (M, K // 32), generator=g).to(torch.uint8)
    v = torch.randint(0, 256, (E, K // 2, N), generator=g).to(torch.uint8)
    s = torch.randint(125, 130, (E, K // 32, N), generator=g).to(torch.uint8)
    return x, xs, v, s, o.dequantize_mxfp8_ref(x, xs), upcast_from_mxfp(v, s, torch.float32, axis=1)


@pytest.mark.parametrize("M", [128, 300, 24, 1])  # the 128-row kernel (whole and ragged) and the swapped-operand one
def test_mxfp8_activations_exact(cuda, M):
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    K, N = 384, 256
    g = torch.Generator().manual_seed(3)
    x, xs, v, s, xdq, wdq = _exact_operands(M, K, N, 1, g)
    pc = PrecisionConfig(a_mx_scale=xs.to(cuda), a_microblock_size=32, b_mx_scale=s.to(cuda), b_microblock_size=32,
                         out_dtype=torch.float16)
    out = matmul(x.to(cuda), v.to(cuda), None, precision_config=pc)
    ref = (xdq @ wdq[0]).to(torch.float16)
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("M", [128, 300, 24])
def test_mx_output_exact(cuda, M):
    """No activation: the fp32 results are exact, so values and scales equal the oracle's bit for bit."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    K, N = 256, 384
    g = torch.Generator().manual_seed(5)
    x, xs, v, s, xdq, wdq = _exact_operands(M, K, N, 1, g)
    c_scale = torch.full((M, N // 32), 255, dtype=torch.uint8, device=cuda)
    pc = PrecisionConfig(a_mx_scale=xs.to(cuda), a_microblock_size=32, b_mx_scale=s.to(cuda), b_microblock_size=32,
                         c_mx_scale=c_scale)
    out = matmul(x.to(cuda), v.to(cuda), None, precision_config=pc, epilogue=_epilogue())
    assert out.dtype == torch.float8_e4m3fn and out.shape == (M, N)
    q_ref, s_ref = o.quantize_mxfp8_ref(xdq @ wdq[0])
    assert torch.equal(c_scale.cpu(), s_ref)
    assert torch.equal(out.cpu().view(torch.uint8), q_ref.view(torch.uint8))


def _check_like_reference(out, scale, ref32, maxtol=4e-1, rmstol=4e-2):
    """Dequantise the kernel's output and the oracle's quantisation of the fp32 result; compare as the reference's
    test does (testing.py assert_close: max relative error of the larger entries and rms error)."""
    got = o.dequantize_mxfp8_ref(out.cpu(), scale.cpu())
    q_ref, s_ref = o.quantize_mxfp8_ref(ref32)
    want = o.dequantize_mxfp8_ref(q_ref, s_ref)
    ref_max = want.abs().max().clamp_min(1e-6)
    assert float((got - want).abs().max() / ref_max) <= maxtol
    assert float(torch.sqrt(((got - want) ** 2).mean()) / torch.sqrt((want ** 2).mean()).clamp_min(1e-6)) <= rmstol
    # the scales are integers: all but the blocks whose amax sits on a power-of-two boundary must be identical
    differ = (scale.cpu() != s_ref)
    assert float(differ.float().mean()) <= 0.01
    assert int((scale.cpu().int() - s_ref.int()).abs().max()) <= 1


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (777, 16, 4), (32, 16, 2), (5000, 8, 2)])  # the last: more work units than SMs
@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_mxfp8_x_mx4_quantised_output(cuda, T, E, k, swiglu):
    """MXFP8 activations x MXFP4 weights -> (SwiGLU) -> gammas -> scatter -> MXFP8 output, grouped by expert."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    from triton_b200.triton_kernels.topk import topk
    K, N = 256, 512
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(T, E, generator=g)
    sm = topk(logits.to(cuda), k)
    mm = sm.mask_metadata
    R = T * k
    rg = make_ragged_tensor_metadata(mm.col_sum, R)
    xq, xs = downcast_to_mxfp(torch.randn(R, K, generator=g).to(torch.bfloat16), torch.float8_e4m3fn, axis=1)
    v, s = downcast_to_mxfp((0.3 * torch.randn(E, K, N, generator=g)).to(torch.bfloat16), torch.uint8, axis=1)
    wdq = upcast_from_mxfp(v, s, torch.float32, axis=1)
    xdq = o.dequantize_mxfp8_ref(xq, xs)
    gam = torch.rand(R, generator=g)
    n_out = N // 2 if swiglu else N
    c_scale = torch.zeros((R, n_out // 32), dtype=torch.uint8, device=cuda)
    pc = PrecisionConfig(a_mx_scale=xs.to(cuda), a_microblock_size=32, b_mx_scale=s.to(cuda), b_microblock_size=32,
                         c_mx_scale=c_scale)
    combine = mm.col_sorted_indx
    out = matmul(xq.to(cuda), v.to(cuda), None, rg, scatter_indx=combine, gammas=gam.to(cuda), precision_config=pc,
                 fused_activation=swiglu_activation(1.1, 7.0) if swiglu else None, epilogue=_epilogue())
    ref = o.grouped_matmul_ref(xdq, wdq, None, mm.col_sum.cpu().numpy(), scatter_indx=combine.cpu().numpy(),
                               gammas=gam, swiglu=(1.1, 7.0) if swiglu else None, out_dtype=torch.float32)
    _check_like_reference(out, c_scale, ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("swiglu", [False, True])
def test_16bit_matmul_quantised_output(cuda, dtype, swiglu):
    """bf16 / fp16 grouped GEMM with the quantising epilogue, ragged N (the last block of a row is short)."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    E, K, N = 4, 192, 336
    g = torch.Generator().manual_seed(11)
    cnt = torch.tensor([130, 0, 77, 300], dtype=torch.int32)
    R = int(cnt.sum())
    rg = make_ragged_tensor_metadata(cnt.to(cuda), R)
    x = torch.randn(R, K, generator=g).to(dtype)
    w = (0.2 * torch.randn(E, K, N, generator=g)).to(dtype)
    bias = torch.randn(E, N, generator=g)
    n_out = N // 2 if swiglu else N
    c_scale = torch.zeros((R, (n_out + 31) // 32), dtype=torch.uint8, device=cuda)
    out = matmul(x.to(cuda), w.to(cuda), bias.to(cuda), rg, precision_config=PrecisionConfig(c_mx_scale=c_scale),
                 fused_activation=swiglu_activation(1.0, None) if swiglu else None, epilogue=_epilogue())
    assert out.dtype == torch.float8_e4m3fn and out.shape == (R, n_out)
    ref = o.grouped_matmul_ref(x, w, bias, cnt.numpy(), swiglu=(1.0, None) if swiglu else None, out_dtype=torch.float32)
    _check_like_reference(out, c_scale, ref)


def test_argument_checks(cuda):
    from triton_b200.triton_kernels.matmul import Epilogue, FnName, FnSpecs, PrecisionConfig, matmul
    x = torch.zeros(128, 128, dtype=torch.bfloat16, device=cuda)
    w = torch.zeros(1, 128, 128, dtype=torch.bfloat16, device=cuda)
    sc = torch.zeros(128, 4, dtype=torch.uint8, device=cuda)
    with pytest.raises(ValueError):  # scales without the epilogue
        matmul(x, w, None, precision_config=PrecisionConfig(c_mx_scale=sc))
    with pytest.raises(ValueError):  # the epilogue without scales
        matmul(x, w, None, epilogue=_epilogue())
    with pytest.raises(NotImplementedError):  # FP4 outputs are not built
        matmul(x, w, None, precision_config=PrecisionConfig(c_mx_scale=sc),
               epilogue=Epilogue(FnSpecs(FnName.QUANTIZE_MXFP4.name, None, (), ())))
    with pytest.raises(NotImplementedError):  # MX-scaled activations need the MXFP4-weight path
        matmul(x, w, None, precision_config=PrecisionConfig(a_mx_scale=sc, a_microblock_size=32))


@pytest.mark.parametrize("T,E,k", [(300, 8, 2), (24, 16, 2)])  # the 128-row kernel and the swapped-operand one
@pytest.mark.parametrize("swiglu", [False, True])
def test_flexpoint_scales(cuda, T, E, k, swiglu):
    """flex_ctx on the fp8 x MXFP4 path: lhs / rhs scales multiply the accumulator, the output is divided by
    expected_scale and max |output| / 448 comes back in actual_scale (reference: matmul.py:116-121, 810-820,
    flexpoint.py:133-188)."""
    from triton_b200.triton_kernels.matmul import FlexCtx, PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.numerics import InFlexData, OutFlexData
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    from triton_b200.triton_kernels.topk import topk
    K, N = 256, 256
    g = torch.Generator().manual_seed(13)
    sm = topk(torch.randn(T, E, generator=g).to(cuda), k)
    mm = sm.mask_metadata
    R = T * k
    rg = make_ragged_tensor_metadata(mm.col_sum, R)
    x = (torch.randn(R, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    v, s = downcast_to_mxfp((0.3 * torch.randn(E, K, N, generator=g)).to(torch.bfloat16), torch.uint8, axis=1)
    wdq = upcast_from_mxfp(v, s, torch.float32, axis=1)
    xs, ws, expected = 0.75, 1.5, 0.05
    actual = torch.zeros(1, dtype=torch.float32, device=cuda)
    fc = FlexCtx(lhs_data=InFlexData(scale=torch.tensor([xs], device=cuda)),
                 rhs_data=InFlexData(scale=torch.tensor([ws], device=cuda)),
                 out_data=OutFlexData(expected_scale=torch.tensor([expected], device=cuda), actual_scale=actual))
    out = matmul(x.to(cuda), v.to(cuda), None, rg, precision_config=PrecisionConfig(b_mx_scale=s.to(cuda), flex_ctx=fc,
                                                                                      flexpoint_saturate_inf=True),
                 fused_activation=swiglu_activation(1.0, None) if swiglu else None)
    assert out.dtype == torch.float8_e4m3fn
    real = o.grouped_matmul_ref(x.float() * xs, wdq * ws, None, mm.col_sum.cpu().numpy(),
                                swiglu=(1.0, None) if swiglu else None, out_dtype=torch.float32)
    want = (real / expected).clamp(-448, 448).to(torch.float8_e4m3fn).float()
    got = out.cpu().float()
    # fp8 rounding of nearly equal fp32 values may fall on either side of a tie: one e4m3 step (2^-3 relative)
    assert float(((got - want).abs() / want.abs().clamp_min(2.0 ** -6)).max()) <= 0.13
    assert float((got != want).float().mean()) < 0.02
    ref_scale = o.flex_actual_scale_ref(real)
    assert abs(float(actual) - ref_scale) <= 1e-5 * ref_scale + 1e-12
