"""FP8 (and bf16 / fp16) activations x MXFP4 weights through ``triton_kernels.matmul.matmul`` (dense and grouped) against the
CPU oracle applied to the dequantised weights. The products are exact in fp32 up to summation order (fp8 x
fp4 values with power-of-two scales), so the tolerance is bf16 output rounding: rtol 1e-2 / atol 1e-2; the
reference's own matmul tolerance is maxtol 2e-2 (triton_kernels testing.py:21-80)."""
import numpy as np
import pytest
import torch

from oracle import moe as o
from triton_b200.triton_kernels.numerics_details.mxfp import downcast_to_mxfp, upcast_from_mxfp

pytestmark = pytest.mark.gpu


def _quantise(w):
    v, s = downcast_to_mxfp(w.to(torch.bfloat16), torch.uint8, axis=1)
    return v, s, upcast_from_mxfp(v, s, torch.float32, axis=1)


def _prepared(v, s, cuda):
    from triton_b200.triton_kernels.tensor import FP4, convert_layout, wrap_torch_tensor
    from triton_b200.triton_kernels.tensor_details.layout import (make_default_matmul_mxfp4_w_layout,
                                                                  make_default_matmul_mxfp4_w_scale_layout)
    wv = convert_layout(wrap_torch_tensor(v.to(cuda), dtype=FP4), make_default_matmul_mxfp4_w_layout(mx_axis=1))
    ws = convert_layout(wrap_torch_tensor(s.to(cuda)), make_default_matmul_mxfp4_w_scale_layout(mx_axis=1))
    return wv, ws


@pytest.mark.parametrize("shape", [(128, 256, 128), (300, 384, 512), (64, 128, 1024), (1024, 1024, 2048),
                                   (16, 384, 512), (32, 256, 4096), (1, 128, 128),
                                   # K and N that are no multiples of 128 (the reference's 300 x 400 x 832 and
                                   # 1000 x 704 x 800, tests/test_matmul.py:194,210), on both kernels
                                   (300, 400, 832), (1000, 704, 800), (24, 400, 416), (5, 48, 96)])
@pytest.mark.parametrize("prepared", [True, False])
def test_dense_fp8_x_mx4(cuda, shape, prepared):
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    M, N, K = shape
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    v, s, wdq = _quantise(torch.randn(1, K, N, generator=g))
    if prepared:
        wv, ws = _prepared(v, s, cuda)
    else:
        wv, ws = v.to(cuda), s.to(cuda)
    out = matmul(x.to(cuda), wv, None, precision_config=PrecisionConfig(b_mx_scale=ws, out_dtype=torch.bfloat16))
    ref = x.float() @ wdq[0]
    assert out.dtype == torch.bfloat16
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-2, atol=1e-2)


def test_exact_on_random_codes(cuda):
    """Random FP4 codes and scale exponents fed to the kernel as they are, small integer activations: every
    product is a multiple of 2^-3 and every partial sum is exact in fp32, so the fp16 output must equal the
    oracle's bit for bit (checks nibble order, scale-atom order and the 32-value block boundaries)."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    M, N, K = 128, 256, 256
    g = torch.Generator().manual_seed(2)
    x = torch.randint(-2, 3, (M, K), generator=g).float().to(torch.float8_e4m3fn)
    v = torch.randint(0, 256, (1, K // 2, N), generator=g).to(torch.uint8)
    s = torch.randint(125, 130, (1, K // 32, N), generator=g).to(torch.uint8)
    wdq = upcast_from_mxfp(v, s, torch.float32, axis=1)
    out = matmul(x.to(cuda), v.to(cuda), None,
                 precision_config=PrecisionConfig(b_mx_scale=s.to(cuda), out_dtype=torch.float16))
    ref = (x.float() @ wdq[0]).to(torch.float16)
    assert torch.equal(out.cpu(), ref)


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (777, 16, 4), (4096, 32, 4), (64, 128, 4), (300, 64, 4)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_fp8_x_mx4(cuda, T, E, k, swiglu):
    """Expert-sorted rows, ragged metadata, bias, optional SwiGLU, gammas and scatter, with an activation scale."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    from triton_b200.triton_kernels.topk import topk
    K, N = 256, 512
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(T, E, generator=g)
    sm = topk(logits.to(cuda), k)
    mm = sm.mask_metadata
    rg = make_ragged_tensor_metadata(mm.col_sum, T * k)
    combine = mm.col_sorted_indx  # sorted row r -> flat (token, slot) entry
    x_tok = (torch.randn(T, K, generator=g) * 0.5)
    x_sorted = x_tok[(combine.cpu().long() // k)].to(torch.float8_e4m3fn)  # rows already in expert order
    v, s, wdq = _quantise(torch.randn(E, K, N, generator=g) * 0.5)
    bias = torch.randn(E, N, generator=g)
    gam = torch.rand(T * k, generator=g)
    wv, ws = _prepared(v, s, cuda)
    act = swiglu_activation(1.1, 7.0) if swiglu else None
    out = matmul(x_sorted.to(cuda), wv, bias.to(cuda), rg, scatter_indx=combine, gammas=gam.to(cuda),
                 precision_config=PrecisionConfig(b_mx_scale=ws, x_scale=0.25, out_dtype=torch.bfloat16),
                 fused_activation=act)
    ref = o.grouped_matmul_ref(x_sorted.float() * 0.25, wdq, bias, mm.col_sum.cpu().numpy(), None,
                               combine.cpu().numpy(), gam, (1.1, 7.0) if swiglu else None, out_dtype=torch.bfloat16)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_exact_on_random_codes_few_rows_kernel(cuda):
    """The same exactness check through the swapped-operand kernel (rows <= 32 per expert)."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    M, N, K = 24, 384, 512
    g = torch.Generator().manual_seed(6)
    x = torch.randint(-2, 3, (M, K), generator=g).float().to(torch.float8_e4m3fn)
    v = torch.randint(0, 256, (1, K // 2, N), generator=g).to(torch.uint8)
    s = torch.randint(125, 130, (1, K // 32, N), generator=g).to(torch.uint8)
    wdq = upcast_from_mxfp(v, s, torch.float32, axis=1)
    out = matmul(x.to(cuda), v.to(cuda), None,
                 precision_config=PrecisionConfig(b_mx_scale=s.to(cuda), out_dtype=torch.float16))
    assert torch.equal(out.cpu(), (x.float() @ wdq[0]).to(torch.float16))


def _fp8_sat(x, dtype):
    """fp32 -> fp8 the way the kernels convert: round to nearest even, saturate to the largest finite value."""
    lim = torch.finfo(dtype).max
    return x.clamp(-lim, lim).to(dtype)


@pytest.mark.parametrize("M", [128, 24])  # the 128-row kernel and the swapped-operand one
@pytest.mark.parametrize("out_dtype", [None, torch.float8_e5m2])
def test_fp8_output_exact(cuda, M, out_dtype):
    """Default output dtype = the activations' (fp8), as in the reference (matmul.py:175). Integer activations and
    random codes make every accumulator exact, so the fp8 output must equal the saturating round-to-nearest cast
    of the oracle's fp32 product bit for bit; the scale exponents are chosen so that some outputs saturate."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    N, K = 384, 256
    g = torch.Generator().manual_seed(11)
    x = torch.randint(-2, 3, (M, K), generator=g).float().to(torch.float8_e4m3fn)
    v = torch.randint(0, 256, (1, K // 2, N), generator=g).to(torch.uint8)
    s = torch.randint(124, 132, (1, K // 32, N), generator=g).to(torch.uint8)
    wdq = upcast_from_mxfp(v, s, torch.float32, axis=1)
    out = matmul(x.to(cuda), v.to(cuda), None, precision_config=PrecisionConfig(b_mx_scale=s.to(cuda), out_dtype=out_dtype))
    want_dtype = out_dtype or torch.float8_e4m3fn
    assert out.dtype == want_dtype
    ref = _fp8_sat(x.float() @ wdq[0], want_dtype)
    if want_dtype == torch.float8_e4m3fn:
        assert (ref.float().abs() == 448).any(), "the case is meant to saturate somewhere"
    assert torch.equal(out.cpu().view(torch.uint8), ref.view(torch.uint8))


def test_fp8_output_swiglu_scatter(cuda):
    """fp8 output through SwiGLU, gammas and scatter (ragged N tail of 16 outputs per 32 columns included)."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    from triton_b200.triton_kernels.topk import topk
    T, E, k, K, N = 300, 16, 4, 256, 384
    g = torch.Generator().manual_seed(12)
    sm = topk(torch.randn(T, E, generator=g).to(cuda), k)
    mm = sm.mask_metadata
    rg = make_ragged_tensor_metadata(mm.col_sum, T * k)
    combine = mm.col_sorted_indx
    x_sorted = (torch.randn(T, K, generator=g) * 0.5)[(combine.cpu().long() // k)].to(torch.float8_e4m3fn)
    v, s, wdq = _quantise(torch.randn(E, K, N, generator=g) * 0.5)
    gam = torch.rand(T * k, generator=g)
    out = matmul(x_sorted.to(cuda), v.to(cuda), None, rg, scatter_indx=combine, gammas=gam.to(cuda),
                 precision_config=PrecisionConfig(b_mx_scale=s.to(cuda)), fused_activation=swiglu_activation(1.1, 7.0))
    assert out.dtype == torch.float8_e4m3fn and out.shape == (T * k, N // 2)
    ref = o.grouped_matmul_ref(x_sorted.float(), wdq, None, mm.col_sum.cpu().numpy(), None, combine.cpu().numpy(), gam,
                               (1.1, 7.0), out_dtype=torch.float32)
    # one fp8 rounding step (2^-3 relative) on top of the fp32 summation-order difference
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=0.07, atol=2e-2)


def test_fp8_x_mx4_gather_indx(cuda):
    """gather_indx with fp8 activations: rows gathered by tb200_gather_rows, then the sorted-row kernel; equal to
    gathering by hand."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    T, R, K, N, E = 100, 384, 256, 256, 4
    g = torch.Generator().manual_seed(13)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.float8_e4m3fn).to(cuda)
    v, s, _ = _quantise(torch.randn(E, K, N, generator=g) * 0.5)
    gather = torch.randint(0, T, (R,), generator=g).to(torch.int32).to(cuda)
    rg = make_ragged_tensor_metadata(torch.full((E,), R // E, dtype=torch.int32, device=cuda), R)
    pc = PrecisionConfig(b_mx_scale=s.to(cuda), out_dtype=torch.bfloat16)
    got = matmul(x, v.to(cuda), None, rg, gather_indx=gather, precision_config=pc)
    want = matmul(x.view(torch.uint8)[gather.long()].view(torch.float8_e4m3fn), v.to(cuda), None, rg, precision_config=pc)
    assert torch.equal(got, want)


def test_upcast_bit_exact(cuda):
    """tb200_mxfp4_upcast against upcast_from_mxfp (itself pinned on the reference's golden vectors): every code,
    every scale byte - 0 (zero), 255 (infinity: NaN for a zero code) and the range where fp16 clamps included -
    and an N that is a multiple of 128 but not of 256 (the blocked layout pads it)."""
    from triton_b200.triton_kernels.matmul import upcast_mxfp4_weight
    E, K, N = 3, 256, 384
    g = torch.Generator().manual_seed(7)
    v = torch.randint(0, 256, (E, K // 2, N), generator=g).to(torch.uint8)
    s = torch.randint(0, 256, (E, K // 32, N), generator=g).to(torch.uint8)
    for dtype in (torch.bfloat16, torch.float16):
        got = upcast_mxfp4_weight(v.to(cuda), s.to(cuda), dtype)
        assert got.shape == (E, K, N) and got.stride(1) == 1
        want = upcast_from_mxfp(v, s, dtype, axis=1)
        got = got.cpu()
        nan = want.isnan()
        assert torch.equal(got.isnan(), nan)
        assert torch.equal(got.view(torch.int16)[~nan], want.view(torch.int16)[~nan])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape", [(128, 256, 128), (300, 384, 512), (1, 128, 128)])
def test_dense_16bit_x_mx4(cuda, shape, dtype):
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    M, N, K = shape
    g = torch.Generator().manual_seed(8)
    x = (torch.randn(M, K, generator=g) * 0.5).to(dtype)
    v, s, wdq = _quantise(torch.randn(1, K, N, generator=g))
    out = matmul(x.to(cuda), v.to(cuda), None, precision_config=PrecisionConfig(b_mx_scale=s.to(cuda)))
    assert out.dtype == dtype
    torch.testing.assert_close(out.cpu().float(), x.float() @ wdq[0], rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("T,E,k", [(64, 8, 2), (777, 16, 4)])
def test_grouped_bf16_x_mx4(cuda, T, E, k):
    """bf16 activations gathered by token, MXFP4 expert weights, SwiGLU, gammas and scatter."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    from triton_b200.triton_kernels.topk import topk
    K, N = 256, 512
    g = torch.Generator().manual_seed(9)
    sm = topk(torch.randn(T, E, generator=g).to(cuda), k)
    mm = sm.mask_metadata
    rg = make_ragged_tensor_metadata(mm.col_sum, T * k)
    combine = mm.col_sorted_indx
    gather = (combine // k).to(torch.int32)
    x = (torch.randn(T, K, generator=g) * 0.5).to(torch.bfloat16)
    v, s, wdq = _quantise(torch.randn(E, K, N, generator=g) * 0.5)
    bias = torch.randn(E, N, generator=g)
    gam = torch.rand(T * k, generator=g)
    wv, ws = _prepared(v, s, cuda)
    out = matmul(x.to(cuda), wv, bias.to(cuda), rg, gather_indx=gather, scatter_indx=combine, gammas=gam.to(cuda),
                 precision_config=PrecisionConfig(b_mx_scale=ws), fused_activation=swiglu_activation(1.1, 7.0))
    ref = o.grouped_matmul_ref(x.float(), wdq, bias, mm.col_sum.cpu().numpy(), gather.cpu().numpy(),
                               combine.cpu().numpy(), gam, (1.1, 7.0), out_dtype=torch.bfloat16)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_argument_checks(cuda):
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    x = torch.zeros(128, 256, device=cuda, dtype=torch.float32)
    v = torch.zeros(1, 128, 128, device=cuda, dtype=torch.uint8)
    s = torch.full((1, 8, 128), 127, device=cuda, dtype=torch.uint8)
    with pytest.raises(NotImplementedError):
        matmul(x, v, None, precision_config=PrecisionConfig(b_mx_scale=s))  # fp32 activations


@pytest.mark.parametrize("swiglu", [False, True])
def test_more_tiles_than_sms(cuda, swiglu):
    """Several tiles per CTA (the persistent loop: the accumulator handed from one tile's epilogue to the next tile's
    MMAs): 6000 rows on 8 experts x 1024 columns = about 200 work units on 148 CTAs, every output checked."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    E, K, N = 8, 384, 1024
    g = torch.Generator().manual_seed(21)
    cnt = torch.tensor([900, 0, 1300, 128, 1, 1671, 1000, 1000], dtype=torch.int32)
    R = int(cnt.sum())
    rg = make_ragged_tensor_metadata(cnt.to(cuda), R)
    x = (torch.randn(R, K, generator=g) * 0.5).to(torch.float8_e4m3fn)
    v, s_, wdq = _quantise(0.3 * torch.randn(E, K, N, generator=g))
    gam = torch.rand(R, generator=g)
    out = matmul(x.to(cuda), v.to(cuda), None, rg, gammas=gam.to(cuda),
                 precision_config=PrecisionConfig(b_mx_scale=s_.to(cuda), out_dtype=torch.bfloat16),
                 fused_activation=swiglu_activation(1.1, 7.0) if swiglu else None)
    ref = o.grouped_matmul_ref(x.float(), wdq, None, cnt.numpy(), gammas=gam, swiglu=(1.1, 7.0) if swiglu else None,
                               out_dtype=torch.float32)
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-2, atol=2e-2)
    # the same call twice: identical bits (no dependence on which CTA got which tile)
    out2 = matmul(x.to(cuda), v.to(cuda), None, rg, gammas=gam.to(cuda),
                  precision_config=PrecisionConfig(b_mx_scale=s_.to(cuda), out_dtype=torch.bfloat16),
                  fused_activation=swiglu_activation(1.1, 7.0) if swiglu else None)
    assert torch.equal(out, out2)
