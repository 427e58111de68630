"""FP8 weights in ``triton_kernels.matmul.matmul``: float8 x float8 (plain, ragged and batched, with and without
flexpoint scales) and float8 / mxfloat8 x mxfloat8, the dtype pairs of the reference's test list
(tests/test_matmul.py:150,154,193,196,214-216,251-265), against the CPU oracle applied to the dequantised operands.

Products of two fp8 values are exact in fp32 and the sums differ from the oracle's only in their order, so what is
left is the rounding of the output type: rtol / atol 1e-2 for bf16, bit-exact for small integers; fp8 outputs are
compared after dequantisation with the reference's tolerance for fp8 (maxtol 2e-2 is for 16-bit outputs; an e5m2
value carries 2 mantissa bits: half a unit in the last place is 2^-3)."""
import pytest
import torch

from oracle import moe as o
from triton_b200.triton_kernels.numerics_details.mxfp import downcast_to_mxfp, upcast_from_mxfp

pytestmark = pytest.mark.gpu

F8 = [torch.float8_e4m3fn, torch.float8_e5m2]


def _col_major(w):
    """[E, K, N] with K contiguous: how the reference lays fp8 weights out (tests/test_matmul.py: the weight is
    transposed, made contiguous and transposed back when the dtype is 8 bits wide)."""
    return w.transpose(-1, -2).contiguous().transpose(-1, -2)


@pytest.mark.parametrize("shape", [(300, 400, 400), (1000, 400, 400), (128, 256, 128), (300, 400, 416), (16, 256, 256),
                                   (1, 16, 16), (1024, 1024, 1024)])
@pytest.mark.parametrize("dtype", F8)
def test_dense_fp8_x_fp8(cuda, shape, dtype):
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    M, N, K = shape
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(M, K, generator=g) * 0.5).to(dtype)
    w = (torch.randn(K, N, generator=g) * 0.5).to(dtype)
    out = matmul(x.to(cuda), _col_major(w).to(cuda), None, precision_config=PrecisionConfig(out_dtype=torch.bfloat16))
    assert out.dtype == torch.bfloat16 and out.shape == (M, N)
    torch.testing.assert_close(out.cpu().float(), x.float() @ w.float(), rtol=1e-2, atol=1e-2)
    # N-contiguous weights are re-laid by the wrapper: same result
    out2 = matmul(x.to(cuda), w.to(cuda), None, precision_config=PrecisionConfig(out_dtype=torch.bfloat16))
    assert torch.equal(out.cpu(), out2.cpu())


def test_exact_on_small_integers(cuda):
    """Integers in [-3, 3]: every partial sum is exact, the fp16 output must equal the oracle's bit for bit (mixed
    e4m3 activations x e5m2 weights; K and N with tails)."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    M, N, K = 200, 272, 400
    g = torch.Generator().manual_seed(2)
    x = torch.randint(-3, 4, (M, K), generator=g).float().to(torch.float8_e4m3fn)
    w = torch.randint(-3, 4, (K, N), generator=g).float().to(torch.float8_e5m2)
    out = matmul(x.to(cuda), _col_major(w).to(cuda), None, precision_config=PrecisionConfig(out_dtype=torch.float16))
    assert torch.equal(out.cpu(), (x.float() @ w.float()).to(torch.float16))


def test_default_output_is_fp8(cuda):
    """Without out_dtype the output has the activations' dtype, as in the reference (matmul.py:243 allocates
    ``a.dtype``); values round to nearest even and saturate."""
    from triton_b200.triton_kernels.matmul import matmul
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(64, 128, generator=g) * 0.25).to(torch.float8_e4m3fn)
    w = (torch.randn(128, 128, generator=g) * 0.25).to(torch.float8_e4m3fn)
    out = matmul(x.to(cuda), _col_major(w).to(cuda), None)
    assert out.dtype == torch.float8_e4m3fn
    ref = (x.float() @ w.float()).clamp(-448, 448).to(torch.float8_e4m3fn)
    d = (out.cpu().float() - ref.float()).abs()
    assert float((d / ref.float().abs().clamp_min(2.0 ** -6)).max()) <= 0.13  # at most one e4m3 step where a sum sits on a tie


@pytest.mark.parametrize("dtype", F8)
@pytest.mark.parametrize("swiglu", [False, True])
def test_grouped_fp8_gather_scatter(cuda, dtype, swiglu):
    """The MoE call: rows gathered per expert, bias, (SwiGLU), gate weights, scatter."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    from triton_b200.triton_kernels.topk import topk
    T, E, k, K, N = 333, 8, 2, 272, 400
    g = torch.Generator().manual_seed(4)
    sm = topk(torch.randn(T, E, generator=g).to(cuda), k)
    mm = sm.mask_metadata
    R = T * k
    rg = make_ragged_tensor_metadata(mm.col_sum, R)
    combine = mm.col_sorted_indx
    gather = torch.div(combine, k, rounding_mode="trunc")
    x = (torch.randn(T, K, generator=g) * 0.5).to(dtype)
    w = (torch.randn(E, K, N, generator=g) * 0.25).to(dtype)
    bias = torch.randn(E, N, generator=g)
    gam = torch.rand(R, generator=g)
    out = matmul(x.to(cuda), _col_major(w).to(cuda), bias.to(cuda), rg, gather_indx=gather, scatter_indx=combine,
                 gammas=gam.to(cuda), precision_config=PrecisionConfig(out_dtype=torch.bfloat16),
                 fused_activation=swiglu_activation(1.1, 7.0) if swiglu else None)
    ref = o.grouped_matmul_ref(x.float(), w.float(), bias, mm.col_sum.cpu().numpy(), gather_indx=gather.cpu().numpy(),
                               scatter_indx=combine.cpu().numpy(), gammas=gam, swiglu=(1.1, 7.0) if swiglu else None,
                               out_dtype=torch.float32)
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-2, atol=2e-2)


def test_more_tiles_than_sms(cuda):
    """Several tiles per CTA with fp8 weights: 5000 rows x 1280 columns = 200 work units on 148 CTAs."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    g = torch.Generator().manual_seed(13)
    x = (torch.randn(5000, 272, generator=g) * 0.5).to(torch.float8_e4m3fn)
    w = (torch.randn(272, 1280, generator=g) * 0.5).to(torch.float8_e4m3fn)
    out = matmul(x.to(cuda), _col_major(w).to(cuda), None, precision_config=PrecisionConfig(out_dtype=torch.bfloat16))
    torch.testing.assert_close(out.cpu().float(), x.float() @ w.float(), rtol=1e-2, atol=1e-2)


def test_preallocated_output(cuda):
    """``c=``: the product lands in the caller's buffer (a row-strided view here) and that tensor is returned."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    g = torch.Generator().manual_seed(12)
    x = (torch.randn(96, 128, generator=g) * 0.5).to(torch.float8_e4m3fn)
    w = (torch.randn(128, 144, generator=g) * 0.5).to(torch.float8_e4m3fn)
    buf = torch.full((96, 160), 7.0, dtype=torch.bfloat16, device=cuda)
    out = matmul(x.to(cuda), _col_major(w).to(cuda), None, precision_config=PrecisionConfig(out_dtype=torch.bfloat16),
                 c=buf[:, :144])
    assert out.data_ptr() == buf.data_ptr()
    torch.testing.assert_close(buf[:, :144].cpu().float(), x.float() @ w.float(), rtol=1e-2, atol=1e-2)
    assert float((buf[:, 144:].float() - 7.0).abs().max()) == 0.0


def test_batched_fp8(cuda):
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    B, M, K, N = 3, 300, 416, 400
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(B, M, K, generator=g) * 0.5).to(torch.float8_e5m2)
    w = (torch.randn(B, K, N, generator=g) * 0.5).to(torch.float8_e5m2)
    out = matmul(x.to(cuda), _col_major(w).to(cuda), None, precision_config=PrecisionConfig(out_dtype=torch.bfloat16))
    assert out.shape == (B, M, N)
    torch.testing.assert_close(out.cpu().float(), torch.bmm(x.float(), w.float()), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("saturate", [False, True])
def test_flexpoint_scales(cuda, saturate):
    """lhs / rhs scales multiply the product, expected_scale divides the output, actual_scale receives
    max |output| / max_finite (numerics_details/flexpoint.py:133-188 in the reference)."""
    from triton_b200.triton_kernels.matmul import FlexCtx, PrecisionConfig, matmul
    from triton_b200.triton_kernels.numerics import InFlexData, OutFlexData
    M, N, K = 256, 384, 256
    g = torch.Generator().manual_seed(6)
    x = torch.randn(M, K, generator=g).to(torch.float8_e5m2)
    w = torch.randn(K, N, generator=g).to(torch.float8_e5m2)
    ls, rs, es = 0.5, 0.25, 0.03125
    actual = torch.zeros(1, device=cuda)
    fc = FlexCtx(lhs_data=InFlexData(scale=torch.tensor(ls, device=cuda)),
                 rhs_data=InFlexData(scale=torch.tensor(rs, device=cuda)),
                 out_data=OutFlexData(expected_scale=torch.tensor(es, device=cuda), actual_scale=actual))
    out = matmul(x.to(cuda), _col_major(w).to(cuda), None,
                 precision_config=PrecisionConfig(flex_ctx=fc, flexpoint_saturate_inf=saturate))
    assert out.dtype == torch.float8_e5m2
    y = (x.float() @ w.float()) * (ls * rs)
    assert abs(float(actual) - o.flex_actual_scale_ref(y, torch.float8_e5m2)) <= 1e-6 * float(actual)
    ref = y / es
    if saturate:
        ref = ref.clamp(-57344, 57344)
    got = out.cpu().float()
    finite = ref.abs() <= 57344
    assert torch.isfinite(got[finite]).all()
    rel = ((got - ref).abs() / ref.abs().clamp_min(1.0))[finite]
    assert float(rel.max()) <= 0.13  # e5m2: 2 mantissa bits


@pytest.mark.parametrize("mx_act", [False, True])
@pytest.mark.parametrize("shape", [(300, 400, 416), (128, 256, 256)])
def test_mxfp8_weights(cuda, mx_act, shape):
    """float8 x mxfloat8 and mxfloat8 x mxfloat8 (tests/test_matmul.py:193,214): e4m3 weights with one e8m0 scale per
    32 values of K, grouped over three experts."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    M, N, K = shape
    E = 3
    g = torch.Generator().manual_seed(7)
    cnt = torch.tensor([M - 100, 0, 100], dtype=torch.int32)
    rg = make_ragged_tensor_metadata(cnt.to(cuda), M)
    wv, ws = downcast_to_mxfp((0.3 * torch.randn(E, K, N, generator=g)).to(torch.bfloat16), torch.float8_e4m3fn, axis=1)
    wdq = upcast_from_mxfp(wv, ws, torch.float32, axis=1)
    if mx_act:
        xv, xs = downcast_to_mxfp(torch.randn(M, K, generator=g).to(torch.bfloat16), torch.float8_e4m3fn, axis=1)
        xdq = upcast_from_mxfp(xv, xs, torch.float32, axis=1)
        pc = PrecisionConfig(a_mx_scale=xs.to(cuda), a_microblock_size=32, b_mx_scale=ws.to(cuda), b_microblock_size=32,
                             out_dtype=torch.bfloat16)
    else:
        xv = (torch.randn(M, K, generator=g) * 0.5).to(torch.float8_e5m2)
        xdq = xv.float()
        pc = PrecisionConfig(b_mx_scale=ws.to(cuda), b_microblock_size=32, out_dtype=torch.bfloat16)
    out = matmul(xv.to(cuda), _col_major(wv).to(cuda), None, rg, precision_config=pc)
    ref = o.grouped_matmul_ref(xdq, wdq, None, cnt.numpy(), out_dtype=torch.float32)
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1e-2, atol=2e-2)


def test_batched_fp8_x_mxfp8_weights(cuda):
    """float8_e5m2 x mxfloat8_e4m3fn, batched (tests/test_matmul.py:196)."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    B, M, K, N = 2, 300, 416, 400
    g = torch.Generator().manual_seed(9)
    wv, ws = downcast_to_mxfp((0.3 * torch.randn(B, K, N, generator=g)).to(torch.bfloat16), torch.float8_e4m3fn, axis=1)
    wdq = upcast_from_mxfp(wv, ws, torch.float32, axis=1)
    x = (torch.randn(B, M, K, generator=g) * 0.5).to(torch.float8_e5m2)
    out = matmul(x.to(cuda), _col_major(wv).to(cuda), None,
                 precision_config=PrecisionConfig(b_mx_scale=ws.to(cuda), out_dtype=torch.bfloat16))
    torch.testing.assert_close(out.cpu().float(), torch.bmm(x.float(), wdq), rtol=1e-2, atol=2e-2)


@pytest.mark.parametrize("swiglu", [False, True])
def test_mxfp8_x_mxfp8_moe_call_with_quantised_output(cuda, swiglu):
    """The whole MoE call on MXFP8 operands: rows (and their block scales) gathered per expert, (SwiGLU), gate
    weights, scatter, MX-quantised output; compared as the reference compares quantised outputs (dequantise both
    sides, maxtol 4e-1, rmstol 4e-2, tests/test_matmul.py:604-625)."""
    from triton_b200.triton_kernels.matmul import Epilogue, FnName, FnSpecs, PrecisionConfig, matmul, swiglu_activation
    from triton_b200.triton_kernels.numerics_details.mxfp import quantize_mxfp8_fn
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    from triton_b200.triton_kernels.topk import topk
    T, E, k, K, N = 200, 8, 2, 256, 512
    g = torch.Generator().manual_seed(10)
    sm = topk(torch.randn(T, E, generator=g).to(cuda), k)
    mm = sm.mask_metadata
    R = T * k
    rg = make_ragged_tensor_metadata(mm.col_sum, R)
    combine = mm.col_sorted_indx
    gather = torch.div(combine, k, rounding_mode="trunc")
    xv, xs = downcast_to_mxfp(torch.randn(T, K, generator=g).to(torch.bfloat16), torch.float8_e4m3fn, axis=1)
    wv, ws = downcast_to_mxfp((0.3 * torch.randn(E, K, N, generator=g)).to(torch.bfloat16), torch.float8_e4m3fn, axis=1)
    xdq, wdq = upcast_from_mxfp(xv, xs, torch.float32, axis=1), upcast_from_mxfp(wv, ws, torch.float32, axis=1)
    gam = torch.rand(R, generator=g)
    n_out = N // 2 if swiglu else N
    c_scale = torch.zeros((R, n_out // 32), dtype=torch.uint8, device=cuda)
    pc = PrecisionConfig(a_mx_scale=xs.to(cuda), a_microblock_size=32, b_mx_scale=ws.to(cuda), b_microblock_size=32,
                         c_mx_scale=c_scale)
    epi = Epilogue(FnSpecs(FnName.QUANTIZE_MXFP8.name, quantize_mxfp8_fn, (), ()), tuple(), tuple(), 6.0)
    out = matmul(xv.to(cuda), _col_major(wv).to(cuda), None, rg, gather_indx=gather, scatter_indx=combine,
                 gammas=gam.to(cuda), precision_config=pc, fused_activation=swiglu_activation(1.1, 7.0) if swiglu else None,
                 epilogue=epi)
    assert out.dtype == torch.float8_e4m3fn and out.shape == (R, n_out)
    ref = o.grouped_matmul_ref(xdq, wdq, None, mm.col_sum.cpu().numpy(), gather_indx=gather.cpu().numpy(),
                               scatter_indx=combine.cpu().numpy(), gammas=gam, swiglu=(1.1, 7.0) if swiglu else None,
                               out_dtype=torch.float32)
    got = o.dequantize_mxfp8_ref(out.cpu(), c_scale.cpu())
    q_ref, s_ref = o.quantize_mxfp8_ref(ref)
    want = o.dequantize_mxfp8_ref(q_ref, s_ref)
    assert float((got - want).abs().max() / want.abs().max().clamp_min(1e-6)) <= 4e-1
    assert float(torch.sqrt(((got - want) ** 2).mean()) / torch.sqrt((want ** 2).mean()).clamp_min(1e-6)) <= 4e-2


@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float16])
def test_mxfp8_activations_x_16bit_weights(cuda, wdtype):
    """mxfloat8 x bfloat16 / float16 (tests/test_matmul.py:217-224): the activations are upcast to the weights' dtype and the
    16-bit kernel runs; the output has that dtype."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    E, K, N = 3, 96, 128
    g = torch.Generator().manual_seed(11)
    cnt = torch.tensor([40, 0, 24], dtype=torch.int32)
    rg = make_ragged_tensor_metadata(cnt.to(cuda), 64)
    xv, xs = downcast_to_mxfp(torch.randn(64, K, generator=g).to(torch.bfloat16), torch.float8_e4m3fn, axis=1)
    xdq = upcast_from_mxfp(xv, xs, torch.float32, axis=1)
    w = (0.3 * torch.randn(E, K, N, generator=g)).to(wdtype)
    out = matmul(xv.to(cuda), w.to(cuda), None, rg, precision_config=PrecisionConfig(a_mx_scale=xs.to(cuda)))
    assert out.dtype == wdtype
    ref = o.grouped_matmul_ref(xdq, w.float(), None, cnt.numpy(), out_dtype=torch.float32)
    torch.testing.assert_close(out.cpu().float(), ref, rtol=2e-2, atol=2e-2)


def test_bf16_x_mxfp8_weights(cuda):
    """bfloat16 x mxfloat8 (tests/test_matmul.py:177): the weight is upcast to bf16, then the 16-bit kernel runs."""
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    E, K, N = 3, 416, 400
    g = torch.Generator().manual_seed(8)
    cnt = torch.tensor([200, 0, 100], dtype=torch.int32)
    rg = make_ragged_tensor_metadata(cnt.to(cuda), 300)
    wv, ws = downcast_to_mxfp((0.3 * torch.randn(E, K, N, generator=g)).to(torch.bfloat16), torch.float8_e4m3fn, axis=1)
    wdq = upcast_from_mxfp(wv, ws, torch.float32, axis=1)
    x = torch.randn(300, K, generator=g).to(torch.bfloat16)
    out = matmul(x.to(cuda), wv.to(cuda), None, rg, precision_config=PrecisionConfig(b_mx_scale=ws.to(cuda)))
    ref = o.grouped_matmul_ref(x.float(), wdq, None, cnt.numpy(), out_dtype=torch.float32)
    assert out.dtype == torch.bfloat16
    torch.testing.assert_close(out.cpu().float(), ref, rtol=2e-2, atol=2e-2)


def test_argument_checks(cuda):
    from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul
    x = torch.zeros(64, 72, device=cuda).to(torch.float8_e4m3fn)
    w = torch.zeros(72, 64, device=cuda).to(torch.float8_e4m3fn)
    with pytest.raises(NotImplementedError):  # K must be a multiple of 16 (the rows of a tensor map)
        matmul(x, w, None)
    x = torch.zeros(64, 64, device=cuda).to(torch.float8_e4m3fn)
    w = torch.zeros(64, 64, device=cuda).to(torch.float8_e4m3fn)
    with pytest.raises(NotImplementedError):
        matmul(x, w, None, betas=torch.ones(64, device=cuda))
    with pytest.raises(NotImplementedError):  # MX-scaled activations need MX-scaled weights
        matmul(x, w, None, precision_config=PrecisionConfig(a_mx_scale=torch.zeros(64, 2, dtype=torch.uint8, device=cuda)))
