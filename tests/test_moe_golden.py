"""The CUDA MoE path against outputs of the reference's own torch twins (tests/golden/moe_cases.npz,
produced by tests/golden/make_moe_fixture.py from the reference checkout): routing indices, bitmatrix
and metadata bit-exact; values within the reference's matmul tolerance (maxtol 2e-2)."""
import os

import numpy as np
import pytest
import torch

from oracle import moe as o

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def fx():
    return np.load(os.path.join(GOLDEN, "moe_cases.npz"))


@pytest.mark.parametrize("name", ["plain", "ties", "padded", "nosoftmax", "bf16"])
def test_topk_matches_reference_twin(cuda, fx, name):
    from triton_b200.triton_kernels.topk import topk
    n_rows, softmax, is_bf16 = (int(v) for v in fx[f"topk_{name}_kw"])
    x = torch.from_numpy(fx[f"topk_{name}_x"])
    if is_bf16:
        x = x.to(torch.bfloat16)
    sm = topk(x.to(cuda), 4, apply_softmax=bool(softmax), n_rows=n_rows if n_rows != x.shape[0] else None)
    assert np.array_equal(sm.indx.cpu().int().numpy(), fx[f"topk_{name}_indx"])
    assert np.array_equal(sm.mask.data.cpu().contiguous().numpy(), fx[f"topk_{name}_bits"])
    tol = dict(rtol=1e-2, atol=1e-3) if is_bf16 else dict(rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(sm.vals.cpu().float().numpy()[:n_rows], fx[f"topk_{name}_vals"][:n_rows], **tol)


def test_topk_with_provided_indices_matches_reference_twin(cuda, fx):
    from triton_b200.triton_kernels.topk import topk
    x = torch.from_numpy(fx["topk_given_x"]).to(cuda)
    given = torch.from_numpy(fx["topk_given_yin"]).to(cuda)
    sm = topk(x, 4, y_indx=given)
    assert np.array_equal(sm.indx.cpu().int().numpy(), fx["topk_given_indx"])
    assert np.array_equal(sm.mask.data.cpu().contiguous().numpy(), fx["topk_given_bits"])
    np.testing.assert_allclose(sm.vals.cpu().numpy(), fx["topk_given_vals"], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("name", ["plain", "ties", "padded"])
def test_bitmatrix_metadata_matches_reference_twin(cuda, fx, name):
    from triton_b200.triton_kernels.tensor import Bitmatrix, make_bitmatrix_metadata
    indx = torch.from_numpy(fx[f"topk_{name}_indx"]).to(torch.int16).to(cuda)
    md = make_bitmatrix_metadata(indx, Bitmatrix(None, shape=[indx.shape[0], 128]))
    assert np.array_equal(md.col_sum.cpu().numpy(), fx[f"bm_{name}_col_sum"])
    assert np.array_equal(md.col_sorted_indx.cpu().numpy(), fx[f"bm_{name}_col_sorted"])
    assert np.array_equal(md.row_sorted_indx.cpu().numpy(), fx[f"bm_{name}_row_sorted"])


@pytest.mark.parametrize("name", ["doc", "mixed", "routing", "empty"])
def test_ragged_metadata_matches_reference_twin(cuda, fx, name):
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata, remap_ragged_tensor_metadata
    ss = torch.from_numpy(fx[f"rg_{name}_slice_sizes"]).to(cuda)
    md = make_ragged_tensor_metadata(ss, int(ss.sum()))
    assert np.array_equal(md.slice_offs.cpu().numpy(), fx[f"rg_{name}_slice_offs"])
    assert np.array_equal(md.block_offs_data.cpu().numpy(), fx[f"rg_{name}_block_offs"])
    assert np.array_equal(md.block_schedule_data.cpu().numpy(), fx[f"rg_{name}_block_sched"])
    if f"rg_{name}_map" in fx:
        rm = remap_ragged_tensor_metadata(md, torch.from_numpy(fx[f"rg_{name}_map"]).to(cuda))
        assert np.array_equal(rm.slice_sizes.cpu().numpy(), fx[f"rg_{name}_re_slice_sizes"])
        assert np.array_equal(rm.slice_offs.cpu().numpy(), fx[f"rg_{name}_re_slice_offs"])
        assert np.array_equal(rm.block_offs_data.cpu().numpy(), fx[f"rg_{name}_re_block_offs"])
        assert np.array_equal(rm.block_schedule_data.cpu().numpy(), fx[f"rg_{name}_re_block_sched"])


def test_grouped_matmul_matches_reference_twin(cuda, fx):
    """matmul_torch's outputs for the gather / bias / gammas / scatter (-1 rows dropped) combinations and
    swiglu_torch on top; the kernels run in bf16, the twin's fp32 result is the target (maxtol 2e-2)."""
    from triton_b200.triton_kernels.matmul import matmul, swiglu_activation
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    bf = torch.bfloat16
    a, w = torch.from_numpy(fx["mm_a"]).to(bf).to(cuda), torch.from_numpy(fx["mm_w"]).to(bf).to(cuda)
    bias, gam = torch.from_numpy(fx["mm_bias"]).to(cuda), torch.from_numpy(fx["mm_gammas"]).to(cuda)
    gather, scatter = torch.from_numpy(fx["mm_gather"]).to(cuda), torch.from_numpy(fx["mm_scatter"]).to(cuda)
    sizes = torch.from_numpy(fx["mm_sizes"]).to(cuda)
    rg = make_ragged_tensor_metadata(sizes, int(sizes.sum()))
    a_sorted = a[gather.long()]
    tol = dict(rtol=2e-2, atol=2e-2)

    def close(got, key):
        np.testing.assert_allclose(got.cpu().float().numpy(), fx[key], **tol)

    close(matmul(a_sorted, w, None, rg), "mm_y_plain")
    close(matmul(a, w, None, rg, gather_indx=gather), "mm_y_gather")
    close(matmul(a_sorted, w, bias, rg, gammas=gam), "mm_y_bias_gamma")
    dropped = torch.from_numpy(fx["mm_scatter"] == -1)
    y = torch.zeros(scatter.shape[0], w.shape[-1], dtype=bf, device=cuda)  # rows nothing maps to stay as they are
    close(matmul(a_sorted, w, None, rg, scatter_indx=scatter, gammas=gam, c=y), "mm_y_scatter")
    y = torch.zeros_like(y)
    close(matmul(a, w, bias, rg, gather_indx=gather, scatter_indx=scatter, gammas=gam, c=y), "mm_y_all")
    np.testing.assert_allclose(y.cpu().float().numpy(), fx["mm_y_all_bf16"], **tol)
    assert int(dropped.sum()) == 6
    for limit in (None, 1.4):
        got = matmul(a, w, bias, rg, gather_indx=gather, fused_activation=swiglu_activation(1.1, limit))
        close(got, f"mm_y_swiglu_{limit}")


def test_swiglu_and_reduce_match_reference_twins(cuda, fx):
    from triton_b200.triton_kernels.reduce import reduce
    from triton_b200.triton_kernels.swiglu import PrecisionConfig, swiglu
    x = torch.from_numpy(fx["sw_x"]).to(cuda)
    np.testing.assert_allclose(swiglu(x, 1.702, PrecisionConfig(None)).cpu().numpy(), fx["sw_y_None"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(swiglu(x, 1.702, PrecisionConfig(2.0)).cpu().numpy(), fx["sw_y_limit"], rtol=1e-5, atol=1e-6)
    xr = torch.from_numpy(fx["rd_x"]).to(torch.bfloat16).to(cuda)
    mask, sc = torch.from_numpy(fx["rd_mask"]).bool().to(cuda), torch.from_numpy(fx["rd_scale"]).to(cuda)
    tol = dict(rtol=1e-2, atol=1e-2)
    np.testing.assert_allclose(reduce(xr, 1)[0].cpu().float().numpy(), fx["rd_y_plain"], **tol)
    np.testing.assert_allclose(reduce(xr, 1, mask=mask)[0].cpu().float().numpy(), fx["rd_y_mask"], **tol)
    np.testing.assert_allclose(reduce(xr, 1, scale=sc)[0].cpu().float().numpy(), fx["rd_y_scale"], **tol)
    got = reduce(xr, 1, mask=mask, scale=sc)[0]
    np.testing.assert_allclose(got.cpu().float().numpy(), fx["rd_y_both_bf16"], rtol=2 ** -7, atol=2 ** -7)


def test_batched_matmul_matches_reference_twin(cuda, fx):
    """[B, M, K] x [B, K, N] + bias against matmul_torch's output (bf16 run of fp32 fixture values: the reference's
    bf16 tolerance), and a larger case against the oracle."""
    from triton_b200.triton_kernels.matmul import matmul, swiglu_activation
    d = fx
    a, w, bias = (torch.from_numpy(d[k]) for k in ("bt_a", "bt_w", "bt_bias"))
    y = matmul(a.to(torch.bfloat16).to(cuda), w.to(torch.bfloat16).to(cuda), bias.to(cuda))
    assert y.shape == (3, 10, 24)
    torch.testing.assert_close(y.cpu().float(), torch.from_numpy(d["bt_y"]), rtol=2e-2, atol=2e-2)
    g = torch.Generator().manual_seed(5)
    a = torch.randn(4, 200, 192, generator=g).to(torch.bfloat16)
    w = (0.1 * torch.randn(4, 192, 320, generator=g)).to(torch.bfloat16)
    y = matmul(a.to(cuda), w.to(cuda), None, fused_activation=swiglu_activation(1.0, None))
    ref = o.batched_matmul_ref(a, w, None, swiglu=(1.0, None))
    torch.testing.assert_close(y.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    with pytest.raises(ValueError):
        matmul(a.to(cuda), w.to(cuda), None, gather_indx=torch.zeros(4, dtype=torch.int32, device=cuda))


def test_ragged_k_matmul_matches_reference_twin(cuda, fx):
    """b_ragged_metadata: out[e] = a[:, ks_e] @ b[ks_e, :] against matmul_torch's output (one empty slice), and a
    larger case (K slices of 128 .. 512, one empty) against the oracle."""
    from triton_b200.triton_kernels.matmul import matmul
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    d = fx
    a, w = torch.from_numpy(d["rk_a"]), torch.from_numpy(d["rk_w"])
    ks = torch.from_numpy(d["rk_sizes"]).to(cuda)
    md = make_ragged_tensor_metadata(ks, int(ks.sum()))
    y = matmul(a.to(torch.bfloat16).to(cuda), w.to(torch.bfloat16).to(cuda), None, md, md)
    assert y.shape == (4, 12, 20)
    torch.testing.assert_close(y.cpu().float(), torch.from_numpy(d["rk_y"]), rtol=2e-2, atol=2e-2)
    assert float(y[1].abs().max()) == 0.0
    g = torch.Generator().manual_seed(6)
    sizes = torch.tensor([256, 0, 128, 512, 136], dtype=torch.int32)
    K = int(sizes.sum())
    a = torch.randn(300, K, generator=g).to(torch.float16)
    w = (0.1 * torch.randn(K, 264, generator=g)).to(torch.float16)
    md = make_ragged_tensor_metadata(sizes.to(cuda), K)
    y = matmul(a.to(cuda), w.to(cuda), None, md, md)
    ref = o.ragged_k_matmul_ref(a, w, sizes.numpy())
    torch.testing.assert_close(y.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    bad = make_ragged_tensor_metadata(torch.tensor([5, K - 5], dtype=torch.int32, device=cuda), K)
    with pytest.raises(NotImplementedError):  # the second slice starts at element 5
        matmul(a.to(cuda), w.to(cuda), None, bad, bad)


def test_fp8_flexpoint_matmul_matches_reference_twin(cuda, fx):
    """float8_e5m2 x float8_e5m2, grouped, with lhs / rhs / expected scales and gate weights against matmul_torch's
    output, and the actual_scale it computed. The kernel's output is e5m2 (2 mantissa bits): compared after
    dequantisation within one rounding step of the twin's fp32 result."""
    from triton_b200.triton_kernels.matmul import FlexCtx, PrecisionConfig, matmul
    from triton_b200.triton_kernels.numerics import InFlexData, OutFlexData
    from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
    d = fx
    a = torch.from_numpy(d["f8_a"]).view(torch.float8_e5m2)
    w = torch.from_numpy(d["f8_w"]).view(torch.float8_e5m2)
    sizes = torch.from_numpy(d["f8_sizes"])
    ls, rs, es = (torch.tensor(float(v), device=cuda) for v in d["f8_scales"])
    actual = torch.zeros(1, device=cuda)
    fc = FlexCtx(lhs_data=InFlexData(scale=ls), rhs_data=InFlexData(scale=rs),
                 out_data=OutFlexData(expected_scale=es, actual_scale=actual))
    md = make_ragged_tensor_metadata(sizes.to(cuda), int(sizes.sum()))
    wk = w.transpose(1, 2).contiguous().transpose(1, 2).to(cuda)  # K contiguous, as the reference stores fp8 weights
    y = matmul(a.to(cuda), wk, None, md, gammas=torch.from_numpy(d["f8_gammas"]).to(cuda),
               precision_config=PrecisionConfig(flex_ctx=fc))
    assert y.dtype == torch.float8_e5m2
    ref = torch.from_numpy(d["f8_y"])
    err = (y.cpu().float() - ref).abs()
    assert float((err / ref.abs().clamp_min(2.0 ** -14)).max()) <= 0.126  # half an e5m2 step is 2^-3 relative
    assert abs(float(actual) - float(d["f8_actual"][0])) <= 1e-5 * float(d["f8_actual"][0]) + 1e-30
    # the same values with a bf16 output: the twin's tolerance for 16-bit outputs
    fc16 = FlexCtx(lhs_data=InFlexData(scale=ls), rhs_data=InFlexData(scale=rs), out_data=OutFlexData(expected_scale=es))
    y16 = matmul(a.to(cuda), wk, None, md, gammas=torch.from_numpy(d["f8_gammas"]).to(cuda),
                 precision_config=PrecisionConfig(flex_ctx=fc16, out_dtype=torch.bfloat16))
    torch.testing.assert_close(y16.cpu().float(), ref, rtol=2e-2, atol=2e-2)
