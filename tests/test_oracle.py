"""Pins the CPU oracle against the reference's own golden material (no GPU needed)."""
import os

import numpy as np
import torch

from oracle import attention as o_attn
from oracle import gemm as o_gemm
from oracle import moe as o_moe
from oracle import mxfp8 as o_mx

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_gemm_oracle_matches_reference_interpreter_fixture():
    """tests/golden/gemm_interp_512.npz holds rows of C produced by the reference's tutorial-03
    Triton kernel under TRITON_INTERPRET=1 (fp16 inputs, seed 0). fp16 output: tolerance 2 fp16
    ulps of the row magnitude (the kernel accumulates K in blocks of 32, the oracle in one go)."""
    fx = np.load(os.path.join(GOLDEN, "gemm_interp_512.npz"))
    torch.manual_seed(int(fx["seed"]))
    a = torch.randn(512, 512).to(torch.float16)
    b = torch.randn(512, 512).to(torch.float16)
    c = o_gemm.gemm_ref(a, b)
    rows = fx["rows"].tolist()
    got = c[rows].float().numpy()
    want = fx["c_rows"].astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=2e-3, atol=0.0625)
    assert abs(float(c.double().sum()) - float(fx["c_sum"])) < 1e-3 * float(fx["c_abs_sum"])


def test_bitmatrix_metadata_docstring_example():
    # reference: tensor_details/bitmatrix.py:10-19
    bm = np.array([[0, 0, 1, 0, 1, 1, 0], [0, 1, 0, 0, 0, 1, 0], [1, 1, 1, 0, 0, 0, 1], [0, 0, 1, 0, 1, 0, 0]])
    flat = np.concatenate([np.nonzero(r)[0] for r in bm])
    md = o_moe.bitmatrix_metadata_ref(flat, 7)
    assert md.col_sum.tolist() == [1, 2, 3, 0, 2, 2, 1]
    assert md.col_sorted_indx.tolist() == [5, 3, 6, 0, 7, 9, 1, 10, 2, 4, 8]
    assert md.row_sorted_indx.tolist() == [3, 6, 8, 1, 9, 0, 2, 4, 10, 5, 7]


def test_ragged_metadata_docstring_example():
    # reference: tensor_details/ragged_tensor.py:14-30 (block_offs are the self-consistent part of
    # that example: slice_offs' last entry and the schedule rows in it do not add up)
    md = o_moe.ragged_metadata_ref([15, 17, 0, 127], 159)
    assert md.slice_offs.tolist()[:4] == [0, 15, 32, 32]
    assert md.block_offs_data.tolist() == [[0, 1, 3, 3, 11], [0, 1, 2, 2, 6], [0, 1, 2, 2, 4], [0, 1, 2, 2, 3]]
    s128 = md.block_schedule_data[3]
    assert s128[:3].tolist() == [(0 << 16) | 0, (0 << 16) | 1, (0 << 16) | 3]
    assert (s128[3:] == -1).all()
    s16 = md.block_schedule_data[0]
    assert s16[:4].tolist() == [0, 1, (1 << 16) | 1, 3] and s16[10] == (7 << 16) | 3


def test_n_blocks_formula():
    # reference: RaggedTensorMetadata.n_blocks, ragged_tensor.py:73-77 — an upper bound on the
    # number of blocks of any split of n rows into n_slices slices
    rng = np.random.default_rng(0)
    for _ in range(200):
        E = int(rng.integers(1, 40))
        n = int(rng.integers(0, 3000))
        bs = int(rng.choice([16, 32, 64, 128]))
        cuts = np.sort(rng.integers(0, n + 1, E - 1))
        sizes = np.diff(np.concatenate([[0], cuts, [n]]))
        assert int(np.sum((sizes + bs - 1) // bs)) <= o_moe.n_blocks(E, n, bs)


def test_remap_ragged_metadata():
    md = o_moe.ragged_metadata_ref([15, 17, 0, 127], 159)
    r = o_moe.remap_ragged_metadata_ref(md, np.array([-1, 0, 1, -1]))
    assert r.slice_sizes.tolist() == [17, 0, -1, -1]
    assert r.block_offs_data[0].tolist() == [1, 3, 2, -1, -1]
    assert r.block_schedule_data[0][:3].tolist() == [0, (1 << 16) | 0, -1]


def test_topk_ties_and_order():
    x = torch.tensor([[1.0, 3.0, 3.0, 2.0, 0.0], [5.0, 5.0, 5.0, 5.0, 5.0]])
    vals, indx, bits = o_moe.topk_ref(x, 2, apply_softmax=False)
    assert indx.tolist() == [[1, 2], [0, 1]]
    assert vals.tolist() == [[3.0, 3.0], [5.0, 5.0]]
    assert bits.view(torch.int32)[:, 0].tolist() == [0b110, 0b11]
    vals, indx, _ = o_moe.topk_ref(x, 3, apply_softmax=True)
    np.testing.assert_allclose(vals.sum(1).numpy(), 1.0, rtol=1e-6)


def test_scale_swizzle_roundtrip_and_atom_order():
    rows, ks = 256, 8
    s = torch.arange(rows * ks, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(rows, ks)
    flat = o_mx.swizzle_scales(s)
    assert torch.equal(o_mx.unswizzle_scales(flat, rows, ks), s)
    # 512-byte atom = [row % 32][row // 32 % 4][k % 4] (blackwell_scale.py:119-122)
    r, kk = 128 + 37, 6
    atom = ((r // 128) * (ks // 4) + kk // 4) * 512
    assert flat[atom + (r % 32) * 16 + ((r % 128) // 32) * 4 + kk % 4] == s[r, kk]


def test_mxfp8_dequant_known_values():
    q = torch.full((128, 32), 1.5).to(torch.float8_e4m3fn)
    s = torch.full((128, 1), 127 + 3, dtype=torch.uint8)
    s4 = torch.cat([s, s, s, s], dim=1)
    d = o_mx.dequantize(torch.cat([q, q, q, q], dim=1), o_mx.swizzle_scales(s4))
    assert torch.all(d == 12.0)


def test_scaled_mm_blockwise_oracle_equals_dequantised_matmul():
    """Blockwise scaling is the same as multiplying each operand element by its own block's scale first
    when scale_b is folded into B (the DeepSeek definition)."""
    torch.manual_seed(2)
    M, N, K = 64, 256, 384
    a, b = torch.randn(M, K), torch.randn(N, K)
    sa, sb = torch.rand(M, K // 128) + 0.5, torch.rand(N // 128, K // 128) + 0.5
    want = (a * sa.repeat_interleave(128, dim=1)) @ (b * sb.repeat_interleave(128, 0).repeat_interleave(128, 1)).t()
    got = o_gemm.scaled_mm_blockwise_ref(a, b, sa, sb, out_dtype=torch.float32)
    torch.testing.assert_close(got, want, atol=1e-4, rtol=1e-5)


def test_attention_oracle_matches_sdpa():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 2, 96, 32) for _ in range(3))
    for causal in (False, True):
        o, lse2 = o_attn.attention_ref(q, k, v, 0.3, causal)
        want = torch.nn.functional.scaled_dot_product_attention(q, k, v, scale=0.3, is_causal=causal)
        torch.testing.assert_close(o, want, atol=1e-5, rtol=1e-5)
        s = (q @ k.transpose(-1, -2)) * 0.3
        if causal:
            s = s.masked_fill(~torch.ones(96, 96, dtype=torch.bool).tril(), float("-inf"))
        torch.testing.assert_close(lse2, torch.logsumexp(s, -1) * 1.4426950408889634, atol=1e-5, rtol=1e-5)


def test_attention_bwd_oracle_matches_autograd():
    """The backward restatement against torch autograd through SDPA (the check the reference's own
    backward test uses, testing/test_correctness.py:919-1068)."""
    torch.manual_seed(3)
    for causal in (False, True):
        q, k, v = (torch.randn(1, 2, 80, 32, dtype=torch.float64, requires_grad=True) for _ in range(3))
        do = torch.randn(1, 2, 80, 32, dtype=torch.float64)
        out = torch.nn.functional.scaled_dot_product_attention(q, k, v, scale=0.5, is_causal=causal)
        out.backward(do)
        dq, dk, dv = o_attn.attention_bwd_ref(q, k, v, do, 0.5, causal)
        torch.testing.assert_close(dq, q.grad.float(), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(dk, k.grad.float(), atol=1e-5, rtol=1e-5)
        torch.testing.assert_close(dv, v.grad.float(), atol=1e-5, rtol=1e-5)


def test_moe_layer_oracle_is_dense_mixture():
    """With k = E every expert sees every token: the layer equals the dense gate-weighted sum."""
    torch.manual_seed(1)
    T, D, F, E = 24, 16, 8, 4
    x = torch.randn(T, D)
    logits = torch.randn(T, E)
    w1 = torch.randn(E, D, 2 * F) * 0.2
    w2 = torch.randn(E, F, D) * 0.2
    got = o_moe.moe_layer_ref(x, logits, w1, w2, k=E, alpha=1.0, limit=None)
    gate = torch.softmax(logits, -1)
    want = torch.zeros(T, D)
    for e in range(E):
        want += gate[:, e:e + 1] * (o_moe.swiglu_ref(x @ w1[e], 1.0) @ w2[e])
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)


# --------------------------------------------------------------------------------------------------
# MoE path: the oracle against outputs of the reference's own torch twins
# (tests/golden/moe_cases.npz, written by tests/golden/make_moe_fixture.py from the reference checkout)
# --------------------------------------------------------------------------------------------------

def _moe_fx():
    return np.load(os.path.join(GOLDEN, "moe_cases.npz"))


def test_topk_oracle_matches_reference_twin():
    """topk_torch (topk.py:144-185): indices and bitmatrix bit-exact, values to 1e-6; covers ties,
    padded rows (n_rows), no softmax and bf16 logits."""
    fx = _moe_fx()
    for name in ("plain", "ties", "padded", "nosoftmax", "bf16"):
        n_rows, softmax, is_bf16 = (int(v) for v in fx[f"topk_{name}_kw"])
        x = torch.from_numpy(fx[f"topk_{name}_x"])
        if is_bf16:
            x = x.to(torch.bfloat16)
        vals, indx, bits = o_moe.topk_ref(x, 4, apply_softmax=bool(softmax), n_rows=n_rows)
        assert np.array_equal(indx.numpy(), fx[f"topk_{name}_indx"]), name
        assert np.array_equal(bits.numpy(), fx[f"topk_{name}_bits"]), name
        np.testing.assert_allclose(vals.float().numpy()[:n_rows], fx[f"topk_{name}_vals"][:n_rows], rtol=1e-6, atol=1e-7)


def test_bitmatrix_metadata_oracle_matches_reference_twin():
    """make_bitmatrix_metadata_torch (tensor_details/bitmatrix.py:157-168), bit-exact."""
    fx = _moe_fx()
    for name in ("plain", "ties", "padded"):
        md = o_moe.bitmatrix_metadata_ref(fx[f"topk_{name}_indx"], 128)
        assert np.array_equal(md.col_sum, fx[f"bm_{name}_col_sum"])
        assert np.array_equal(md.col_sorted_indx, fx[f"bm_{name}_col_sorted"])
        assert np.array_equal(md.row_sorted_indx, fx[f"bm_{name}_row_sorted"])


def test_ragged_metadata_oracle_matches_reference_twin():
    """make_ragged_tensor_metadata_torch and remap_ragged_tensor_metadata_torch
    (tensor_details/ragged_tensor.py:217-253, 388-433), bit-exact."""
    fx = _moe_fx()
    for name in ("doc", "mixed", "routing", "empty"):
        ss = fx[f"rg_{name}_slice_sizes"]
        md = o_moe.ragged_metadata_ref(ss, int(ss.sum()))
        assert np.array_equal(md.slice_offs, fx[f"rg_{name}_slice_offs"]), name
        assert np.array_equal(md.block_offs_data, fx[f"rg_{name}_block_offs"]), name
        assert np.array_equal(md.block_schedule_data, fx[f"rg_{name}_block_sched"]), name
        if f"rg_{name}_map" in fx:
            rm = o_moe.remap_ragged_metadata_ref(md, fx[f"rg_{name}_map"])
            assert np.array_equal(rm.slice_sizes, fx[f"rg_{name}_re_slice_sizes"]), name
            assert np.array_equal(rm.slice_offs, fx[f"rg_{name}_re_slice_offs"]), name
            assert np.array_equal(rm.block_offs_data, fx[f"rg_{name}_re_block_offs"]), name
            assert np.array_equal(rm.block_schedule_data, fx[f"rg_{name}_re_block_sched"]), name


def test_grouped_matmul_oracle_matches_reference_twin():
    """matmul_torch (matmul.py:823-914) with gather, scatter incl. -1, gammas and bias, and
    swiglu_torch applied to its result; fp32 holders of bf16 values, so 1e-5 is rounding of the sums."""
    fx = _moe_fx()
    a, w = torch.from_numpy(fx["mm_a"]), torch.from_numpy(fx["mm_w"])
    bias, gam = torch.from_numpy(fx["mm_bias"]), torch.from_numpy(fx["mm_gammas"])
    sizes, gather, scatter = fx["mm_sizes"], fx["mm_gather"], fx["mm_scatter"]
    a_sorted = a[torch.from_numpy(gather).long()]
    tol = dict(rtol=1e-5, atol=1e-5)
    f32 = torch.float32
    got = o_moe.grouped_matmul_ref(a_sorted, w, None, sizes, out_dtype=f32)
    np.testing.assert_allclose(got.numpy(), fx["mm_y_plain"], **tol)
    got = o_moe.grouped_matmul_ref(a, w, None, sizes, gather_indx=gather, out_dtype=f32)
    np.testing.assert_allclose(got.numpy(), fx["mm_y_gather"], **tol)
    got = o_moe.grouped_matmul_ref(a_sorted, w, bias, sizes, gammas=gam, out_dtype=f32)
    np.testing.assert_allclose(got.numpy(), fx["mm_y_bias_gamma"], **tol)
    got = o_moe.grouped_matmul_ref(a_sorted, w, None, sizes, scatter_indx=scatter, gammas=gam, out_dtype=f32)
    np.testing.assert_allclose(got.numpy(), fx["mm_y_scatter"], **tol)
    got = o_moe.grouped_matmul_ref(a, w, bias, sizes, gather_indx=gather, scatter_indx=scatter, gammas=gam, out_dtype=f32)
    np.testing.assert_allclose(got.numpy(), fx["mm_y_all"], **tol)
    for limit in (None, 1.4):
        got = o_moe.grouped_matmul_ref(a, w, bias, sizes, gather_indx=gather, swiglu=(1.1, limit), out_dtype=f32)
        np.testing.assert_allclose(got.numpy(), fx[f"mm_y_swiglu_{limit}"], **tol)
    # bf16 in, bf16 out: the twin rounds once per expert block, as the oracle does at the end
    got = o_moe.grouped_matmul_ref(a.to(torch.bfloat16), w.to(torch.bfloat16), bias, sizes, gather_indx=gather,
                                   scatter_indx=scatter, gammas=gam)
    np.testing.assert_allclose(got.float().numpy(), fx["mm_y_all_bf16"], rtol=0, atol=0)


def test_swiglu_and_reduce_oracles_match_reference_twins():
    """swiglu_torch (swiglu.py:89-100) with and without limit; reduce_torch (reduce.py:1173-1206)
    with mask and scale."""
    fx = _moe_fx()
    x = torch.from_numpy(fx["sw_x"])
    np.testing.assert_allclose(o_moe.swiglu_ref(x, 1.702, None).numpy(), fx["sw_y_None"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(o_moe.swiglu_ref(x, 1.702, 2.0).numpy(), fx["sw_y_limit"], rtol=1e-6, atol=1e-7)
    xr = torch.from_numpy(fx["rd_x"])
    mask, sc = torch.from_numpy(fx["rd_mask"]), torch.from_numpy(fx["rd_scale"])
    tol = dict(rtol=1e-6, atol=1e-6)
    np.testing.assert_allclose(o_moe.reduce_ref(xr, 1).numpy(), fx["rd_y_plain"], **tol)
    np.testing.assert_allclose(o_moe.reduce_ref(xr, 1, mask=mask).numpy(), fx["rd_y_mask"], **tol)
    np.testing.assert_allclose(o_moe.reduce_ref(xr, 1, scale=sc).numpy(), fx["rd_y_scale"], **tol)
    np.testing.assert_allclose(o_moe.reduce_ref(xr, 1, mask=mask, scale=sc).numpy(), fx["rd_y_both"], **tol)
    got = o_moe.reduce_ref(xr.to(torch.bfloat16), 1, mask=mask, scale=sc)
    np.testing.assert_allclose(got.float().numpy(), fx["rd_y_both_bf16"], rtol=0, atol=0)


def test_quantize_mxfp8_oracle_matches_reference_twin():
    """oracle.moe.quantize_mxfp8_ref against the outputs of the reference's downcast_to_mxfp_torch (e4m3 values,
    e8m0 scales, ROUND_UP) and upcast_from_mxfp_torch held in mxfp_cases.npz: bit-exact."""
    d = np.load(os.path.join(os.path.dirname(__file__), "golden", "mxfp_cases.npz"))
    for name in ("normal", "wide", "ties", "zeros"):
        x = torch.from_numpy(d[f"{name}_x"])
        q, s = o_moe.quantize_mxfp8_ref(x)
        assert np.array_equal(q.view(torch.uint8).numpy(), d[f"{name}_e4m3_ROUND_UP_v"]), name
        assert np.array_equal(s.numpy(), d[f"{name}_e4m3_ROUND_UP_s"]), name
        up = o_moe.dequantize_mxfp8_ref(q, s)
        assert np.array_equal(up.numpy(), d[f"{name}_e4m3_ROUND_UP_up"]), name


def test_batched_and_ragged_k_oracles_match_reference_twin():
    """oracle.moe.batched_matmul_ref / ragged_k_matmul_ref against matmul_torch outputs (batched inputs with bias;
    K-ragged slices with an empty slice) in moe_cases.npz."""
    d = np.load(os.path.join(GOLDEN, "moe_cases.npz"))
    t = lambda k: torch.from_numpy(d[k])
    y = o_moe.batched_matmul_ref(t("bt_a"), t("bt_w"), t("bt_bias"))
    torch.testing.assert_close(y, t("bt_y"), rtol=1e-5, atol=1e-5)
    y = o_moe.ragged_k_matmul_ref(t("rk_a"), t("rk_w"), d["rk_sizes"])
    torch.testing.assert_close(y, t("rk_y"), rtol=1e-5, atol=1e-5)
    assert float(y[1].abs().max()) == 0.0


def test_grouped_oracle_matches_reference_twin_on_fp8_flexpoint():
    """oracle.moe.grouped_matmul_ref on fp8 operands times their flexpoint scales, divided by expected_scale, and
    flex_actual_scale_ref, against matmul_torch's output for the float8_e5m2 case in moe_cases.npz."""
    d = np.load(os.path.join(GOLDEN, "moe_cases.npz"))
    a = torch.from_numpy(d["f8_a"]).view(torch.float8_e5m2).float()
    w = torch.from_numpy(d["f8_w"]).view(torch.float8_e5m2).float()
    ls, rs, es = (float(v) for v in d["f8_scales"])
    y = o_moe.grouped_matmul_ref(a * ls, w * rs, None, d["f8_sizes"], gammas=torch.from_numpy(d["f8_gammas"]),
                                 out_dtype=torch.float32)
    torch.testing.assert_close(y / es, torch.from_numpy(d["f8_y"]), rtol=1e-5, atol=1e-5)
    assert abs(o_moe.flex_actual_scale_ref(y, torch.float8_e5m2) - float(d["f8_actual"][0])) <= 1e-6 * float(d["f8_actual"][0]) + 1e-29
