"""Parity of the FP8 paths against the CPU oracle: tensorwise-scaled e4m3 GEMM (tolerance of the
reference's own test, atol 0.1 / rtol 0.05, test_correctness.py:554-562) and the MXFP8 block-scaled
GEMM (target: rtol 3e-2; the reference's test uses atol 0.1, rtol 0.01 on N(0, 0.5) inputs)."""
import pytest
import torch

from oracle import gemm as o_gemm
from oracle import mxfp8 as o_mx

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (2048, 2048, 2048), (384, 256, 640)])
@pytest.mark.parametrize("num_ctas", [1, 2])
def test_scaled_mm_tensorwise(cuda, shape, num_ctas):
    from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
    M, N, K = shape
    torch.manual_seed(0)
    a = (torch.randn(M, K) * 0.1).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K) * 0.1).to(torch.float8_e4m3fn)
    sa, sb = torch.rand(1), torch.rand(1)
    out = blackwell_scaled_mm_ws(a.to(cuda), b.to(cuda), sa.to(cuda), sb.to(cuda), scale_mode="tensorwise",
                                 NUM_CTAS=num_ctas)
    ref = o_gemm.scaled_mm_tensorwise_ref(a, b, sa, sb)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=0.1, rtol=0.05)
    # tighter: within bf16 rounding of the fp32 result
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=1e-3, rtol=1e-2)


@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (384, 256, 640)])
def test_scaled_mm_rowwise(cuda, shape):
    """out[m, n] = (a @ b.T)[m, n] * scale_a[m] * scale_b[n] — ScaledMM.get_reference, rowwise branch
    (test_correctness.py:548-551)."""
    from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
    M, N, K = shape
    torch.manual_seed(0)
    a = (torch.randn(M, K) * 0.1).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K) * 0.1).to(torch.float8_e4m3fn)
    sa, sb = torch.rand(M), torch.rand(N)
    out = blackwell_scaled_mm_ws(a.to(cuda), b.to(cuda), sa.to(cuda), sb.to(cuda), scale_mode="rowwise")
    ref = o_gemm.scaled_mm_rowwise_ref(a, b, sa, sb)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=1e-3, rtol=1e-2)
    # the 256 x 512 CTA-pair tile (permuted accumulator columns: the per-column scale must follow)
    out = blackwell_scaled_mm_ws(a.to(cuda), b.to(cuda), sa.to(cuda), sb.to(cuda), scale_mode="rowwise", NUM_CTAS=2,
                                 BLOCK_N=512)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=1e-3, rtol=1e-2)


@pytest.mark.parametrize("shape", [(1024, 1024, 1024), (384, 256, 640), (200, 128, 256), (4096, 2048, 4096)])
def test_scaled_mm_blockwise(cuda, shape):
    """DeepSeek blockwise: scale_a [M, K//128] M-major, scale_b [N//128, K//128]; inputs as in the
    reference's ScaledMM.create_inputs (test_correctness.py:518-532), its tolerance atol 0.1 / rtol 0.05, and
    a tighter bound near bf16 rounding of the fp32 result."""
    from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
    M, N, K = shape
    torch.manual_seed(0)
    a = (torch.randn(M, K) * 0.1).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K) * 0.1).to(torch.float8_e4m3fn)
    sa = torch.rand(M, K // 128).t().contiguous().t()  # M-major
    sb = torch.rand(N // 128, K // 128)
    out = blackwell_scaled_mm_ws(a.to(cuda), b.to(cuda), sa.to(cuda), sb.to(cuda))  # blockwise is the default mode
    ref = o_gemm.scaled_mm_blockwise_ref(a, b, sa, sb)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=0.1, rtol=0.05)
    torch.testing.assert_close(out.cpu().float(), ref.float(), atol=2e-3, rtol=1e-2)


def test_scaled_mm_blockwise_exact_powers_of_two(cuda):
    """Power-of-two data and scales: every product and partial sum is exact, so the fp32 output must equal
    the oracle bit for bit (checks group/row/block indexing at a non-trivial size, fp32 out, row-major scale_a)."""
    from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
    M, N, K = 512, 640, 1024
    g = torch.Generator().manual_seed(5)
    a = torch.pow(2.0, torch.randint(-3, 3, (M, K), generator=g).float()).to(torch.float8_e4m3fn)
    b = torch.pow(2.0, torch.randint(-3, 3, (N, K), generator=g).float()).to(torch.float8_e4m3fn)
    sa = torch.pow(2.0, torch.randint(-4, 4, (M, K // 128), generator=g).float())
    sb = torch.pow(2.0, torch.randint(-4, 4, (N // 128, K // 128), generator=g).float())
    out = blackwell_scaled_mm_ws(a.to(cuda), b.to(cuda), sa.to(cuda), sb.to(cuda), out_dtype=torch.float32,
                                 scale_mode="blockwise")
    ref = o_gemm.scaled_mm_blockwise_ref(a, b, sa, sb, out_dtype=torch.float32)
    assert torch.equal(out.cpu(), ref)


def test_scaled_mm_argument_checks(cuda):
    from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
    a = torch.zeros(128, 128, device=cuda).to(torch.float8_e4m3fn)
    s = torch.ones(1, device=cuda)
    with pytest.raises(AssertionError):
        blackwell_scaled_mm_ws(a, a, s, s, scale_mode="blockwise")  # scalar scales are not blockwise scales
    with pytest.raises(AssertionError):
        blackwell_scaled_mm_ws(a[:, :64].contiguous(), a[:, :64].contiguous(), s, s, scale_mode="tensorwise")
    with pytest.raises(KeyError):
        blackwell_scaled_mm_ws(a, a, s, s, scale_mode="columnwise")


def _mx_case(cuda, M, N, K, bn, seed=3):
    from triton_b200.tutorials.blackwell_gemm_ws_mxfp8 import matmul
    g = torch.Generator().manual_seed(seed)
    a, sa = o_mx.make_mxfp8_operand(M, K, g)
    b, sb = o_mx.make_mxfp8_operand(N, K, g)
    out = matmul(a.to(cuda), b.to(cuda), sa.to(cuda).view(torch.float8_e8m0fnu), sb.to(cuda).view(torch.float8_e8m0fnu),
                 {"BLOCK_SIZE_N": bn} if bn else None)
    ref = o_mx.dequantize(a, sa) @ o_mx.dequantize(b, sb).t()
    # rtol 3e-2 (the target) on entries, with an absolute floor of 3e-2 x the mean magnitude
    torch.testing.assert_close(out.cpu().float(), ref, rtol=3e-2, atol=3e-2 * float(ref.abs().mean()))


@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 256, 256), (384, 256, 512), (384, 384, 1024)])
@pytest.mark.parametrize("bn", [0, 128, 256, 512])  # 512: CTA pair, 256 x 256 tile
def test_mxfp8_reference_test_shapes(cuda, shape, bn):
    """Shapes of the reference's Mxfp8Gemm.SHAPES (test_correctness.py:446-450) plus a ragged-N tile."""
    _mx_case(cuda, *shape, bn)


def test_mxfp8_scale_layout_known_answer(cuda):
    """All-ones operands with scales that differ per row (A) and per K block (B): every output is
    an exact power-of-two sum, so any mistake in the 512-byte-atom addressing shows up exactly."""
    from triton_b200.tutorials.blackwell_gemm_ws_mxfp8 import matmul
    M, N, K = 256, 384, 512
    a = torch.ones(M, K).to(torch.float8_e4m3fn)
    b = torch.ones(N, K).to(torch.float8_e4m3fn)
    sa = (127 + (torch.arange(M)[:, None] % 5) - 2).to(torch.uint8).expand(M, K // 32).contiguous()
    sb = (127 + (torch.arange(K // 32)[None, :] % 3) + (torch.arange(N)[:, None] % 2)).to(torch.uint8)
    fa, fb = o_mx.swizzle_scales(sa), o_mx.swizzle_scales(sb)
    out = matmul(a.to(cuda), b.to(cuda), fa.to(cuda).view(torch.float8_e8m0fnu), fb.to(cuda).view(torch.float8_e8m0fnu))
    ref = o_mx.dequantize(a, fa) @ o_mx.dequantize(b, fb).t()
    assert torch.equal(out.cpu().float(), ref.to(torch.bfloat16).float())


def test_mxfp8_2048_and_linearity_at_full_size(cuda):
    _mx_case(cuda, 2048, 2048, 2048, 0)
    # the benchmark size (8192^3): the CPU oracle is too slow; use exactness instead — with
    # all-ones data and power-of-two scales every product is exact, so C = K/32 * sum of 2^(ea+eb).
    from triton_b200.tutorials.blackwell_gemm_ws_mxfp8 import matmul
    n = 8192
    a = torch.ones(n, n, device=cuda).to(torch.float8_e4m3fn)
    ea = (torch.arange(n, device=cuda) % 4).to(torch.uint8)      # per-row exponent of A
    eb = (torch.arange(n, device=cuda) % 3).to(torch.uint8)      # per-row exponent of B
    sa = (127 + ea)[:, None].expand(n, n // 32).contiguous()
    sb = (127 + eb)[:, None].expand(n, n // 32).contiguous()
    fa = o_mx.swizzle_scales(sa.cpu()).to(cuda).view(torch.float8_e8m0fnu)
    fb = o_mx.swizzle_scales(sb.cpu()).to(cuda).view(torch.float8_e8m0fnu)
    out = matmul(a, a, fa, fb)
    want = (n * torch.pow(2.0, ea.float())[:, None] * torch.pow(2.0, eb.float())[None, :]).to(torch.bfloat16)
    assert torch.equal(out, want)


def test_mxfp8_full_size_bands(cuda):
    """MXFP8 benchmark configuration (8192^3, per-block scales 2^u, u in [-4, 4], seed 3): one band of full rows per
    tile-row class (first, a middle and the last 256 rows; each crosses every column block) against the oracle."""
    from triton_b200.tutorials.blackwell_gemm_ws_mxfp8 import matmul
    n = 8192
    g = torch.Generator().manual_seed(3)
    qa, sa = o_mx.make_mxfp8_operand(n, n, g)
    qb, sb = o_mx.make_mxfp8_operand(n, n, g)
    out = matmul(qa.to(cuda), qb.to(cuda), sa.to(cuda).view(torch.float8_e8m0fnu), sb.to(cuda).view(torch.float8_e8m0fnu))
    da, db = o_mx.dequantize(qa, sa), o_mx.dequantize(qb, sb)
    for band in (slice(0, 256), slice(4096 - 128, 4096 + 128), slice(n - 256, n)):
        ref = da[band] @ db.t()
        torch.testing.assert_close(out[band].cpu().float(), ref, rtol=3e-2, atol=3e-2 * float(ref.abs().mean()))


def test_mxfp8_asserts(cuda):
    from triton_b200.tutorials.blackwell_gemm_ws_mxfp8 import matmul
    a = torch.zeros(128, 128, device=cuda).to(torch.float8_e4m3fn)
    s = torch.zeros(128 * 4, dtype=torch.uint8, device=cuda).view(torch.float8_e8m0fnu)
    with pytest.raises(AssertionError):
        matmul(a.to(torch.bfloat16), a, s, s)
    with pytest.raises(AssertionError):
        matmul(a[:, :64].contiguous(), a[:, :64].contiguous(), s, s)
    with pytest.raises(AssertionError):
        matmul(a, a, s[:100], s)


def test_rowwise_scaled_skinny_takes_the_in_cluster_split(cuda):
    """M = 64 against N = 1024, K = 4096 (e4m3, row-wise scales): one row of tiles, so K is split inside a cluster
    and the scales are applied by the reducing CTAs."""
    from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
    g = torch.Generator().manual_seed(31)
    M, N, K = 64, 1024, 4096
    a = (torch.randn(M, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    b = (torch.randn(N, K, generator=g) * 0.1).to(torch.float8_e4m3fn)
    sa, sb = torch.rand(M, generator=g) + 0.5, torch.rand(N, generator=g) + 0.5
    out = blackwell_scaled_mm_ws(a.to(cuda), b.to(cuda), sa.to(cuda), sb.to(cuda), scale_mode="rowwise")
    ref = o_gemm.scaled_mm_rowwise_ref(a, b, sa, sb)
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=1e-2, atol=2e-3)
