"""Parity of the tcgen05 GEMM (through the C ABI, via the reference-named Python entry point)
against the CPU oracle. Target tolerances: bf16 within rtol 1e-2 / atol 1e-2 of the
fp32 product; fp16 the same bounds."""
import os

import numpy as np
import pytest
import torch

from oracle import gemm as o_gemm

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
RTOL, ATOL = 1e-2, 1e-2


def _mm():
    from triton_b200.tutorials.blackwell_gemm_ws import matmul
    return matmul


def _check(c, ref):
    torch.testing.assert_close(c.cpu().float(), ref.float(), rtol=RTOL, atol=ATOL)


def test_config1_512_cubed_row_major(cuda):
    """Benchmark config 1: seed 0, N(0,1) entries, row-major A and B, bf16 out."""
    torch.manual_seed(0)
    a = torch.randn(512, 512).to(torch.bfloat16)
    b = torch.randn(512, 512).to(torch.bfloat16)
    c = _mm()(a.to(cuda), b.to(cuda))
    # |C| ~ sqrt(512) here: bf16 rounding of the result alone is up to 2^-8 relative
    torch.testing.assert_close(c.cpu().float(), o_gemm.gemm_ref(a, b).float(), rtol=RTOL, atol=ATOL)


def test_config1_against_reference_interpreter_fixture(cuda):
    """fp16 copies of the config-1 inputs against rows the reference's tutorial kernel produced
    under TRITON_INTERPRET=1 (tests/golden/gemm_interp_512.npz)."""
    fx = np.load(os.path.join(GOLDEN, "gemm_interp_512.npz"))
    torch.manual_seed(int(fx["seed"]))
    a = torch.randn(512, 512).to(torch.float16)
    b = torch.randn(512, 512).to(torch.float16)
    c = _mm()(a.to(cuda), b.to(cuda)).cpu()
    got = c[fx["rows"].tolist()].float().numpy()
    np.testing.assert_allclose(got, fx["c_rows"].astype(np.float32), rtol=2e-3, atol=0.0625)


@pytest.mark.parametrize("a_t", [False, True])
@pytest.mark.parametrize("b_t", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_layouts(cuda, a_t, b_t, dtype):
    torch.manual_seed(1)
    M, N, K = 384, 320, 448
    a = (torch.randn(K, M).T if a_t else torch.randn(M, K)).to(dtype) / K ** 0.5
    b = (torch.randn(N, K).T if b_t else torch.randn(K, N)).to(dtype)
    c = _mm()(a.to(cuda) if not a_t else a.T.contiguous().to(cuda).T,
              b.to(cuda) if not b_t else b.T.contiguous().to(cuda).T)
    _check(c, o_gemm.gemm_ref(a, b))


@pytest.mark.parametrize("shape", [(1, 8, 8), (129, 8, 8), (300, 200, 72), (128, 256, 64), (1000, 1000, 1000),
                                   (127, 513, 1032), (2048, 24, 40)])
def test_ragged_shapes(cuda, shape):
    M, N, K = shape
    torch.manual_seed(2)
    a = (torch.randn(M, K) / K ** 0.5).to(torch.bfloat16)
    w = torch.randn(N, K).to(torch.bfloat16)
    c = _mm()(a.to(cuda), w.to(cuda).T)
    _check(c, o_gemm.gemm_ref(a, w.T))


def test_empty_and_zero_k(cuda):
    mm = _mm()
    a = torch.zeros(0, 64, dtype=torch.bfloat16, device=cuda)
    b = torch.zeros(64, 32, dtype=torch.bfloat16, device=cuda)
    assert mm(a, b).shape == (0, 32)
    a = torch.zeros(16, 0, dtype=torch.bfloat16, device=cuda)
    b = torch.zeros(0, 32, dtype=torch.bfloat16, device=cuda)
    c = mm(a, b)
    assert c.shape == (16, 32) and torch.count_nonzero(c) == 0


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("split_k", [1, 3, 4])
def test_tile_widths_and_split_k(cuda, bn, split_k):
    torch.manual_seed(3)
    M, N, K = 256, 512, 2048
    a = (torch.randn(M, K) / K ** 0.5).to(torch.bfloat16)
    w = torch.randn(N, K).to(torch.bfloat16)
    c = _mm()(a.to(cuda), w.to(cuda).T, config={"BLOCK_SIZE_N": bn, "SPLIT_K": split_k})
    _check(c, o_gemm.gemm_ref(a, w.T))


@pytest.mark.parametrize("tile", [512, 1024])  # CTA pair: 256 x 256 and 256 x 512 tiles
@pytest.mark.parametrize("layout", ["nn", "nt", "tn", "tt"])
@pytest.mark.parametrize("shape", [(512, 1024, 512), (300, 700, 264), (1000, 1000, 1000)])
def test_cta_pair_tiles(cuda, tile, layout, shape):
    """Both CTA-pair tilings on all four operand layouts, with ragged M / N / K edges (the wide tile permutes
    its accumulator columns: every 128-column group must land on the right output columns)."""
    M, N, K = shape
    torch.manual_seed(6)
    a = (torch.randn(M, K) / K ** 0.5).to(torch.bfloat16)
    b = torch.randn(K, N).to(torch.bfloat16)
    ad = a.to(cuda) if layout[0] == "n" else a.t().contiguous().to(cuda).t()
    bd = b.to(cuda) if layout[1] == "n" else b.t().contiguous().to(cuda).t()
    if (ad.stride(0) if ad.stride(1) == 1 else ad.stride(1)) % 8 or (bd.stride(0) if bd.stride(1) == 1 else bd.stride(1)) % 8:
        pytest.skip("leading dimension not 16-byte aligned in this layout")
    c = _mm()(ad, bd, config={"BLOCK_SIZE_N": tile})
    _check(c, o_gemm.gemm_ref(a, b))


def test_wide_tile_fp16(cuda):
    """fp16 in and out through the 256 x 512 tile's TMA-store epilogue."""
    torch.manual_seed(8)
    M, N, K = 512, 1536, 320
    a = (torch.randn(M, K) / K ** 0.5).to(torch.float16)
    w = torch.randn(N, K).to(torch.float16)
    c = _mm()(a.to(cuda), w.to(cuda).T, config={"BLOCK_SIZE_N": 1024})
    assert c.dtype == torch.float16
    _check(c, o_gemm.gemm_ref(a, w.T))


def test_wide_tile_split_k(cuda):
    torch.manual_seed(7)
    M, N, K = 256, 1024, 4096
    a = (torch.randn(M, K) / K ** 0.5).to(torch.bfloat16)
    w = torch.randn(N, K).to(torch.bfloat16)
    c = _mm()(a.to(cuda), w.to(cuda).T, config={"BLOCK_SIZE_N": 1024, "SPLIT_K": 3})
    _check(c, o_gemm.gemm_ref(a, w.T))


def test_skinny_config2(cuda):
    """The skinny case of benchmark config 2, M=128, N=K=8192 (B K-major), seed 1."""
    torch.manual_seed(1)
    M, N, K = 128, 8192, 8192
    a = (torch.randn(M, K) / K ** 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K) / K ** 0.5).to(torch.bfloat16)
    c = _mm()(a.to(cuda), w.to(cuda).T)
    _check(c, o_gemm.gemm_ref(a, w.T))


def test_full_size_linearity_property(cuda):
    """8192^3 (benchmark config 2) is too slow for the CPU oracle; check size-independent
    properties instead: (i) a 256-row band against the oracle, (ii) linearity A(B1+B2) = AB1 + AB2
    on exactly-representable inputs (small integers: every partial sum is exact in fp32)."""
    torch.manual_seed(1)
    n = 8192
    a = (torch.randn(n, n) / n ** 0.5).to(torch.bfloat16)
    w = (torch.randn(n, n) / n ** 0.5).to(torch.bfloat16)
    mm = _mm()
    c = mm(a.to(cuda), w.to(cuda).T)
    # one band of full rows per tile-row class of the 256 x 512 tiling: the first, a middle and the last 256-row
    # block (each band crosses every 512-column block, the first and the last included)
    for band in (slice(0, 256), slice(4096 - 128, 4096 + 128), slice(n - 256, n)):
        _check(c[band], o_gemm.gemm_ref(a[band], w.T))
    g = torch.Generator().manual_seed(5)
    ai = torch.randint(-2, 3, (n, n), generator=g).to(torch.bfloat16).to(cuda)
    b1 = torch.randint(-1, 2, (n, n), generator=g).to(torch.bfloat16).to(cuda)
    b2 = torch.randint(-1, 2, (n, n), generator=g).to(torch.bfloat16).to(cuda)
    lhs = mm(ai, (b1 + b2).T).float()
    rhs = mm(ai, b1.T).float() + mm(ai, b2.T).float()
    # |entries| <= 2*2*8192 = 32768 > 256: bf16 output rounding applies to both sides
    torch.testing.assert_close(lhs, rhs, rtol=2 ** -6, atol=2.0)
    from triton_b200 import _lib
    _lib.sync_check()


def test_bad_inputs_raise(cuda):
    mm = _mm()
    a = torch.zeros(8, 16, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(AssertionError):
        mm(a, torch.zeros(8, 16, dtype=torch.bfloat16, device=cuda))
    with pytest.raises(RuntimeError):
        mm(torch.zeros(8, 16, dtype=torch.bfloat16), torch.zeros(16, 8, dtype=torch.bfloat16))


@pytest.mark.parametrize("bn,split_k", [(128, 2), (128, 4), (256, 4), (256, 8), (64, 2)])
@pytest.mark.parametrize("shape", [(128, 1024, 4096), (16, 1000, 4104), (100, 512, 8192)])
def test_in_cluster_split_k(cuda, lib, bn, split_k, shape):
    """Few tiles and a long K: the split_k CTAs of a tile run as one thread-block cluster and sum their fp32
    partials through distributed shared memory (one launch, no workspace). Ragged M / N / K, every tile width,
    cluster sizes 2, 4 and 8; the rank-ordered sum makes two runs bit-identical."""
    import ctypes
    from triton_b200 import _lib
    M, N, K = shape
    torch.manual_seed(12)
    a = (torch.randn(M, K) / K ** 0.5).to(torch.bfloat16)
    w = torch.randn(N, K).to(torch.bfloat16)
    ad, wd = a.to(cuda), w.to(cuda)
    cfg = {"BLOCK_SIZE_N": bn, "SPLIT_K": split_k}
    c = _mm()(ad, wd.T, config=cfg)
    _check(c, o_gemm.gemm_ref(a, w.T))
    assert torch.equal(c, _mm()(ad, wd.T, config=cfg))
    # this plan needs no workspace: the partial sums never leave the SMs
    args = _lib.GemmArgs()
    args.a = args.b = args.c = 16
    args.m, args.n, args.k = M, N, K
    args.lda = args.ldb = K
    args.ldc = N
    args.in_dtype = args.out_dtype = _lib.BF16
    args.a_k_major = args.b_k_major = 1
    args.split_k, args.block_n = split_k, bn
    with torch.cuda.device(cuda):
        assert lib.tb200_gemm_workspace_bytes(ctypes.byref(args)) == 0


def test_in_cluster_split_k_fp16_and_default_plan(cuda):
    """The library's own choice for one row of tiles (the skinny shape scaled down) and fp16 output."""
    torch.manual_seed(13)
    M, N, K = 128, 2048, 8192
    for dt in (torch.float16, torch.bfloat16):
        a = (torch.randn(M, K) / K ** 0.5).to(dt)
        w = torch.randn(N, K).to(dt)
        c = _mm()(a.to(cuda), w.to(cuda).T)
        _check(c, o_gemm.gemm_ref(a, w.T))


def test_tensors_on_another_device_than_the_current_one(cuda):
    """Operands on cuda:1 while cuda:0 is current: the wrappers switch devices for the call (and only then) and launch
    on that device's current stream. Needs two GPUs."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from triton_b200 import _lib
    from triton_b200.triton_kernels.matmul import matmul as moe_matmul
    other = torch.device("cuda:1")
    torch.manual_seed(14)
    a = (torch.randn(256, 512) / 512 ** 0.5).to(torch.bfloat16)
    w = torch.randn(384, 512).to(torch.bfloat16)
    with torch.cuda.device(cuda):
        c = _mm()(a.to(other), w.to(other).T)
        assert c.device == other and torch.cuda.current_device() == 0
        _check(c, o_gemm.gemm_ref(a, w.T))
        y = moe_matmul(a.to(other), w.t().contiguous().unsqueeze(0).to(other), None)
        assert y.device == other
        _check(y, o_gemm.gemm_ref(a, w.T))
        _lib.sync_check(other)
