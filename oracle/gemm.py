"""Oracle for the dense GEMMs (test infrastructure only).

Follows the reference's checks:
  * bf16/fp16 GEMM: ``torch.matmul`` of the inputs, compared with ``assert_close``
    (``third_party/tlx/tutorials/testing/test_correctness.py:279-290``); here the product is
    taken in fp32 and rounded once to the output dtype.
  * tensorwise FP8: ``ScaledMM.get_reference`` (``test_correctness.py:534-552``):
    ``(a.float() @ b.float().T) * scale_a * scale_b`` rounded to bf16.
"""
import torch


def gemm_ref(a: torch.Tensor, b: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """C = A @ B with fp32 accumulation on CPU; a is (M, K), b is (K, N)."""
    out_dtype = out_dtype or a.dtype
    return (a.detach().cpu().float() @ b.detach().cpu().float()).to(out_dtype)


def scaled_mm_tensorwise_ref(a, b, scale_a, scale_b, out_dtype=torch.bfloat16):
    """a (M, K) and b (N, K) in an fp8 dtype, one fp32 scale each."""
    af, bf = a.detach().cpu().float(), b.detach().cpu().float()
    prod = af @ bf.t()
    return (prod * scale_a.detach().cpu().float().reshape(()) * scale_b.detach().cpu().float().reshape(())).to(out_dtype)


def scaled_mm_rowwise_ref(a, b, scale_a, scale_b, out_dtype=torch.bfloat16):
    """a (M, K), b (N, K) fp8; scale_a [M], scale_b [N]: out = (a @ b.T) * scale_a[:, None] * scale_b[None, :]
    (ScaledMM.get_reference, rowwise branch, test_correctness.py:548-551)."""
    prod = a.detach().cpu().float() @ b.detach().cpu().float().t()
    return (prod * scale_a.detach().cpu().float()[:, None] * scale_b.detach().cpu().float()[None, :]).to(out_dtype)


def scaled_mm_blockwise_ref(a, b, scale_a, scale_b, out_dtype=torch.bfloat16):
    """Blockwise (DeepSeek) scaled matmul: every 128-wide K group of A @ B^T is multiplied by
    scale_a[:, g] (per row) and scale_b[n // 128, g] (per 128-column block) before it is summed —
    ``ScaledMM.get_reference``, blockwise branch (``testing/test_correctness.py:535-547``)."""
    af, bf = a.detach().cpu().float(), b.detach().cpu().float()
    sa, sb = scale_a.detach().cpu().float(), scale_b.detach().cpu().float()
    M, K = af.shape
    N = bf.shape[0]
    out = torch.zeros(M, N, dtype=torch.float32)
    for g in range(K // 128):
        partial = af[:, g * 128:(g + 1) * 128] @ bf[:, g * 128:(g + 1) * 128].t()
        out += partial * sa[:, g][:, None] * sb[:, g].repeat_interleave(128)[None, :]
    return out.to(out_dtype)
