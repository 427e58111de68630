"""Parity of the flash-attention backward kernel (dq, dk, dv) against the CPU oracle. Tolerance: the
reference's own setting for this test, atol 1e-2 / rtol 0 on N(0,1) inputs with sm_scale 0.5
(test_correctness.py:919-1068), and atol + rtol 2e-2 elsewhere (bf16 outputs)."""
import math

import pytest
import torch

from oracle import attention as o_attn

pytestmark = pytest.mark.gpu


def _run(cuda, B, H, S, causal, dtype=torch.bfloat16, scale=None, seed=5, Skv=None, std=1.0, D=128):
    from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_backward, attention_with_lse
    Skv = Skv or S
    g = torch.Generator().manual_seed(seed)
    q = (torch.randn(B, H, S, D, generator=g) * std).to(dtype)
    k = (torch.randn(B, H, Skv, D, generator=g) * std).to(dtype)
    v = (torch.randn(B, H, Skv, D, generator=g) * std).to(dtype)
    do = torch.randn(B, H, S, D, generator=g).to(dtype)
    scale = scale or 1.0 / math.sqrt(D)
    qc, kc, vc, doc = (t.to(cuda) for t in (q, k, v, do))
    o, lse = attention_with_lse(qc, kc, vc, scale, causal)
    dq, dk, dv = attention_backward(qc, kc, vc, o, lse, doc, scale, causal)
    from triton_b200 import _lib
    _lib.sync_check(cuda)
    ref = o_attn.attention_bwd_ref(q, k, v, do, scale, causal)
    return (dq.cpu().float(), dk.cpu().float(), dv.cpu().float()), ref


def _check(got, ref, atol, rtol):
    for name, a, b in zip(("dq", "dk", "dv"), got, ref):
        assert torch.isfinite(a).all(), name
        torch.testing.assert_close(a, b, atol=atol, rtol=rtol, msg=lambda m, n=name: f"{n}: {m}")


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [64, 128, 256, 1024])
def test_bf16_block_multiples(cuda, causal, S):
    got, ref = _run(cuda, 2, 2, S, causal)
    _check(got, ref, 2e-2, 2e-2)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [32, 64])
def test_smaller_head_dims(cuda, causal, D):
    """Head dims below 128 run zero-padded through the 128-wide backward kernel."""
    got, ref = _run(cuda, 1, 2, 320, causal, D=D)
    assert got[0].shape[-1] == D
    _check(got, ref, 2e-2, 2e-2)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [1, 77, 129, 1000])
def test_ragged_sequence_lengths(cuda, causal, S):
    got, ref = _run(cuda, 1, 3, S, causal)
    _check(got, ref, 2e-2, 2e-2)


@pytest.mark.parametrize("causal", [False, True])
def test_reference_test_setting_fp16(cuda, causal):
    """Shape, input distribution and tolerance of the reference's backward test: (4, 8, 1024, 128) fp16,
    q/k/v ~ N(0, 0.5^2), dO ~ N(0, 1), sm_scale 0.5, atol 1e-2 / rtol 0."""
    got, ref = _run(cuda, 4, 8, 1024, causal, dtype=torch.float16, scale=0.5, seed=20, std=0.5)
    _check(got, ref, 1e-2, 0.0)


def test_cross_attention_lengths(cuda):
    got, ref = _run(cuda, 1, 2, 200, False, Skv=333)
    _check(got, ref, 2e-2, 2e-2)
    got, ref = _run(cuda, 1, 2, 333, False, Skv=64)
    _check(got, ref, 2e-2, 2e-2)


def test_autograd_function_matches_sdpa(cuda):
    """attention(...) with requires_grad inputs: .backward() fills q/k/v.grad like the reference's autograd
    Function; compared with SDPA autograd in fp32 on the GPU."""
    from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention
    torch.manual_seed(7)
    q, k, v = (torch.randn(2, 4, 512, 128, device=cuda, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    do = torch.randn(2, 4, 512, 128, device=cuda, dtype=torch.bfloat16)
    for causal in (False, True):
        out = attention(q, k, v, 0.1, causal)
        out.backward(do)
        got = [t.grad.float().clone() for t in (q, k, v)]
        for t in (q, k, v):
            t.grad = None
        q32, k32, v32 = (t.detach().float().requires_grad_() for t in (q, k, v))
        ref = torch.nn.functional.scaled_dot_product_attention(q32, k32, v32, scale=0.1, is_causal=causal)
        ref.backward(do.float())
        for a, b in zip(got, (q32.grad, k32.grad, v32.grad)):
            torch.testing.assert_close(a, b, atol=2e-2, rtol=2e-2)


def test_linearity_in_do_at_config3_length(cuda):
    """S = 8192 (the benchmark length), one head: gradients are linear in dO, so bwd(2 dO) = 2 bwd(dO)
    up to output rounding; and dV of a constant dO row pattern sums to the column sums of P."""
    from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_backward, attention_with_lse
    torch.manual_seed(11)
    q, k, v, do = (torch.randn(1, 2, 8192, 128, device=cuda, dtype=torch.bfloat16) for _ in range(4))
    scale = 1.0 / math.sqrt(128)
    for causal in (False, True):
        o, lse = attention_with_lse(q, k, v, scale, causal)
        g1 = attention_backward(q, k, v, o, lse, do, scale, causal)
        g2 = attention_backward(q, k, v, o, lse, do * 2, scale, causal)
        for a, b in zip(g1, g2):
            assert torch.isfinite(a).all()
            torch.testing.assert_close(b.float(), 2 * a.float(), atol=2e-3, rtol=2e-2)
        # spot-check one KV block and one query block against fp32 math on the GPU
        qf, kf, vf, dof, of = (t[0, 1].float() for t in (q, k, v, do, o))
        s = (qf @ kf.t()) * scale
        if causal:
            s = s.masked_fill(~torch.ones(8192, 8192, dtype=torch.bool, device=cuda).tril(), float("-inf"))
        p = torch.softmax(s, dim=-1)
        dv_ref = p.t() @ dof
        ds = p * (dof @ vf.t() - (of * dof).sum(-1, keepdim=True))
        dq_ref = scale * (ds @ kf)
        dk_ref = scale * (ds.t() @ qf)
        torch.testing.assert_close(g1[0][0, 1].float(), dq_ref, atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(g1[1][0, 1].float(), dk_ref, atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(g1[2][0, 1].float(), dv_ref, atol=2e-2, rtol=2e-2)


def test_argument_checks(cuda):
    from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_backward
    q = torch.randn(1, 1, 64, 256, device=cuda, dtype=torch.bfloat16)
    lse = torch.zeros(1, 1, 64, device=cuda)
    with pytest.raises(NotImplementedError):
        attention_backward(q, q, q, q, lse, q, 0.1, False)
