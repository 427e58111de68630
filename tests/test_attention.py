"""Parity of the flash-attention forward kernel against the CPU oracle (fp32 softmax(QK^T)V and
base-2 LSE). Tolerances: bf16 rtol 1e-2 / atol 1e-2 (the target tolerance); fp16 case uses the reference's own
test setting (atol 1e-2, rtol 0, test_correctness.py:425-435)."""
import math

import pytest
import torch

from oracle import attention as o_attn

pytestmark = pytest.mark.gpu


def _run(cuda, B, H, S, D, causal, dtype=torch.bfloat16, scale=None, std=1.0, seed=2):
    from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_with_lse
    g = torch.Generator().manual_seed(seed)
    q, k, v = ((torch.randn(B, H, S, D, generator=g) * std).to(dtype) for _ in range(3))
    scale = scale or 1.0 / math.sqrt(D)
    o, lse = attention_with_lse(q.to(cuda), k.to(cuda), v.to(cuda), scale, causal)
    ref_o, ref_lse = o_attn.attention_ref(q, k, v, scale, causal)
    return o.cpu().float(), lse.cpu(), ref_o.float(), ref_lse


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [128, 256, 384, 1024])
@pytest.mark.parametrize("D", [64, 128])
def test_bf16_block_multiples(cuda, causal, S, D):
    o, lse, ro, rl = _run(cuda, 2, 3, S, D, causal)
    torch.testing.assert_close(o, ro, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lse, rl, rtol=0, atol=1e-3)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [16, 32])
def test_small_head_dims(cuda, causal, D):
    """Head dims 16 and 32 of the reference's set (blackwell_fa_ws_pipelined_persistent.py:3291-3292) run zero-padded
    through the 64-wide kernel."""
    o, lse, ro, rl = _run(cuda, 2, 2, 300, D, causal)
    assert o.shape[-1] == D
    torch.testing.assert_close(o, ro, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lse, rl, rtol=0, atol=1e-3)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [128, 300, 1024, 77])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_head_dim_256(cuda, causal, S, dtype):
    """Head dim 256, the largest of the reference's set: one 128-row query group per CTA, two-deep K / V ring; several
    tiles per CTA at S = 1024 (B H S / 128 = 192 tiles on 148 CTAs)."""
    o, lse, ro, rl = _run(cuda, 4, 6, S, 256, causal, dtype=dtype)
    torch.testing.assert_close(o, ro, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lse, rl, rtol=0, atol=1e-3)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("S", [1, 77, 129, 1000])
def test_ragged_sequence_lengths(cuda, causal, S):
    o, lse, ro, rl = _run(cuda, 1, 2, S, 128, causal)
    torch.testing.assert_close(o, ro, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(lse, rl, rtol=0, atol=1e-3)


@pytest.mark.parametrize("causal", [False, True])
def test_reference_test_setting_fp16(cuda, causal):
    """(Z, H, N_CTX, D) = (4, 8, 1024, 128), fp16, N(0, 0.5), sm_scale 0.5 — the reference's
    FlashAttention test (test_correctness.py:302, 425-435): atol 1e-2, rtol 0."""
    o, lse, ro, rl = _run(cuda, 4, 8, 1024, 128, causal, dtype=torch.float16, scale=0.5, std=0.5, seed=20)
    torch.testing.assert_close(o, ro, rtol=0, atol=1e-2)
    torch.testing.assert_close(lse, rl, rtol=0, atol=1e-3)


def test_rescale_path_with_growing_logits(cuda):
    """Keys whose norm grows along the sequence force the running max up by more than 2^8 several
    times, so the accumulator-rescale branch runs; checks it against the oracle."""
    from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_with_lse
    B, H, S, D = 1, 2, 1024, 128
    g = torch.Generator().manual_seed(7)
    q = torch.randn(B, H, S, D, generator=g).abs().to(torch.bfloat16)
    ramp = torch.linspace(0.05, 3.0, S).view(1, 1, S, 1)
    k = (torch.randn(B, H, S, D, generator=g).abs() * ramp).to(torch.bfloat16)
    v = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    o, lse = attention_with_lse(q.to(cuda), k.to(cuda), v.to(cuda), 1.0 / math.sqrt(D), False)
    ro, rl = o_attn.attention_ref(q, k, v, 1.0 / math.sqrt(D), False)
    torch.testing.assert_close(o.cpu().float(), ro.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(lse.cpu(), rl, rtol=1e-5, atol=1e-2)


def test_config3_shapes_by_properties(cuda):
    """The benchmark sizes ([4,32,8192,128] and [32,32,1024,128]) are too large for the CPU
    oracle in full: check (i) the last 384 query rows of one (batch, head) against the oracle (its
    causal mask is aligned to the end of the sequence), (ii) the size-independent identity that
    with V = all-ones every output is 1 (softmax rows sum to 1), (iii) causal row 0 returns V[0]."""
    from triton_b200 import _lib
    from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_with_lse
    g = torch.Generator().manual_seed(2)
    D = 128
    sc = 1.0 / math.sqrt(D)
    for (B, H, S) in [(4, 32, 8192), (32, 32, 1024)]:
        q = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
        k = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
        v = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
        qd, kd, vd = q.to(cuda), k.to(cuda), v.to(cuda)
        ones = torch.ones_like(vd)
        for causal in (False, True):
            o, lse = attention_with_lse(qd, kd, vd, sc, causal)
            ro, rl = o_attn.attention_ref(q[-1:, -1:, -384:], k[-1:, -1:], v[-1:, -1:], sc, causal)
            torch.testing.assert_close(o[-1:, -1:, -384:].cpu().float(), ro.float(), rtol=1e-2, atol=1e-2)
            torch.testing.assert_close(lse[-1:, -1:, -384:].cpu(), rl, rtol=0, atol=1e-3)
            # the first and a middle 256-row query tile of another (batch, head): a causal mask that ends inside the
            # keys is the full-length mask restricted to the keys up to the tile's last row
            for r0 in (0, (S // 2 // 256) * 256):
                r1 = r0 + 256
                kv_end = r1 if causal else S
                ro, rl = o_attn.attention_ref(q[1:2, 3:4, r0:r1], k[1:2, 3:4, :kv_end], v[1:2, 3:4, :kv_end], sc, causal)
                torch.testing.assert_close(o[1:2, 3:4, r0:r1].cpu().float(), ro.float(), rtol=1e-2, atol=1e-2)
                torch.testing.assert_close(lse[1:2, 3:4, r0:r1].cpu(), rl, rtol=0, atol=1e-3)
            if causal:
                torch.testing.assert_close(o[:, :, 0].cpu().float(), v[:, :, 0].float(), rtol=1e-2, atol=1e-2)
            o1, _ = attention_with_lse(qd, kd, ones, sc, causal)
            torch.testing.assert_close(o1.float(), torch.ones_like(o1, dtype=torch.float32), rtol=0, atol=8e-3)
    _lib.sync_check()


def test_argument_checks(cuda):
    from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention
    q = torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(AssertionError):
        attention(q, q[..., :64].contiguous(), q, 1.0, False)
    with pytest.raises(RuntimeError):
        attention(q.cpu(), q.cpu(), q.cpu(), 1.0, False)
