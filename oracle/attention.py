"""Oracle for flash-attention forward and backward (test infrastructure only).

The reference checks its kernel against ``F.scaled_dot_product_attention(q, k, v, scale=sm_scale,
is_causal=causal)`` (``third_party/tlx/tutorials/testing/test_correctness.py:425-435``). Its
kernel also produces the row statistic ``M = m * sm_scale * log2(e) + log2(l)``
(``blackwell_fa_ws_pipelined_persistent.py:886-894``), i.e. the base-2 log-sum-exp of the scaled
scores. Both are restated here in fp32, one (batch, head) at a time to bound memory.
"""
import math

import torch


def attention_ref(q, k, v, sm_scale: float, causal: bool):
    """q, k, v: (B, H, S, D). Returns (o in q.dtype, lse2 fp32 (B, H, S))."""
    q32, k32, v32 = (t.detach().cpu().float() for t in (q, k, v))
    B, H, S, D = q32.shape
    Sk = k32.shape[2]
    o = torch.empty(B, H, S, v32.shape[3], dtype=torch.float32)
    lse2 = torch.empty(B, H, S, dtype=torch.float32)
    mask = None
    if causal:
        mask = torch.ones(S, Sk, dtype=torch.bool).tril(diagonal=Sk - S)
    for b in range(B):
        for h in range(H):
            s = (q32[b, h] @ k32[b, h].t()) * sm_scale
            if mask is not None:
                s = s.masked_fill(~mask, float("-inf"))
            lse = torch.logsumexp(s, dim=-1)
            p = torch.exp(s - lse[:, None])
            o[b, h] = p @ v32[b, h]
            lse2[b, h] = lse * math.log2(math.e)
    return o.to(q.dtype), lse2


def attention_bwd_ref(q, k, v, do, sm_scale: float, causal: bool):
    """Gradients of ``sum(attention(q, k, v) * do)`` restated from the formulas the reference's
    backward kernel implements (``blackwell_fa_ws_pipelined_persistent.py:1252-1266`` Delta,
    ``:2272-2440`` P, dS; dV = P^T dO, dK = sm_scale dS^T Q, dQ = sm_scale dS K), in fp64.
    The reference's own test compares with torch autograd (``testing/test_correctness.py:919-1068``);
    ``tests/test_oracle.py`` pins this restatement against autograd the same way.
    Returns (dq, dk, dv) in fp32 on the CPU."""
    q64, k64, v64, do64 = (t.detach().cpu().double() for t in (q, k, v, do))
    B, H, S, D = q64.shape
    Sk = k64.shape[2]
    dq = torch.empty(B, H, S, D, dtype=torch.float64)
    dk = torch.empty(B, H, Sk, D, dtype=torch.float64)
    dv = torch.empty(B, H, Sk, D, dtype=torch.float64)
    mask = torch.ones(S, Sk, dtype=torch.bool).tril(diagonal=Sk - S) if causal else None
    for b in range(B):
        for h in range(H):
            s = (q64[b, h] @ k64[b, h].t()) * sm_scale
            if mask is not None:
                s = s.masked_fill(~mask, float("-inf"))
            p = torch.softmax(s, dim=-1)
            o = p @ v64[b, h]
            delta = (o * do64[b, h]).sum(dim=-1, keepdim=True)
            dp = do64[b, h] @ v64[b, h].t()
            ds = p * (dp - delta)
            dv[b, h] = p.t() @ do64[b, h]
            dk[b, h] = sm_scale * (ds.t() @ q64[b, h])
            dq[b, h] = sm_scale * (ds @ k64[b, h])
    return dq.float(), dk.float(), dv.float()


def attention_mxfp8_ref(q, k, v, q_scale, k_scale, v_scale, sm_scale: float, causal: bool):
    """MXFP8 attention as the product of the dequantised operands in fp32: q, k, v ``[Z, H, N, D]`` e4m3; the
    scales as flat 512-byte atoms (``oracle.mxfp8.swizzle_scales`` order) - Q and K per 32 values of D, V per 32
    keys of each head-dim column (its transpose ``[D, Z*H*N]`` was quantised). This is the check of the reference's own
    test (``third_party/tlx/tutorials/testing/test_correctness.py:1071-1106``: SDPA on the unquantised tensors,
    absolute tolerance 0.04-0.11), applied to the dequantised tensors so that only the kernel's own rounding (the
    quantised probabilities, the bf16 output) is left. Returns ``(o fp32, lse2)``."""
    from . import mxfp8 as mx
    Z, H, N, D = q.shape
    Nk = k.shape[2]
    def dq(x2d, atoms):  # the atoms cover the matrix padded to 128 rows x 4 blocks
        rows, cols = x2d.shape
        rp, bp = -(-rows // 128) * 128, -(-(cols // 32) // 4) * 4
        xp = torch.zeros(rp, bp * 32, dtype=torch.float32)
        xp[:rows, :cols] = x2d.float()
        sc = mx.unswizzle_scales(atoms.reshape(-1).cpu().view(torch.uint8), rp, bp)
        return (xp * mx.e8m0_to_float(sc).repeat_interleave(32, dim=1))[:rows, :cols]
    qd = dq(q.reshape(Z * H * N, D).cpu(), q_scale).reshape(Z, H, N, D)
    kd = dq(k.reshape(Z * H * Nk, D).cpu(), k_scale).reshape(Z, H, Nk, D)
    vt = v.reshape(Z * H * Nk, D).t().contiguous().cpu()            # [D, ZHN]: the matrix that was quantised
    vd = dq(vt, v_scale).t().reshape(Z, H, Nk, D)
    return attention_ref(qd, kd, vd, sm_scale, causal)
