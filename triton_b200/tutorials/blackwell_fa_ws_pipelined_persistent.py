"""``attention(q, k, v, sm_scale, causal, config=None)`` — counterpart of the reference's Blackwell
flash-attention forward, ``third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent.py:3491``.

q, k, v: ``[B, H, S, D]`` fp16 or bf16 CUDA tensors with equal head dims; returns ``o`` with the shape
and dtype of ``q``. Like the reference (``_attention``, ``:3285-3488``) the call is an autograd Function
when an input requires grad: ``backward`` runs the backward kernel (built for head_dim 128; 16, 32 and 64 run
zero-padded) and returns
``dq, dk, dv`` in the input dtype; ``attention_backward`` is the same step as a plain function.
The reference keeps the row statistic ``M = m*sm_scale*log2(e) + log2(l)`` (base-2 log-sum-exp, ``:886-894``) internal;
``attention_with_lse`` returns it as a second fp32 ``[B, H, S]`` tensor without changing the
signature of ``attention``. ``config`` is accepted for call compatibility (the tiling is fixed:
256 query rows per CTA as two groups of 128, KV blocks of 128; head dim 256: one group of 128 rows). Head dims of the
reference's set (``:3291-3292``): 64, 128 and 256 natively in the forward pass, 16 and 32 zero-padded to 64; the
backward pass serves up to 128.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


def _pad_head_dim(t, d):
    return torch.nn.functional.pad(t, (0, d - t.shape[-1])) if t.shape[-1] < d else t


def attention_with_lse(q, k, v, sm_scale, causal, config=None):
    HEAD_DIM_Q, HEAD_DIM_K, HEAD_DIM_V = q.shape[-1], k.shape[-1], v.shape[-1]
    assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V
    assert HEAD_DIM_K in {16, 32, 64, 128, 256}
    if not q.is_cuda:
        raise RuntimeError("triton_b200 attention needs CUDA tensors (there is no CPU path)")
    if HEAD_DIM_K < 64:
        # zero columns add nothing to q k^T (sm_scale is the caller's) and give zero output columns: the 64-wide
        # kernel serves head dims 16 and 32 at the cost of the padded work
        o, M = attention_with_lse(_pad_head_dim(q, 64), _pad_head_dim(k, 64), _pad_head_dim(v, 64), sm_scale, causal)
        return o[..., :HEAD_DIM_K].contiguous(), M
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4
    assert q.dtype in _DT and k.dtype == q.dtype and v.dtype == q.dtype
    assert k.shape == v.shape and q.shape[:2] == k.shape[:2]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, H, S, D = q.shape
    o = torch.empty_like(q)
    M = torch.empty((B, H, S), device=q.device, dtype=torch.float32)
    if q.numel() == 0:
        return o, M
    args = _lib.AttentionArgs()
    args.q, args.k, args.v, args.o, args.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), M.data_ptr()
    args.batch, args.heads, args.seq_q, args.seq_kv = B, H, S, k.shape[2]
    args.head_dim = D
    args.dtype = _DT[q.dtype]
    args.causal = 1 if causal else 0
    args.sm_scale = float(sm_scale)
    with _lib.device_guard(q.device):
        rc = _lib.lib().tb200_attention_fwd(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(q.device)))
    _lib.check(rc, "tb200_attention_fwd")
    return o, M


def attention_backward(q, k, v, o, lse, do, sm_scale, causal):
    """dq, dk, dv for ``o, lse = attention_with_lse(q, k, v, sm_scale, causal)`` and the output gradient
    ``do`` (the reference's ``_attention.backward``, ``:3362``). The kernel is built for head_dim 128; 16, 32 and 64
    run zero-padded."""
    if not q.is_cuda:
        raise RuntimeError("triton_b200 attention needs CUDA tensors (there is no CPU path)")
    if q.shape[-1] not in (16, 32, 64, 128):
        raise NotImplementedError(f"attention backward: head_dim {q.shape[-1]} (16, 32, 64 and 128 are implemented)")
    if q.shape[-1] < 128:
        # the backward kernel is built for 128: smaller head dims run zero-padded (zero columns of q, k, v, o and do
        # contribute nothing to the scores, to Delta or to the other columns' gradients)
        d = q.shape[-1]
        dq, dk, dv = attention_backward(*(_pad_head_dim(t, 128) for t in (q, k, v, o)), lse,
                                        _pad_head_dim(do.to(q.dtype), 128), sm_scale, causal)
        return dq[..., :d].contiguous(), dk[..., :d].contiguous(), dv[..., :d].contiguous()
    assert q.dtype in _DT and k.dtype == q.dtype and v.dtype == q.dtype and o.dtype == q.dtype
    assert o.shape == q.shape and do.shape == q.shape and k.shape == v.shape
    q, k, v, o = q.contiguous(), k.contiguous(), v.contiguous(), o.contiguous()
    do = do.to(q.dtype).contiguous()
    lse = lse.contiguous()
    assert lse.dtype == torch.float32 and lse.shape == q.shape[:3]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if q.numel() == 0 or k.numel() == 0:
        return dq.zero_(), dk.zero_(), dv.zero_()
    B, H, S, D = q.shape
    args = _lib.AttentionBwdArgs()
    args.q, args.k, args.v, args.o, args.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), do.data_ptr()
    args.lse = lse.data_ptr()
    args.dq, args.dk, args.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    args.batch, args.heads, args.seq_q, args.seq_kv = B, H, S, k.shape[2]
    args.head_dim = D
    args.dtype = _DT[q.dtype]
    args.causal = 1 if causal else 0
    args.sm_scale = float(sm_scale)
    need = _lib.lib().tb200_attention_bwd_workspace_bytes(ctypes.byref(args))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    args.workspace, args.workspace_bytes = ws.data_ptr(), need
    with _lib.device_guard(q.device):
        rc = _lib.lib().tb200_attention_bwd(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(q.device)))
    _lib.check(rc, "tb200_attention_bwd")
    return dq, dk, dv


class _attention(torch.autograd.Function):
    """Forward + saved (q, k, v, o, M); backward through ``attention_backward``."""

    @staticmethod
    def forward(ctx, q, k, v, sm_scale, causal):
        o, M = attention_with_lse(q, k, v, sm_scale, causal)
        ctx.save_for_backward(q, k, v, o, M)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, M = ctx.saved_tensors
        dq, dk, dv = attention_backward(q, k, v, o, M, do, ctx.sm_scale, ctx.causal)
        return dq, dk, dv, None, None


def attention(q, k, v, sm_scale, causal, config=None):
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return _attention.apply(q, k, v, sm_scale, causal)
    return attention_with_lse(q, k, v, sm_scale, causal, config)[0]
