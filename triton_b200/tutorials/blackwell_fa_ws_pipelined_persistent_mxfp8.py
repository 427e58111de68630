"""``attention(q, k, v, q_scale, k_scale, v_scale, sm_scale, causal, config=None)`` — counterpart of the reference's
MXFP8 flash-attention forward, ``third_party/tlx/tutorials/blackwell_fa_ws_pipelined_persistent_mxfp8.py:3374``.

Same contract: ``q``, ``k``, ``v`` are ``[Z, H, N_CTX, HEAD_DIM]`` ``float8_e4m3fn``; the scales are e8m0 bytes, one per
32 values, in the 512-byte-atom ("swizzled") order the reference builds with ``MXTensor.to_mx(...,
is_swizzled_scales=True)`` and ``swizzled_to_tma_preshuffled`` (``:3290-3371``): Q and K quantised along
``HEAD_DIM``, V along the sequence (its transpose ``[HEAD_DIM, Z*H*N_CTX]`` is what was quantised). The scale tensors
may have any shape (the reference's is ``[Z*H, blocks, 1, 2, 256]``) as long as their bytes are the atoms in
``(batch*head, 128-row block)`` order. The result is a new bf16 tensor of ``q``'s shape. ``HEAD_DIM`` 128 (and 64,
zero-padded to 128: the reference's test runs both) and sequence lengths that are multiples of 128 are implemented.

``generate_attention_inputs(shape, device, dtype)`` mirrors the reference's helper of the same name (``:3320-3371``)
with this library's own quantiser (``triton_kernels.numerics_details.mxfp.downcast_to_mxfp``, scale rounded up) in
place of torchao's ``MXTensor``.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib


def swizzle_block_scales(scales: torch.Tensor) -> torch.Tensor:
    """``[rows, blocks]`` e8m0 bytes (padded to a multiple of 128 rows and of 4 blocks) -> the 512-byte atoms
    ``[rows/128][blocks/4][row % 32][row / 32 % 4][block % 4]``, flat."""
    rows, cols = scales.shape
    if rows % 128 or cols % 4:  # whole 128 x 4 atoms, zero bytes in the unused slots (what the reference's layout does)
        scales = torch.nn.functional.pad(scales, (0, (-cols) % 4, 0, (-rows) % 128))
        rows, cols = scales.shape
    t = scales.reshape(rows // 128, 4, 32, cols // 4, 4)  # [rb][row/32][row%32][cb][c%4]
    return t.permute(0, 3, 2, 1, 4).contiguous().reshape(-1)


def swizzled_to_tma_preshuffled(swizzled_scales: torch.Tensor, M: int, K: int, block_size: int, batch: int):
    """The reference's view of the flat atoms: ``(batch, ceil(M/128), ceil(K/block_size/4), 2, 256)``."""
    B = (M + 127) // 128
    C = (K // block_size + 3) // 4
    return swizzled_scales.view(batch, B, C, 2, 256)


def generate_attention_inputs(shape, device, dtype=torch.float8_e4m3fn):
    """Returns ``((q, q_scale, q_ref), (k, k_scale, k_ref), (v, v_scale, v_ref))``: MXFP8 values, swizzled scales and
    the bf16 tensors they were quantised from (N(0, 0.5), as in the reference)."""
    from ..triton_kernels.numerics_details.mxfp import downcast_to_mxfp
    assert dtype == torch.float8_e4m3fn
    Z, H, N, D = shape
    refs = [torch.empty(shape, device=device, dtype=torch.bfloat16).normal_(mean=0.0, std=0.5) for _ in range(3)]
    out = []
    for i, ref in enumerate(refs):
        x2d = ref.reshape(Z * H * N, D)
        if i < 2:  # Q, K: blocks of 32 along the head dimension
            val, sc = downcast_to_mxfp(x2d, dtype, axis=1)                      # [ZHN, D], [ZHN, D/32]
            data = val.reshape(shape).contiguous()
            scale = swizzled_to_tma_preshuffled(swizzle_block_scales(sc), N, D, 32, Z * H)
        else:      # V: its transpose [D, ZHN] is quantised along the sequence
            val, sc = downcast_to_mxfp(x2d.t().contiguous(), dtype, axis=1)     # [D, ZHN], [D, ZHN/32]
            data = val.t().reshape(shape).contiguous()
            scale = swizzled_to_tma_preshuffled(swizzle_block_scales(sc), D, N, 32, Z * H)
        out.append((data, scale, ref))
    return tuple(out)


def _attention_d64(q, k, v, q_scale, k_scale, v_scale, sm_scale, causal):
    """Head dim 64 through the 128-wide kernel: zero value columns (they add nothing to q k^T and give zero output
    columns) and scale 1.0 in the atoms' unused slots - blocks 2, 3 of every row for Q and K, rows 64..127 for V
    (the reference's swizzled layout pads its atoms to 128 rows x 4 blocks, so the atom counts are the same)."""
    Z, H, N, D = q.shape
    Nk = k.shape[2]
    pad = lambda t: torch.nn.functional.pad(t.view(torch.uint8), (0, 64)).view(torch.float8_e4m3fn)
    qs, ks, vs = (t.contiguous().view(torch.uint8).reshape(-1, 32, 4, 4).clone() for t in (q_scale, k_scale, v_scale))
    assert qs.shape[0] == Z * H * N // 128 and ks.shape[0] == Z * H * Nk // 128 and vs.shape[0] == Z * H * Nk // 128, \
        "scale tensor: one 512-byte atom per 128 rows"
    qs[:, :, :, 2:] = 127   # [row % 32][row / 32][block]: blocks 2, 3 cover head-dim columns 64..127
    ks[:, :, :, 2:] = 127
    vs[:, :, 2:, :] = 127   # rows = head-dim columns: 64..127 are padding
    o = attention(pad(q), pad(k), pad(v), qs, ks, vs, sm_scale, causal)
    return o[..., :64].contiguous()


def attention(q, k, v, q_scale, k_scale, v_scale, sm_scale, causal, config=None):
    """MXFP8 flash-attention forward (``tb200_attention_mxfp8_fwd``); ``config`` is accepted and ignored (the tiling is
    the kernel's own)."""
    assert q.dim() == 4 and q.shape[-1] == k.shape[-1] == v.shape[-1]
    if not q.is_cuda:
        raise RuntimeError("triton_b200 attention needs CUDA tensors (there is no CPU path)")
    assert q.dtype == k.dtype == v.dtype == torch.float8_e4m3fn, "MXFP8 attention takes float8_e4m3fn values"
    Z, H, N, D = q.shape
    Nk = k.shape[2]
    if D == 64:
        return _attention_d64(q, k, v, q_scale, k_scale, v_scale, sm_scale, causal)
    if D != 128:
        raise NotImplementedError("MXFP8 attention: head dims 64 and 128 are implemented")
    if N % 128 or Nk % 128:
        raise NotImplementedError("MXFP8 attention: sequence lengths must be multiples of 128 (whole scale atoms)")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    scales = []
    for t, n_atoms in ((q_scale, Z * H * N // 128), (k_scale, Z * H * Nk // 128), (v_scale, Z * H * Nk // 128)):
        t = t.contiguous().view(torch.uint8) if t.dtype != torch.uint8 else t.contiguous()
        assert t.numel() == n_atoms * 512, "scale tensor: one 512-byte atom per 128 rows"
        scales.append(t)
    o = torch.empty((Z, H, N, D), dtype=torch.bfloat16, device=q.device)
    if o.numel() == 0:
        return o
    args = _lib.AttentionMxfp8Args()
    args.q, args.k, args.v, args.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    args.q_scale, args.k_scale, args.v_scale = (s.data_ptr() for s in scales)
    args.lse = None
    args.batch, args.heads, args.seq_q, args.seq_kv = Z, H, N, Nk
    args.head_dim, args.causal, args.sm_scale = D, int(bool(causal)), float(sm_scale)
    with _lib.device_guard(q.device):
        rc = _lib.lib().tb200_attention_mxfp8_fwd(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(q.device)))
    _lib.check(rc, "tb200_attention_mxfp8_fwd")
    return o
