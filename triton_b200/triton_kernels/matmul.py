"""``matmul(a, b, bias, a_ragged_metadata=None, ..., gather_indx=None, scatter_indx=None, ...,
gammas=None, ..., fused_activation=None, ...)`` — counterpart of ``triton_kernels/matmul.py:243`` in
the reference for the bf16/fp16 MoE subset: per-expert GEMM over expert-sorted rows with the row
gather fused into the load and bias, SwiGLU, per-row gammas and row scatter fused into the epilogue.
``fused_comm`` fuses the expert-parallel combine: the epilogue stores each output row straight into the
buffer of the rank that owns the token (peer stores over NVLink; the reference's fused-comm epilogue,
``matmul_details/_p_matmul.py:755-782``).
``betas`` (per-row factor on the bias), ``out_alpha`` and ``c_acc_in`` (a matrix added to the result) follow the
reference's epilogue order (``_p_matmul.py:606-622``).
``precision_config.c_mx_scale`` with ``epilogue=Epilogue(FnSpecs(FnName.QUANTIZE_MXFP8.name, quantize_mxfp8_fn, ...))``
returns the output MX-quantised (fp8 values + one e8m0 scale per 32 outputs of a row written to ``c_mx_scale``,
``matmul.py:362-366`` / ``_p_matmul.py:650-704``); ``precision_config.a_mx_scale`` makes the fp8 activations of the
MXFP4-weight path MXFP8 (one e8m0 scale per 32 values of K, fed to the block-scaled MMA).
Batched inputs (``[B, M, K] x [B, K, N]``) run as the grouped kernel with one slice per batch entry; ragged K
(``b_ragged_metadata``) as one dense GEMM per slice.
Unsupported combinations (flexpoint / NVFP4 precision, other epilogues) raise
``NotImplementedError``, as the reference does for combinations it
cannot serve (``:288,437-447,467``)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from enum import Enum, auto

import torch

from .. import _lib
from .numerics import InFlexData, OutFlexData
from .swiglu import swiglu_fn
from .tensor import RaggedTensorMetadata, make_ragged_tensor_metadata

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}


@dataclass(frozen=True)
class FnSpecs:
    name: str
    fn: object
    fn_arg_names: tuple = tuple()
    fn_arg_do_not_specialize: tuple = tuple()
    reduction_n: int = 1

    @staticmethod
    def default():
        return FnSpecs("dflt", None, tuple())


class FnName(Enum):
    """Names of the quantising epilogues (``triton_kernels/matmul.py:53-56`` in the reference)."""
    QUANTIZE_MXFP8 = auto()
    QUANTIZE_MXFP4 = auto()
    QUANTIZE_NVFP4 = auto()


@dataclass(frozen=True)
class FusedActivation:
    specs: FnSpecs = FnSpecs.default()
    fn_args: tuple = tuple()


@dataclass(frozen=True)
class Epilogue:
    specs: FnSpecs = FnSpecs.default()
    fn_arg_values_matmul: tuple = tuple()
    fn_arg_values_finalize: tuple = tuple()
    effective_itemsize: float | None = None


@dataclass(frozen=True)
class FlexCtx:
    """Per-tensor scales of the operands and the output (``triton_kernels/matmul.py:116-121``)."""
    lhs_data: InFlexData = InFlexData()
    rhs_data: InFlexData = InFlexData()
    out_data: OutFlexData = OutFlexData()
    acc_data: InFlexData = InFlexData()


@dataclass
class PrecisionConfig:
    max_num_imprecise_acc: int | None = None
    allow_tf32: bool = True
    flex_ctx: FlexCtx = FlexCtx()  # honoured on the fp8 x MXFP4 path (scalar scales); must be empty elsewhere
    acc_scale: float = 1.0
    flexpoint_saturate_inf: bool = False
    out_dtype: torch.dtype | None = None
    a_mx_scale: object = None  # e8m0 block scales of MXFP8 activations: [rows, K/32] uint8 (with an MXFP4 weight)
    a_microblock_size: int | None = None
    b_mx_scale: object = None  # e8m0 scales of an MXFP4 weight: [E, K/32, N] uint8, or the Tensor convert_layout returns
    b_microblock_size: int | None = None
    # MX-quantised output (with epilogue = Epilogue(FnSpecs(FnName.QUANTIZE_MXFP8.name, quantize_mxfp8_fn, ...))): a
    # [rows, ceil(N_out / 32)] uint8 tensor that receives the e8m0 scales; the values come back as fp8
    c_mx_scale: object = None
    c_microblock_size: int | None = None
    x_scale: object = None     # one fp32 value multiplying the fp8 activations (the reference's flexpoint scale)


@dataclass(frozen=True)
class FusedComm:
    """Destination of a matmul whose output rows leave this GPU (``triton_kernels/matmul.py:59-81`` in the
    reference, where the row -> (shard, row) map is a jitted closure). Here the map is the one the
    expert-parallel combine needs, stated declaratively: the row with output index ``i`` (``scatter_indx[r]``,
    or ``r`` without a scatter) is stored to row ``i % rows_per_shard`` of ``out_handles[i // rows_per_shard]``.
    ``out_handles``: one entry per shard, a CUDA tensor of this process or any object with ``data_ptr()``
    (a peer's buffer mapped through ``SymmetricMemoryPool``); each ``[rows_per_shard, n_out]`` with row pitch
    ``row_stride`` elements. The stores are plain: barrier (``hdl.barrier()``) before any rank reads."""
    out_handles: tuple
    rows_per_shard: int
    row_stride: int | None = None


def swiglu_activation(alpha: float = 1.0, limit: float | None = None) -> FusedActivation:
    """The fused SwiGLU spec the reference builds as
    ``FusedActivation(FnSpecs("swiglu", swiglu_fn, ("alpha", "limit"), reduction_n=2), (alpha, limit))``."""
    return FusedActivation(FnSpecs("swiglu", swiglu_fn, ("alpha", "limit"), reduction_n=2), (alpha, limit))


def matmul(a, b, bias, a_ragged_metadata: RaggedTensorMetadata | None = None, b_ragged_metadata=None,
           gather_indx=None, scatter_indx=None, precision_config: PrecisionConfig | None = None, betas=None,
           gammas=None, out_alpha=None, c=None, fused_comm=None, fused_activation: FusedActivation | None = None,
           epilogue: Epilogue | None = None, c_acc_in=None, _tile_mode: int = 0, _gammas_by_out_row: bool = False):
    if isinstance(c, torch.Tensor) and c.ndim >= 2 and c.stride(-1) != 1 and fused_comm is None:
        # a transposed (column-major) output buffer, as the reference's c_transpose cases pass: the kernels write
        # rows, so the product is formed in a row-major temporary and copied over
        out = matmul(a, b, bias, a_ragged_metadata, b_ragged_metadata, gather_indx, scatter_indx, precision_config, betas,
                     gammas, out_alpha, None, None, fused_activation, epilogue, c_acc_in, _tile_mode, _gammas_by_out_row)
        assert out.shape == c.shape and out.dtype == c.dtype, "c does not match the product's shape or dtype"
        c.copy_(out)
        return c
    if b_ragged_metadata is not None:
        if (gather_indx is not None or scatter_indx is not None or fused_comm is not None or c_acc_in is not None
                or (fused_activation is not None and fused_activation.specs.name != "dflt")
                or (epilogue is not None and epilogue.specs.name != "dflt")
                or (precision_config is not None and (precision_config.a_mx_scale is not None
                                                      or precision_config.b_mx_scale is not None
                                                      or precision_config.c_mx_scale is not None))):
            raise NotImplementedError("matmul (ragged K): plain 16-bit products only")
        return _matmul_ragged_k(a, b, a_ragged_metadata, b_ragged_metadata, c)
    if isinstance(a, torch.Tensor) and a.ndim == 3 and isinstance(b, torch.Tensor) and b.ndim == 3 \
            and a_ragged_metadata is None:
        return _matmul_batched(a, b, bias, precision_config, betas, gammas, out_alpha, c, fused_comm, fused_activation,
                               epilogue, c_acc_in, gather_indx, scatter_indx, _tile_mode)
    if (betas is not None or out_alpha is not None or c_acc_in is not None) and precision_config is not None \
            and precision_config.b_mx_scale is not None:
        raise NotImplementedError("matmul: betas / out_alpha / c_acc_in with an MXFP4 weight are not implemented")
    if c_acc_in is not None and (scatter_indx is not None or fused_comm is not None):
        raise NotImplementedError("matmul: c_acc_in with a scatter index or fused communication (as in the reference)")
    if fused_comm is not None and (c is not None or (precision_config is not None
                                                     and precision_config.b_mx_scale is not None)):
        raise NotImplementedError("matmul: fused_comm takes the 16-bit path and owns the output buffers")
    quantize_out = False
    if epilogue is not None and epilogue.specs.name != "dflt":
        if epilogue.specs.name != FnName.QUANTIZE_MXFP8.name:
            raise NotImplementedError(f"matmul: epilogue {epilogue.specs.name!r} (the MXFP8 quantising epilogue is implemented)")
        if precision_config is None or precision_config.c_mx_scale is None:
            raise ValueError("matmul: the quantising epilogue needs precision_config.c_mx_scale")
        quantize_out = True
    if precision_config is not None and precision_config.c_mx_scale is not None:
        if not quantize_out:
            raise ValueError("matmul: precision_config.c_mx_scale needs epilogue = the MXFP8 quantising epilogue")
        if fused_comm is not None:
            raise NotImplementedError("fused comm with output MX scales is not supported")  # as the reference (:287)
        if c_acc_in is not None or c is not None:
            raise NotImplementedError("matmul: MX-quantised output with c / c_acc_in is not implemented")
        if precision_config.c_microblock_size not in (None, 32):
            raise NotImplementedError("matmul: microblock size 32 (e8m0 scales) only")
    fp8_w = isinstance(b, torch.Tensor) and b.dtype in _F8
    if fp8_w and isinstance(a, torch.Tensor) and a.dtype in _F8 and (precision_config is None
                                                                   or precision_config.b_mx_scale is None):
        # fp8 x fp8 (tensor-wide flexpoint scales, or none): the block-scaled kernel with scale columns of 1.0
        if precision_config is not None and precision_config.a_mx_scale is not None:
            raise NotImplementedError("matmul: MX-scaled activations need an MX-scaled weight (b_mx_scale)")
        if betas is not None or out_alpha is not None or c_acc_in is not None or fused_comm is not None:
            raise NotImplementedError("matmul (fp8 weights): betas / out_alpha / c_acc_in / fused_comm are not implemented")
        if gather_indx is not None:
            a = _gather_fp8_rows(a, gather_indx)
        return _matmul_mx4(a, b, bias, a_ragged_metadata, scatter_indx, precision_config or PrecisionConfig(), gammas,
                           fused_activation, c)
    if precision_config is not None and precision_config.a_mx_scale is not None and precision_config.b_mx_scale is None \
            and isinstance(a, torch.Tensor) and a.dtype in _F8 and isinstance(b, torch.Tensor) and b.dtype in _DT:
        # mxfloat8 activations x 16-bit weights (tests/test_matmul.py:217-224 in the reference): the activations are
        # upcast to the weight dtype with torch ops, then the 16-bit grouped GEMM runs
        import dataclasses
        from .numerics_details.mxfp import upcast_from_mxfp
        if precision_config.a_microblock_size not in (None, 32):
            raise NotImplementedError("matmul: microblock size 32 (e8m0 scales) only")
        a16 = upcast_from_mxfp(a, _plain_scale(precision_config.a_mx_scale), b.dtype, axis=a.ndim - 1)
        pc16 = dataclasses.replace(precision_config, a_mx_scale=None, a_microblock_size=None)
        return matmul(a16, b, bias, a_ragged_metadata, b_ragged_metadata, gather_indx, scatter_indx, pc16, betas, gammas,
                      out_alpha, c, fused_comm, fused_activation, epilogue, c_acc_in, _tile_mode, _gammas_by_out_row)
    if precision_config is not None and precision_config.a_mx_scale is not None:
        if precision_config.b_mx_scale is None or not isinstance(a, torch.Tensor) or a.dtype not in _F8:
            raise NotImplementedError("matmul: MX-scaled activations are implemented as MXFP8 x MXFP4 "
                                      "(fp8 values, precision_config.a_mx_scale and b_mx_scale)")
        if precision_config.a_microblock_size not in (None, 32):
            raise NotImplementedError("matmul: microblock size 32 (e8m0 scales) only")
    if precision_config is not None and precision_config.b_mx_scale is not None:
        if isinstance(a, torch.Tensor) and a.dtype in _DT:
            if _flex_in_use(precision_config.flex_ctx):
                raise NotImplementedError("matmul: flexpoint scales are implemented for fp8 activations x MXFP4 weights")
            # 16-bit activations: the weight is upcast to the activation dtype (what the reference's
            # tl.dot_scaled(x, None, "bf16", w, w_scales, "e2m1") computes), then the 16-bit grouped GEMM runs
            if fp8_w:  # MXFP8 weight (bfloat16 x mxfloat8 in the reference's test list): upcast with torch ops
                from .numerics_details.mxfp import upcast_from_mxfp
                if precision_config.b_microblock_size not in (None, 32):
                    raise NotImplementedError("matmul (MXFP8 weight): microblock size 32 (e8m0 scales) only")
                b3 = b if b.ndim == 3 else b.unsqueeze(0)
                sc = _plain_scale(precision_config.b_mx_scale)
                w16 = upcast_from_mxfp(b3, sc if sc.ndim == 3 else sc.unsqueeze(0), a.dtype, axis=1)
            else:
                w16 = upcast_mxfp4_weight(b, precision_config.b_mx_scale, a.dtype,
                                          precision_config.b_microblock_size)
            pc16 = PrecisionConfig(out_dtype=precision_config.out_dtype, c_mx_scale=precision_config.c_mx_scale,
                                   c_microblock_size=precision_config.c_microblock_size)
            return matmul(a, w16, bias, a_ragged_metadata, None, gather_indx, scatter_indx, pc16, None, gammas,
                          None, c, None, fused_activation, epilogue, None, _tile_mode)
        if gather_indx is not None:
            # this kernel reads sorted rows only: indexed rows are gathered by a pass of their own first
            a = _gather_fp8_rows(a, gather_indx)
            if precision_config.a_mx_scale is not None:  # the rows' block scales travel with them
                import dataclasses
                sc = _plain_scale(precision_config.a_mx_scale)
                precision_config = dataclasses.replace(precision_config, a_mx_scale=_gather_scale_rows(sc, gather_indx))
        return _matmul_mx4(a, b, bias, a_ragged_metadata, scatter_indx, precision_config, gammas, fused_activation, c)
    if precision_config is not None and _flex_in_use(precision_config.flex_ctx):
        raise NotImplementedError("matmul: flexpoint scales are implemented for fp8 activations x MXFP4 weights")
    if not isinstance(a, torch.Tensor) or not isinstance(b, torch.Tensor):
        raise NotImplementedError("matmul: wrapped Tensor operands need precision_config.b_mx_scale (MXFP4 weights)")
    if a.ndim != 2:
        raise NotImplementedError("matmul: batched input is not implemented")
    if not a.is_cuda:
        raise RuntimeError("triton_b200 matmul needs CUDA tensors (there is no CPU path)")
    if a.dtype not in _DT or b.dtype != a.dtype:
        raise NotImplementedError(f"matmul: dtype {a.dtype}/{b.dtype} (bf16 and fp16 are implemented)")
    dev = a.device
    if b.ndim == 2:
        b = b.unsqueeze(0)
    E, K, N = b.shape
    assert a.shape[1] == K, "inner dimensions differ"
    if a.stride(1) != 1:
        a = a.contiguous()
    # weight layout: [E, K, N] with N contiguous, or K contiguous (the reference's benches store W
    # column-major per expert)
    if b.stride(2) == 1 and b.stride(1) == N and b.stride(0) == K * N:
        w_n_major = 1
    elif b.stride(1) == 1 and b.stride(2) == K and b.stride(0) == K * N:
        w_n_major = 0
    else:
        b = b.contiguous()
        w_n_major = 1

    swiglu, alpha, limit = 0, 1.0, None
    if fused_activation is not None and fused_activation.specs.name != "dflt":
        if fused_activation.specs.name != "swiglu":
            raise NotImplementedError(f"matmul: fused activation {fused_activation.specs.name!r}")
        swiglu = 1
        alpha = float(fused_activation.fn_args[0])
        limit = fused_activation.fn_args[1] if len(fused_activation.fn_args) > 1 else None
    n_out = N // 2 if swiglu else N

    R = a.shape[0] if gather_indx is None else gather_indx.shape[0]
    if gather_indx is not None and R >= _PREGATHER_MIN_ROWS and (K * a.element_size()) % 16 == 0 \
            and (a.stride(0) * a.element_size()) % 16 == 0 and a.data_ptr() % 16 == 0:
        # many rows: gather them in a pass of their own, so that the GEMM loads A with tiled TMA copies instead of
        # its gather warps' 16-byte copies (16384 tokens x top-4: the layer takes 3.29 ms instead of 3.90)
        a = _gather_rows(a, gather_indx)
        gather_indx = None
    if a_ragged_metadata is None:
        assert E == 1, "several weight matrices need a_ragged_metadata"
        a_ragged_metadata = make_ragged_tensor_metadata(torch.tensor([R], dtype=torch.int32, device=dev), R)
    md = a_ragged_metadata
    sched = md.block_schedule(128)
    rows_y = R if scatter_indx is None else scatter_indx.shape[0]
    out_dtype = a.dtype
    c_sf = None
    if quantize_out:
        # MX-quantised output: fp8 values (e4m3 unless out_dtype says e5m2) + the caller's scale tensor
        out_dtype = precision_config.out_dtype or torch.float8_e4m3fn
        if out_dtype not in _F8:
            raise NotImplementedError("matmul: MX-quantised output is fp8 (e4m3fn / e5m2)")
        c_sf = _plain_scale(precision_config.c_mx_scale)
        assert c_sf.shape == (rows_y, (n_out + 31) // 32) and c_sf.stride(1) == 1, \
            "c_mx_scale: [rows, ceil(N_out / 32)] uint8, row-major"
    elif precision_config is not None and precision_config.out_dtype not in (None, a.dtype):
        raise NotImplementedError("matmul: out_dtype different from the input dtype")
    peers = None
    if fused_comm is not None:
        peers = _lib.pointer_array([h.data_ptr() for h in fused_comm.out_handles])
        assert rows_y <= len(fused_comm.out_handles) * fused_comm.rows_per_shard
    elif c is None:
        # rows no sorted row maps to stay zero, as in the torch twin (matmul.py:902-906)
        c = (torch.zeros if scatter_indx is not None else torch.empty)((rows_y, n_out), dtype=out_dtype, device=dev)
    else:
        assert c.shape == (rows_y, n_out) and c.dtype == out_dtype and c.stride(1) == 1

    def i32(t):
        return None if t is None else t.to(torch.int32).contiguous()

    gi, si = i32(gather_indx), i32(scatter_indx)
    gm = None if gammas is None else gammas.float().contiguous()
    bs = None
    if bias is not None:
        bs = bias.float().reshape(E, N).contiguous()
    args = _lib.MoeGemmArgs()
    args.x, args.w = a.data_ptr(), b.data_ptr()
    if peers is not None:
        args.y, args.y_peers, args.y_world = None, peers, len(fused_comm.out_handles)
        args.rows_per_peer = fused_comm.rows_per_shard
    else:
        args.y = c.data_ptr()
    args.bias = bs.data_ptr() if bs is not None else None
    args.slice_offs, args.block_schedule = md.slice_offs.data_ptr(), sched.data_ptr()
    args.slice_sizes = md.slice_sizes.data_ptr()
    args.gather_indx = gi.data_ptr() if gi is not None else None
    args.scatter_indx = si.data_ptr() if si is not None else None
    args.gammas = gm.data_ptr() if gm is not None else None
    args.n_experts, args.k, args.n = E, K, N
    args.rows_x, args.rows_y = a.shape[0], rows_y
    args.ldx = a.stride(0)
    args.ldy = c.stride(0) if peers is None else (fused_comm.row_stride or n_out)
    args.n_sched = sched.shape[0]
    args.w_n_major = w_n_major
    args.dtype = _DT[a.dtype]
    args.swiglu = swiglu
    args.swiglu_alpha = alpha
    args.swiglu_limit = float(limit) if limit is not None else 0.0
    args.swiglu_has_limit = 1 if limit is not None else 0
    if betas is not None:
        bt = betas.float().contiguous()
        assert bt.numel() == R
        args.betas = bt.data_ptr()
    if out_alpha is not None:
        args.out_alpha, args.has_out_alpha = float(out_alpha), 1
    if c_acc_in is not None:
        assert c_acc_in.shape == c.shape and c_acc_in.dtype == c.dtype and c_acc_in.stride(1) == 1
        args.c_acc_in, args.ld_acc_in = c_acc_in.data_ptr(), c_acc_in.stride(0)
    if c_sf is not None:
        args.y_mx_scale, args.ld_y_mx_scale, args.y_mx_dtype = c_sf.data_ptr(), c_sf.stride(0), _F8[out_dtype]
    args.moe_tile_mode = int(_tile_mode)  # extension: 0 choose, 1 one CTA per block, 2 CTA pair per two blocks
    # extension: gammas holds one value per OUTPUT row (e.g. the top-k values in (token, slot) order) instead of per sorted row
    args.gammas_by_out_row = 1 if _gammas_by_out_row else 0
    with _lib.device_guard(dev):
        rc = _lib.lib().tb200_moe_gemm(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
    _lib.check(rc, "tb200_moe_gemm")
    return c if peers is None else fused_comm.out_handles


_F8 = {torch.float8_e4m3fn: _lib.E4M3, torch.float8_e5m2: _lib.E5M2}

_PREGATHER_MIN_ROWS = 2048


def _gather_rows(a, gather_indx):
    """``a[gather_indx]`` with zero rows for indices outside ``[0, a.shape[0])`` (``tb200_gather_rows``)."""
    gi = gather_indx.to(torch.int32).contiguous()
    out = torch.empty((gi.shape[0], a.shape[1]), dtype=a.dtype, device=a.device)
    esz = a.element_size()
    with _lib.device_guard(a.device):
        rc = _lib.lib().tb200_gather_rows(a.data_ptr(), a.stride(0) * esz, a.shape[0], out.data_ptr(), out.stride(0) * esz,
                                          gi.data_ptr(), gi.numel(), a.shape[1] * esz,
                                          ctypes.c_void_p(_lib.current_stream_ptr(a.device)))
    _lib.check(rc, "tb200_gather_rows")
    return out


def _matmul_batched(a, b, bias, precision_config, betas, gammas, out_alpha, c, fused_comm, fused_activation, epilogue,
                    c_acc_in, gather_indx, scatter_indx, _tile_mode):
    """Batched inputs ([B, M, K] x [B, K, N] -> [B, M, N], matmul.py:864-868 in the reference): the batch entries are
    the slices of the grouped kernel - entry i owns rows [i M, (i + 1) M) of the flattened activations and weight
    matrix i."""
    if gather_indx is not None or scatter_indx is not None:
        raise ValueError("gather / scatter are not supported in batched mode")  # asserted in the reference too
    if fused_comm is not None or c is not None or c_acc_in is not None or betas is not None or gammas is not None:
        raise NotImplementedError("matmul (batched): bias, fused activation and the quantising epilogue are implemented")
    B, M, K = a.shape
    assert b.shape[0] == B and b.shape[1] == K, "batched operands differ in batch size or inner dimension"
    md = make_ragged_tensor_metadata(torch.full((B, ), M, dtype=torch.int32, device=a.device), B * M)
    y = matmul(a.reshape(B * M, K), b, bias, md, None, None, None, precision_config, None, None, out_alpha, None, None,
               fused_activation, epilogue, None, _tile_mode)
    return y.view(B, M, y.shape[-1])


def _matmul_ragged_k(a, b, a_md, b_md, c):
    """Ragged K (``b_ragged_metadata``; the weight-gradient shape of an MoE layer, matmul.py:836-861 in the
    reference): ``out[e] = a[:, xo_e : xo_e + k_e] @ b[wo_e : wo_e + k_e, :]`` with the column slices of ``a``
    described by ``a_ragged_metadata`` (default: the same slices as ``b``) and the row slices of ``b`` by
    ``b_ragged_metadata``. One dense GEMM (``tb200_gemm``) per non-empty slice on operand views - the slice sizes
    are read back to the host once; slices must start on multiples of 8 elements (TMA alignment), as the
    reference asks of K-ragged operands (``slice_sizes_divisibility``)."""
    from ..tutorials.blackwell_gemm_ws import matmul as dense_matmul
    if not (isinstance(a, torch.Tensor) and isinstance(b, torch.Tensor) and a.ndim == 2 and b.ndim == 2):
        raise NotImplementedError("matmul (ragged K): 2-D torch tensors")
    if not a.is_cuda:
        raise RuntimeError("triton_b200 matmul needs CUDA tensors (there is no CPU path)")
    if a.dtype not in _DT or b.dtype != a.dtype:
        raise NotImplementedError(f"matmul (ragged K): dtype {a.dtype}/{b.dtype} (bf16 and fp16 are implemented)")
    a_md = a_md or b_md
    sizes = b_md.slice_sizes.tolist()
    xo, wo = a_md.slice_offs.tolist(), b_md.slice_offs.tolist()
    E, M, N = len(sizes), a.shape[0], b.shape[1]
    if c is None:
        c = torch.empty((E, M, N), dtype=a.dtype, device=a.device)
    assert c.shape == (E, M, N) and c.dtype == a.dtype and c.stride(2) == 1
    # row pitches that are no multiple of 16 bytes (N or K_total not a multiple of 8): work on padded copies
    n8 = (N + 7) // 8 * 8
    if a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16:
        a = torch.nn.functional.pad(a, (0, (-a.shape[1]) % 8))
    if n8 != N or b.stride(1) != 1 or b.stride(0) % 8 or b.data_ptr() % 16:
        b = torch.nn.functional.pad(b, (0, n8 - N))
    work = c if (n8 == N and c.stride(1) % 8 == 0 and c.data_ptr() % 16 == 0) else \
        torch.empty((E, M, n8), dtype=a.dtype, device=a.device)
    for e, k in enumerate(sizes):
        if k == 0:
            work[e].zero_()
            continue
        if xo[e] % 8 or wo[e] % 8:
            raise NotImplementedError("matmul (ragged K): slices must start on multiples of 8 elements")
        dense_matmul(a[:, xo[e]:xo[e] + k], b[wo[e]:wo[e] + k, :], out=work[e])
    if work is not c:
        c.copy_(work[..., :N])
    return c


def _flex_in_use(fc) -> bool:
    return fc is not None and any(t is not None for t in (fc.lhs_data.scale, fc.rhs_data.scale, fc.acc_data.scale,
                                                            fc.out_data.expected_scale, fc.out_data.actual_scale,
                                                            fc.out_data.checksum_scale))


def _flex_scalar(t, dev, what):
    """A flexpoint scale as a one-element fp32 tensor on ``dev`` (per-batch scales are not implemented)."""
    if t is None:
        return None
    t = torch.as_tensor(t, device=dev)
    if t.numel() != 1:
        raise NotImplementedError(f"matmul: per-batch {what} (one scale per tensor is implemented)")
    return t.to(torch.float32).reshape(1).contiguous()


def _plain_scale(t):
    """A scale tensor given plain or wrapped (strided layout) as the plain uint8 tensor."""
    from .tensor import Tensor
    if isinstance(t, Tensor):
        from .tensor_details.layout import StridedLayout
        if t.layout is not None and not isinstance(t.layout, StridedLayout):
            raise NotImplementedError("matmul: activation / output MX scales in a strided (row-major) layout only")
        t = t.data
    if t.dtype != torch.uint8:
        raise NotImplementedError("matmul: MX scales are e8m0 bytes (torch.uint8)")
    return t


def _gather_fp8_rows(a, gather_indx):
    """The fp8 kernels read sorted rows only: indexed rows are gathered by a pass of their own first."""
    if not isinstance(a, torch.Tensor) or a.ndim != 2 or not a.is_cuda:
        raise NotImplementedError("matmul (fp8 activations): gather_indx needs a 2-D CUDA activation tensor")
    if a.stride(1) != 1 or a.stride(0) % 16 or a.shape[1] % 16:
        a = a.contiguous()
    return _gather_rows(a.view(torch.uint8), gather_indx).view(a.dtype)


def _fp8_weight_kernel_layout(b, b_mx_scale, microblock):
    """An fp8 weight [E, K, N] as the [E, N, K] byte matrix the kernel reads (no copy when K is the contiguous
    dimension, which is how the reference lays fp8 weights out) and, for an MXFP8 weight, its [E, K/32, N] e8m0
    scales as 512-byte atoms [E][ceil(N/128)][ceil(K/128)][n % 32][n / 32 % 4][k / 32 % 4] (127 past N and K)."""
    if microblock not in (None, 32):
        raise NotImplementedError("matmul (MXFP8 weight): microblock size 32 (e8m0 scales) only")
    if b.ndim == 2:
        b = b.unsqueeze(0)
    E, K, N = b.shape
    if K % 16:
        raise NotImplementedError("matmul (fp8 weights): K must be a multiple of 16")
    w = b.transpose(1, 2)
    if not w.is_contiguous():
        w = w.contiguous()
    atoms = None
    if b_mx_scale is not None:
        sc = _plain_scale(b_mx_scale)
        if sc.ndim == 2:
            sc = sc.unsqueeze(0)
        assert sc.shape == (E, (K + 31) // 32, N), "b_mx_scale: [E, ceil(K / 32), N] e8m0 bytes"
        kb, nb = (K + 127) // 128, (N + 127) // 128
        full = torch.full((E, kb * 4, nb * 128), 127, dtype=torch.uint8, device=sc.device)
        full[:, :sc.shape[1], :N] = sc
        atoms = full.view(E, kb, 4, nb, 4, 32).permute(0, 3, 1, 5, 4, 2).contiguous()
    return w, atoms, (E, K, N)


def _gather_scale_rows(sc, gather_indx):
    if sc.stride(1) == 1 and sc.shape[1] % 16 == 0 and sc.stride(0) % 16 == 0:
        return _gather_rows(sc, gather_indx)
    gi = gather_indx.long()
    ok = (gi >= 0) & (gi < sc.shape[0])
    out = sc[gi.clamp(0, max(sc.shape[0] - 1, 0))]
    out[~ok] = 127
    return out


def _mx4_kernel_layout(b, b_mx_scale, microblock):
    """The weight and its scales as the Tensors the kernels read (converted here when given as plain uint8)."""
    from .tensor import FP4, Tensor, convert_layout, wrap_torch_tensor
    from .tensor_details.layout import (BlackwellMX4ValueLayout, BlackwellMXScaleLayout,
                                        make_default_matmul_mxfp4_w_layout, make_default_matmul_mxfp4_w_scale_layout)
    if microblock not in (None, 32):
        raise NotImplementedError("matmul (MXFP4 weight): microblock size 32 (e8m0 scales) only")
    if not isinstance(b, Tensor) and b.dtype != torch.uint8:
        raise NotImplementedError(f"matmul: b_mx_scale with a {b.dtype} weight (packed FP4 in uint8 is implemented)")
    w = b if isinstance(b, Tensor) else wrap_torch_tensor(b, dtype=FP4)
    ws = b_mx_scale if isinstance(b_mx_scale, Tensor) else wrap_torch_tensor(b_mx_scale)
    if not isinstance(w.layout, BlackwellMX4ValueLayout):
        w = convert_layout(w, make_default_matmul_mxfp4_w_layout(mx_axis=1))
    if not isinstance(ws.layout, BlackwellMXScaleLayout):
        ws = convert_layout(ws, make_default_matmul_mxfp4_w_scale_layout(mx_axis=1))
    E, K, N = w.shape
    assert ws.shape == (E, (K + 31) // 32, N), "scale shape does not match the weight"
    return w, ws


def upcast_mxfp4_weight(b, b_mx_scale, dtype, microblock=None):
    """An MXFP4 weight ([E, K/2, N] uint8 + [E, K/32, N] e8m0, or the converted Tensors) as a ``[E, K, N]``
    bf16 / fp16 view with K contiguous (``tb200_mxfp4_upcast``)."""
    w, ws = _mx4_kernel_layout(b, b_mx_scale, microblock)
    E, K, N = w.shape
    if K % 128 or N % 128:
        raise NotImplementedError("matmul (16-bit activations x MXFP4): K and N must be multiples of 128")
    dev = w.data.device
    if not w.data.is_cuda:
        raise RuntimeError("triton_b200 matmul needs CUDA tensors (there is no CPU path)")
    out = torch.empty((E, N, K), dtype=dtype, device=dev)
    if out.numel():
        args = _lib.Mxfp4UpcastArgs()
        args.w, args.w_scale, args.out = w.data.data_ptr(), ws.data.data_ptr(), out.data_ptr()
        args.n_experts, args.k, args.n = E, K, N
        args.out_dtype = _DT[dtype]
        with _lib.device_guard(dev):
            rc = _lib.lib().tb200_mxfp4_upcast(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
        _lib.check(rc, "tb200_mxfp4_upcast")
    return out.transpose(1, 2)


def _matmul_mx4(a, b, bias, a_ragged_metadata, scatter_indx, pc: PrecisionConfig, gammas, fused_activation, c=None):
    """FP8 activations x MXFP4 weights (the reference's Blackwell "fp8 x mx4" MoE configuration,
    bench/bench_mlp.py:253-279). ``b`` / ``pc.b_mx_scale`` are either what ``downcast_to_mxfp(w, torch.uint8,
    axis=1)`` returned ([E, K/2, N] and [E, K/32, N] uint8: re-laid here on every call) or the Tensors
    ``convert_layout`` produced from them (no per-call work)."""
    if not isinstance(a, torch.Tensor) or a.dtype not in _F8:
        raise NotImplementedError("matmul (MXFP4 weight): activations must be fp8 (e4m3fn / e5m2), bf16 or fp16")
    if not a.is_cuda:
        raise RuntimeError("triton_b200 matmul needs CUDA tensors (there is no CPU path)")
    if a.ndim != 2:
        raise NotImplementedError("matmul: batched input is not implemented")
    w_fp8 = isinstance(b, torch.Tensor) and b.dtype in _F8
    if w_fp8:
        w_bytes, ws_bytes, (E, K, N) = _fp8_weight_kernel_layout(b, pc.b_mx_scale, pc.b_microblock_size)
    else:
        w, ws = _mx4_kernel_layout(b, pc.b_mx_scale, pc.b_microblock_size)
        E, K, N = w.shape
        w_bytes, ws_bytes = w.data, ws.data
    assert a.shape[1] == K, "inner dimensions differ"
    dev = a.device
    if a.stride(1) != 1 or a.stride(0) % 16:
        a = a.contiguous()
    swiglu, alpha, limit = 0, 1.0, None
    if fused_activation is not None and fused_activation.specs.name != "dflt":
        if fused_activation.specs.name != "swiglu":
            raise NotImplementedError(f"matmul: fused activation {fused_activation.specs.name!r}")
        swiglu = 1
        alpha = float(fused_activation.fn_args[0])
        limit = fused_activation.fn_args[1] if len(fused_activation.fn_args) > 1 else None
    n_out = N // 2 if swiglu else N
    R = a.shape[0]
    if a_ragged_metadata is None:
        assert E == 1, "several weight matrices need a_ragged_metadata"
        a_ragged_metadata = make_ragged_tensor_metadata(torch.tensor([R], dtype=torch.int32, device=dev), R)
    md = a_ragged_metadata
    # few rows per expert (decode): the 32-row schedule and the kernel with swapped operand roles (which cannot
    # quantise a SwiGLU output: a block of 32 outputs would span two of its warps)
    block_rows = 32 if R <= 32 * E and not w_fp8 and not (swiglu and pc.c_mx_scale is not None) else 128
    sched = md.block_schedule(block_rows)
    rows_y = R if scatter_indx is None else scatter_indx.shape[0]
    out_dtype = pc.out_dtype or a.dtype  # as the reference: the activation dtype (fp8) unless asked otherwise
    out_codes = {**_DT, **_F8}
    if out_dtype not in out_codes:
        raise NotImplementedError("matmul (MXFP4 weight): bf16 / fp16 / fp8 output")
    if c is not None:  # the caller's output buffer (rows a scatter index does not name are zeroed, as in a fresh one)
        if pc.c_mx_scale is not None:
            raise NotImplementedError("matmul: MX-quantised output with c / c_acc_in is not implemented")
        assert c.shape == (rows_y, n_out) and c.dtype == out_dtype and c.device == dev and c.stride(1) == 1, \
            "c must be a [rows, n_out] tensor of the output dtype with unit column stride"
        if scatter_indx is not None:
            c.zero_()
    else:
        c = (torch.zeros if scatter_indx is not None else torch.empty)((rows_y, n_out), dtype=out_dtype, device=dev)
    a_sf = c_sf = None
    if pc.a_mx_scale is not None:
        a_sf = _plain_scale(pc.a_mx_scale)
        assert a_sf.shape == (R, (K + 31) // 32), "a_mx_scale: one e8m0 byte per 32 values of K, [rows, K/32]"
        k_steps4 = (K + 127) // 128 * 4
        if a_sf.shape[1] < k_steps4:  # the kernel reads four bytes per 128 values of K: pad the last step with 1.0
            a_sf = torch.nn.functional.pad(a_sf, (0, k_steps4 - a_sf.shape[1]), value=127)
        if a_sf.stride(1) != 1 or a_sf.stride(0) % 4 or a_sf.data_ptr() % 4:
            a_sf = a_sf.contiguous()
    if pc.c_mx_scale is not None:
        if out_dtype not in _F8:
            raise NotImplementedError("matmul: MX-quantised output is fp8 (e4m3fn / e5m2)")
        c_sf = _plain_scale(pc.c_mx_scale)
        assert c_sf.shape == (rows_y, (n_out + 31) // 32) and c_sf.stride(1) == 1, \
            "c_mx_scale: [rows, ceil(N_out / 32)] uint8, row-major"
    si = None if scatter_indx is None else scatter_indx.to(torch.int32).contiguous()
    gm = None if gammas is None else gammas.float().contiguous()
    bs = None if bias is None else bias.float().reshape(E, N).contiguous()
    fc = pc.flex_ctx if pc.flex_ctx is not None else FlexCtx()
    if fc.acc_data.scale is not None or fc.out_data.checksum_scale is not None:
        raise NotImplementedError("matmul: flexpoint acc_data / checksum_scale are not implemented")
    if pc.x_scale is not None and fc.lhs_data.scale is not None:
        raise ValueError("matmul: x_scale and flex_ctx.lhs_data.scale name the same factor")
    xs = _flex_scalar(pc.x_scale if pc.x_scale is not None else fc.lhs_data.scale, dev, "lhs scale")
    wfs = _flex_scalar(fc.rhs_data.scale, dev, "rhs scale")
    y_exp = _flex_scalar(fc.out_data.expected_scale, dev, "expected_scale")
    y_act = fc.out_data.actual_scale
    if y_act is not None:
        if not (isinstance(y_act, torch.Tensor) and y_act.is_cuda and y_act.dtype == torch.float32
                and y_act.numel() == 1):
            raise ValueError("matmul: flex_ctx.out_data.actual_scale is a one-element fp32 CUDA tensor the kernel updates")
        if out_dtype not in _F8 and out_dtype != torch.float16:
            raise NotImplementedError("matmul: actual_scale needs an fp8 or fp16 output")
    args = _lib.MoeGemmMx4Args()
    args.x, args.w, args.y = a.data_ptr(), w_bytes.data_ptr(), c.data_ptr()
    args.w_scale = ws_bytes.data_ptr() if ws_bytes is not None else None
    args.w_dtype = _F8[b.dtype] if w_fp8 else 0
    args.x_scale = xs.data_ptr() if xs is not None else None
    args.bias = bs.data_ptr() if bs is not None else None
    args.slice_offs, args.slice_sizes, args.block_schedule = (md.slice_offs.data_ptr(), md.slice_sizes.data_ptr(),
                                                             sched.data_ptr())
    args.scatter_indx = si.data_ptr() if si is not None else None
    args.gammas = gm.data_ptr() if gm is not None else None
    args.n_experts, args.k, args.n = E, K, N
    args.rows_x, args.rows_y = R, rows_y
    args.ldx, args.ldy = a.stride(0), c.stride(0)
    args.n_sched = sched.shape[0]
    args.x_dtype, args.out_dtype = _F8[a.dtype], out_codes[out_dtype]
    args.swiglu = swiglu
    args.swiglu_alpha = alpha
    args.swiglu_limit = float(limit) if limit is not None else 0.0
    args.swiglu_has_limit = 1 if limit is not None else 0
    args.block_rows = block_rows
    if wfs is not None:
        args.w_flex_scale = wfs.data_ptr()
    if y_exp is not None:
        args.y_expected_scale = y_exp.data_ptr()
        args.flexpoint_saturate_inf = 1 if pc.flexpoint_saturate_inf else 0
    if y_act is not None:
        args.y_actual_scale = y_act.data_ptr()
    if a_sf is not None:
        args.x_mx_scale, args.ld_x_mx_scale = a_sf.data_ptr(), a_sf.stride(0)
    if c_sf is not None:
        args.y_mx_scale, args.ld_y_mx_scale = c_sf.data_ptr(), c_sf.stride(0)
    with _lib.device_guard(dev):
        rc = _lib.lib().tb200_moe_gemm_mx4(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
    _lib.check(rc, "tb200_moe_gemm_mx4")
    return c
