"""ctypes binding of ``libtriton_b200.so`` (the C ABI declared in ``include/triton_b200.h``).

There is no CPU fallback: if the shared library is missing or a call fails, the wrappers
raise. ``lib()`` loads the library on first use.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libtriton_b200.so"

OK = 0
ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_TMAP, ERR_TOO_LARGE = -1, -2, -3, -4, -5, -6

BF16, F16, F32, E4M3, E5M2 = 0, 1, 2, 3, 4


class Tb200Error(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        super().__init__(f"{what}: {error_string(code)} (code {code})")


class GemmArgs(Structure):
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("c", c_void_p),
        ("m", c_int64), ("n", c_int64), ("k", c_int64),
        ("lda", c_int64), ("ldb", c_int64), ("ldc", c_int64),
        ("in_dtype", c_int32), ("out_dtype", c_int32),
        ("a_k_major", c_int32), ("b_k_major", c_int32),
        ("split_k", c_int32), ("block_n", c_int32),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("scale_a", c_void_p), ("scale_b", c_void_p),
        ("scale_mode", c_int32), ("reserved", c_int32),
    ]


class GemmMxfp8Args(Structure):
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("a_scale", c_void_p), ("b_scale", c_void_p), ("c", c_void_p),
        ("m", c_int64), ("n", c_int64), ("k", c_int64), ("ldc", c_int64),
        ("block_n", c_int32), ("reserved", c_int32),
    ]


class GemmFp8BlockwiseArgs(Structure):
    _fields_ = [
        ("a", c_void_p), ("b", c_void_p), ("c", c_void_p), ("scale_a", c_void_p), ("scale_b", c_void_p),
        ("m", c_int64), ("n", c_int64), ("k", c_int64), ("ldc", c_int64),
        ("in_dtype", c_int32), ("out_dtype", c_int32),
    ]


class AttentionArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("lse", c_void_p),
        ("batch", c_int64), ("heads", c_int64), ("seq_q", c_int64), ("seq_kv", c_int64),
        ("head_dim", c_int32), ("dtype", c_int32), ("causal", c_int32), ("sm_scale", c_float),
    ]


class AttentionMxfp8Args(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("q_scale", c_void_p), ("k_scale", c_void_p),
        ("v_scale", c_void_p), ("o", c_void_p), ("lse", c_void_p),
        ("batch", c_int64), ("heads", c_int64), ("seq_q", c_int64), ("seq_kv", c_int64),
        ("head_dim", c_int32), ("causal", c_int32), ("sm_scale", c_float), ("reserved0", c_int32),
    ]


class AttentionBwdArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("d_o", c_void_p), ("lse", c_void_p),
        ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("batch", c_int64), ("heads", c_int64), ("seq_q", c_int64), ("seq_kv", c_int64),
        ("head_dim", c_int32), ("dtype", c_int32), ("causal", c_int32), ("sm_scale", c_float),
    ]


class TopkArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("y_vals", c_void_p), ("y_indx", c_void_p), ("bitmatrix", c_void_p),
        ("rows_alloc", c_int64), ("n_rows", c_int64), ("n_cols", c_int64),
        ("stride_x", c_int64), ("stride_y", c_int64),
        ("bits_stride_row", c_int64), ("bits_stride_word", c_int64),
        ("k", c_int32), ("dtype", c_int32), ("apply_softmax", c_int32), ("use_provided_indx", c_int32),
    ]


class BitmatrixMetadataArgs(Structure):
    _fields_ = [
        ("indx", c_void_p), ("col_sum", c_void_p), ("col_sorted_indx", c_void_p), ("row_sorted_indx", c_void_p),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("n_entries", c_int64), ("n_cols", c_int32), ("indx_is_int16", c_int32),
    ]


class RaggedMetadataArgs(Structure):
    _fields_ = [
        ("slice_sizes", c_void_p), ("slice_offs", c_void_p), ("block_offs", c_void_p), ("block_schedule", c_void_p),
        ("n_slices", c_int32), ("max_n_blocks", c_int32),
    ]


class ReduceKArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("mask", c_void_p), ("scale", c_void_p), ("y", c_void_p),
        ("n_tokens", c_int64), ("d", c_int64), ("k", c_int32), ("dtype", c_int32), ("row_indx", c_void_p),
        ("x_rows", c_int64),
    ]


class SwigluArgs(Structure):
    _fields_ = [
        ("a", c_void_p), ("out", c_void_p), ("rows", c_int64), ("n_in", c_int64), ("lda", c_int64), ("ldo", c_int64),
        ("alpha", c_float), ("limit", c_float), ("has_limit", c_int32), ("dtype", c_int32),
    ]


class MoeGemmArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("y", c_void_p),
        ("slice_offs", c_void_p), ("block_schedule", c_void_p),
        ("gather_indx", c_void_p), ("scatter_indx", c_void_p), ("gammas", c_void_p),
        ("n_experts", c_int64), ("k", c_int64), ("n", c_int64),
        ("rows_x", c_int64), ("rows_y", c_int64), ("ldx", c_int64), ("ldy", c_int64),
        ("n_sched", c_int32), ("w_n_major", c_int32), ("dtype", c_int32), ("swiglu", c_int32),
        ("swiglu_alpha", c_float), ("swiglu_limit", c_float), ("swiglu_has_limit", c_int32), ("moe_tile_mode", c_int32),
        ("slice_sizes", c_void_p),
        ("y_peers", POINTER(c_void_p)), ("rows_per_peer", c_int64), ("y_world", c_int32), ("gammas_by_out_row", c_int32),
        ("betas", c_void_p), ("c_acc_in", c_void_p), ("ld_acc_in", c_int64), ("out_alpha", c_float), ("has_out_alpha", c_int32),
        ("y_mx_scale", c_void_p), ("ld_y_mx_scale", c_int64), ("y_mx_dtype", c_int32), ("reserved0", c_int32),
    ]


class RemapRaggedMetadataArgs(Structure):
    _fields_ = [
        ("slice_sizes", c_void_p), ("slice_offs", c_void_p), ("block_offs", c_void_p), ("block_schedule", c_void_p),
        ("slice_map", c_void_p),
        ("out_slice_sizes", c_void_p), ("out_slice_offs", c_void_p), ("out_block_offs", c_void_p),
        ("out_block_schedule", c_void_p),
        ("n_slices", c_int32), ("max_n_blocks", c_int32),
    ]


class EpDispatchArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("x_pitch_bytes", c_int64), ("expt_indx", c_void_p), ("dispatch_indx", c_void_p),
        ("expt_owner", c_void_p), ("dst_peers", POINTER(c_void_p)), ("dst_pitch_bytes", c_int64), ("dst_rows", c_int64),
        ("row_bytes", c_int64), ("n_tokens_local", c_int64), ("token_offset", c_int64),
        ("k", c_int32), ("n_experts", c_int32), ("world", c_int32), ("indx_is_int16", c_int32),
    ]


class EpCombineArgs(Structure):
    _fields_ = [
        ("src", c_void_p), ("src_pitch_bytes", c_int64), ("expt_indx", c_void_p), ("combine_indx", c_void_p),
        ("expt_owner", c_void_p), ("dst_peers", POINTER(c_void_p)), ("dst_pitch_bytes", c_int64), ("row_bytes", c_int64),
        ("n_rows", c_int64), ("rows_per_rank", c_int64),
        ("n_experts", c_int32), ("world", c_int32), ("rank", c_int32), ("indx_is_int16", c_int32),
    ]


class MoeGemmMx4Args(Structure):
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("w_scale", c_void_p), ("x_scale", c_void_p), ("bias", c_void_p), ("y", c_void_p),
        ("slice_offs", c_void_p), ("slice_sizes", c_void_p), ("block_schedule", c_void_p),
        ("scatter_indx", c_void_p), ("gammas", c_void_p),
        ("n_experts", c_int64), ("k", c_int64), ("n", c_int64), ("rows_x", c_int64), ("rows_y", c_int64),
        ("ldx", c_int64), ("ldy", c_int64),
        ("n_sched", c_int32), ("x_dtype", c_int32), ("out_dtype", c_int32), ("swiglu", c_int32),
        ("swiglu_alpha", c_float), ("swiglu_limit", c_float), ("swiglu_has_limit", c_int32), ("block_rows", c_int32),
        ("x_mx_scale", c_void_p), ("ld_x_mx_scale", c_int64), ("y_mx_scale", c_void_p), ("ld_y_mx_scale", c_int64),
        ("w_flex_scale", c_void_p), ("y_expected_scale", c_void_p), ("y_actual_scale", c_void_p),
        ("flexpoint_saturate_inf", c_int32), ("w_dtype", c_int32),
    ]


class Mxfp4UpcastArgs(Structure):
    _fields_ = [
        ("w", c_void_p), ("w_scale", c_void_p), ("out", c_void_p),
        ("n_experts", c_int64), ("k", c_int64), ("n", c_int64), ("out_dtype", c_int32),
    ]


_lib = None


def _declare(l: ctypes.CDLL) -> None:
    l.tb200_version.restype = c_int
    l.tb200_version.argtypes = []
    l.tb200_error_string.restype = c_char_p
    l.tb200_error_string.argtypes = [c_int]
    l.tb200_check.restype = c_int
    l.tb200_check.argtypes = [c_void_p]
    l.tb200_last_status_code.restype = c_int
    l.tb200_last_status_code.argtypes = []
    l.tb200_selftest_wait.restype = c_int
    l.tb200_selftest_wait.argtypes = [ctypes.c_uint64, c_void_p, c_void_p]
    l.tb200_gemm.restype = c_int
    l.tb200_gemm.argtypes = [POINTER(GemmArgs), c_void_p]
    l.tb200_gemm_plan.restype = c_int
    l.tb200_gemm_plan.argtypes = [POINTER(GemmArgs), POINTER(c_int32)]
    l.tb200_gemm_workspace_bytes.restype = c_size_t
    l.tb200_gemm_workspace_bytes.argtypes = [POINTER(GemmArgs)]
    l.tb200_attention_fwd.restype = c_int
    l.tb200_attention_fwd.argtypes = [POINTER(AttentionArgs), c_void_p]
    l.tb200_attention_mxfp8_fwd.restype = c_int
    l.tb200_attention_mxfp8_fwd.argtypes = [POINTER(AttentionMxfp8Args), c_void_p]
    l.tb200_attention_bwd.restype = c_int
    l.tb200_attention_bwd.argtypes = [POINTER(AttentionBwdArgs), c_void_p]
    l.tb200_attention_bwd_workspace_bytes.restype = c_size_t
    l.tb200_attention_bwd_workspace_bytes.argtypes = [POINTER(AttentionBwdArgs)]
    for name, typ in (("tb200_topk", TopkArgs), ("tb200_bitmatrix_metadata", BitmatrixMetadataArgs),
                      ("tb200_ragged_metadata", RaggedMetadataArgs), ("tb200_reduce_k", ReduceKArgs),
                      ("tb200_swiglu", SwigluArgs), ("tb200_moe_gemm", MoeGemmArgs),
                      ("tb200_remap_ragged_metadata", RemapRaggedMetadataArgs), ("tb200_ep_dispatch", EpDispatchArgs),
                      ("tb200_ep_combine", EpCombineArgs)):
        fn = getattr(l, name)
        fn.restype = c_int
        fn.argtypes = [POINTER(typ), c_void_p]
    l.tb200_symm_alloc.restype = c_int
    l.tb200_symm_alloc.argtypes = [c_size_t, POINTER(c_void_p)]
    l.tb200_symm_free.restype = c_int
    l.tb200_symm_free.argtypes = [c_void_p]
    l.tb200_symm_export.restype = c_int
    l.tb200_symm_export.argtypes = [c_void_p, c_void_p]
    l.tb200_symm_open.restype = c_int
    l.tb200_symm_open.argtypes = [c_void_p, POINTER(c_void_p)]
    l.tb200_symm_close.restype = c_int
    l.tb200_symm_close.argtypes = [c_void_p]
    l.tb200_symm_put.restype = c_int
    l.tb200_symm_put.argtypes = [c_void_p, c_size_t, POINTER(c_void_p), c_int32, c_void_p]
    l.tb200_symm_barrier.restype = c_int
    l.tb200_symm_barrier.argtypes = [POINTER(c_void_p), c_int32, c_int32, ctypes.c_uint64, c_void_p]
    l.tb200_bitmatrix_metadata_static.restype = c_int
    l.tb200_bitmatrix_metadata_static.argtypes = [c_void_p, c_int32, c_int64, c_int32, c_void_p, c_void_p, c_void_p, c_void_p]
    l.tb200_gather_rows.restype = c_int
    l.tb200_gather_rows.argtypes = [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p]
    l.tb200_move_rows.restype = c_int
    l.tb200_move_rows.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int32, c_int64,
                                  c_void_p]
    l.tb200_bitmatrix_metadata_workspace_bytes.restype = c_size_t
    l.tb200_bitmatrix_metadata_workspace_bytes.argtypes = [c_int64, c_int32]
    l.tb200_gemm_fp8_blockwise.restype = c_int
    l.tb200_gemm_fp8_blockwise.argtypes = [POINTER(GemmFp8BlockwiseArgs), c_void_p]
    l.tb200_moe_gemm_mx4.restype = c_int
    l.tb200_moe_gemm_mx4.argtypes = [POINTER(MoeGemmMx4Args), c_void_p]
    l.tb200_mxfp4_upcast.restype = c_int
    l.tb200_mxfp4_upcast.argtypes = [POINTER(Mxfp4UpcastArgs), c_void_p]
    l.tb200_gemm_mxfp8.restype = c_int
    l.tb200_gemm_mxfp8.argtypes = [POINTER(GemmMxfp8Args), c_void_p]


def lib() -> ctypes.CDLL:
    """Returns the loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m triton_b200.build` "
                "(triton_b200 has no CPU or PyTorch fallback)")
        l = ctypes.CDLL(str(LIB_PATH))
        _declare(l)
        _lib = l
    return _lib


def error_string(code: int) -> str:
    return lib().tb200_error_string(code).decode()


def check(rc: int, what: str) -> None:
    if rc != OK:
        raise Tb200Error(rc, what)


def pointer_array(ptrs):
    """A ctypes array of device pointers (the HOST arrays of peer pointers some entry points take)."""
    return (c_void_p * len(ptrs))(*[int(p) for p in ptrs])


def _device_index(device) -> int:
    import torch
    if device is None:
        return torch.cuda.current_device()
    if isinstance(device, int):
        return device
    idx = torch.device(device).index if not isinstance(device, torch.device) else device.index
    return torch.cuda.current_device() if idx is None else idx


def current_stream_ptr(device=None) -> int:
    """The raw cudaStream_t of torch's current stream on `device` (the stream every entry point is launched on)."""
    import torch
    return torch._C._cuda_getCurrentRawStream(_device_index(device))


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def device_guard(device):
    """``torch.cuda.device(device)`` when `device` is not the current one, else a context manager that does nothing
    (switching devices costs a few microseconds per call, which matters for launch-bound shapes)."""
    import torch
    idx = _device_index(device)
    if idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(idx)


def sync_check(device=None) -> None:
    """Synchronises the current stream and raises if a device-side wait timed out."""
    check(lib().tb200_check(c_void_p(current_stream_ptr(device))), "tb200_check")
