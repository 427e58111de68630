"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/triton_b200.h declares (no compute calls here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    src = open(os.path.join(ROOT, "include", "triton_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", src)))


def test_header_declares_entry_points():
    names = declared_functions()
    assert "tb200_gemm" in names and "tb200_check" in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"libtriton_b200.so does not export {name}"
        assert isinstance(getattr(lib, name), ctypes._CFuncPtr)


def test_version_and_error_strings(lib):
    assert lib.tb200_version() >= 1
    from triton_b200 import _lib
    for code in (0, -1, -2, -3, -4, -5, -6):
        assert _lib.error_string(code) != "unknown error"


def test_gemm_rejects_bad_arguments_without_gpu(lib):
    from triton_b200 import _lib
    args = _lib.GemmArgs()
    assert lib.tb200_gemm(ctypes.byref(args), None) == _lib.ERR_BAD_ARG  # null pointers
    args.a = args.b = args.c = 4096
    args.m = args.n = 128
    args.k = 60  # row pitch 120 bytes: not a multiple of 16
    args.lda = args.ldb = 60
    args.ldc = 128
    args.a_k_major = args.b_k_major = 1
    assert lib.tb200_gemm(ctypes.byref(args), None) == _lib.ERR_BAD_ARG
    args.k = args.lda = args.ldb = 64
    args.in_dtype = 2  # fp32 inputs are not supported
    assert lib.tb200_gemm(ctypes.byref(args), None) == _lib.ERR_UNSUPPORTED


def test_product_does_not_import_oracle():
    """Nothing under triton_b200/ may reference the CPU oracle."""
    pkg = os.path.join(ROOT, "triton_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), f


def test_heuristic_config_reports_the_plan_the_library_takes(lib):
    """get_heuristic_config reads the tiling from the C side (no GPU needed): the headline shape takes the
    256 x 512 CTA-pair tile, the skinny shape 128-wide tiles with K split, a tiny shape one CTA per tile."""
    from triton_b200.tutorials.blackwell_gemm_ws import get_heuristic_config
    big = get_heuristic_config(8192, 8192, 8192)
    assert (big["BLOCK_SIZE_M"], big["BLOCK_SIZE_N"], big["NUM_CTAS"], big["SPLIT_K"]) == (256, 512, 2, 1)
    skinny = get_heuristic_config(128, 8192, 8192)
    assert skinny["BLOCK_SIZE_M"] == 128 and skinny["NUM_CTAS"] == 1 and skinny["SPLIT_K"] >= 2
    small = get_heuristic_config(128, 128, 128)
    assert small["NUM_CTAS"] == 1 and small["SPLIT_K"] == 1
