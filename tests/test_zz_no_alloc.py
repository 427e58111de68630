"""The fixed-scratch routing-metadata entry point, `tb200_bitmatrix_metadata_static`.

Some users of this library cannot hand it a workspace: their process decides how every byte of
GPU memory is used when it starts and refuses (or is forbidden) to allocate afterwards. For them
the library carries its own small scratch array. This test calls that entry point straight
through the C ABI, twice in a row on different inputs, and requires the three outputs to be
identical (they are integers) to those of the regular entry point that takes a caller workspace.
Two consecutive calls matter because both reuse the same scratch: the second must not be affected
by what the first left behind. The file name sorts last so that a `-x` run has already executed
every other test when it gets here; it also passes when run on its own in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(l, _lib, indx, n_cols, dev):
    n = indx.numel()
    col_sum = torch.empty(n_cols, dtype=torch.int32, device=dev)
    col_sorted = torch.empty(n, dtype=torch.int32, device=dev)
    row_sorted = torch.empty(n, dtype=torch.int32, device=dev)
    need = l.tb200_bitmatrix_metadata_workspace_bytes(n, n_cols)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    args = _lib.BitmatrixMetadataArgs()
    args.indx = indx.data_ptr()
    args.col_sum, args.col_sorted_indx, args.row_sorted_indx = col_sum.data_ptr(), col_sorted.data_ptr(), row_sorted.data_ptr()
    args.workspace, args.workspace_bytes = ws.data_ptr(), need
    args.n_entries, args.n_cols = n, n_cols
    args.indx_is_int16 = 1 if indx.dtype == torch.int16 else 0
    rc = l.tb200_bitmatrix_metadata(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
    assert rc == 0, _lib.error_string(rc)
    return col_sum, col_sorted, row_sorted


def _static(l, _lib, indx, n_cols, dev):
    n = indx.numel()
    # outputs come from the caller, as for every entry point; the call itself allocates nothing
    col_sum = torch.empty(n_cols, dtype=torch.int32, device=dev)
    col_sorted = torch.empty(n, dtype=torch.int32, device=dev)
    row_sorted = torch.empty(n, dtype=torch.int32, device=dev)
    rc = l.tb200_bitmatrix_metadata_static(indx.data_ptr(), 1 if indx.dtype == torch.int16 else 0, n, n_cols,
                                           col_sum.data_ptr(), col_sorted.data_ptr(), row_sorted.data_ptr(),
                                           ctypes.c_void_p(_lib.current_stream_ptr(dev)))
    assert rc == 0, _lib.error_string(rc)
    return col_sum, col_sorted, row_sorted


def test_static_scratch_matches_workspace_version_twice(cuda, lib):
    from triton_b200 import _lib
    g = torch.Generator().manual_seed(11)
    cases = [
        (torch.randint(0, 128, (16384, 4), generator=g).to(torch.int16), 128),   # config-5 sized routing table
        (torch.randint(-1, 40, (3001, 2), generator=g).to(torch.int32), 40),     # ragged size, some -1 entries
    ]
    with torch.cuda.device(cuda):
        for indx_cpu, n_cols in cases:            # two calls in a row share the library's scratch
            indx = indx_cpu.to(cuda)
            got = _static(lib, _lib, indx, n_cols, cuda)
            want = _regular(lib, _lib, indx, n_cols, cuda)
            torch.cuda.synchronize()
            for a, b in zip(got, want):
                assert torch.equal(a, b)
        # and once more on the first input: nothing stale from the second call leaks in
        indx = cases[0][0].to(cuda)
        got = _static(lib, _lib, indx, cases[0][1], cuda)
        want = _regular(lib, _lib, indx, cases[0][1], cuda)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
    _lib.sync_check(cuda)


def test_static_scratch_rejects_oversized_problems(cuda, lib):
    from triton_b200 import _lib
    with torch.cuda.device(cuda):
        dummy = torch.zeros(8, dtype=torch.int32, device=cuda)
        # 1,000,000 entries x 1024 columns needs 977 * 1024 + 1024 words: far over the fixed capacity
        rc = lib.tb200_bitmatrix_metadata_static(dummy.data_ptr(), 0, 1_000_000, 1024, dummy.data_ptr(), dummy.data_ptr(),
                                                 dummy.data_ptr(), None)
        assert rc == _lib.ERR_TOO_LARGE
        assert "capacity" in _lib.error_string(rc)


def test_static_scratch_capacity_boundary_and_empty_input(cuda, lib):
    """262144 entries x 1024 columns needs 256 * 1024 + 1024 = 263168 words, exactly the capacity: accepted and
    equal to the workspace version. One entry more starts a 257th block of histograms: refused. An empty
    routing table is accepted and yields an all-zero histogram."""
    from triton_b200 import _lib
    g = torch.Generator().manual_seed(12)
    with torch.cuda.device(cuda):
        indx = torch.randint(0, 1024, (262144, ), generator=g).to(torch.int32).to(cuda)
        got = _static(lib, _lib, indx, 1024, cuda)
        want = _regular(lib, _lib, indx, 1024, cuda)
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        one_more = torch.zeros(262145, dtype=torch.int32, device=cuda)
        out = torch.empty(262145, dtype=torch.int32, device=cuda)
        rc = lib.tb200_bitmatrix_metadata_static(one_more.data_ptr(), 0, 262145, 1024, out.data_ptr(), out.data_ptr(),
                                                 out.data_ptr(), None)
        assert rc == _lib.ERR_TOO_LARGE
        col_sum = torch.full((128, ), 7, dtype=torch.int32, device=cuda)
        rc = lib.tb200_bitmatrix_metadata_static(None, 0, 0, 128, col_sum.data_ptr(), None, None,
                                                 ctypes.c_void_p(_lib.current_stream_ptr(cuda)))
        assert rc == 0, _lib.error_string(rc)
        assert int(col_sum.abs().sum()) == 0
    _lib.sync_check(cuda)
