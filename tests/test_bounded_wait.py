"""The bounded-wait path: a device-side wait that nothing completes must give up after its limit, record its
code in the status word, let the kernel return, and leave the context usable.

`tb200_selftest_wait` launches one block whose thread 0 waits (with the routine all kernels of the library use)
on an mbarrier nobody arrives on, with a 1 ms limit given at run time. Nothing faults, traps or hangs: the wait
returns false and the block exits."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

WAIT_SELFTEST = 9


def test_wait_runs_out_and_is_reported_once(cuda, lib):
    from oracle import gemm as o_gemm
    from triton_b200 import _lib
    from triton_b200.tutorials.blackwell_gemm_ws import matmul
    with torch.cuda.device(cuda):
        stream = ctypes.c_void_p(_lib.current_stream_ptr(cuda))
        assert lib.tb200_check(stream) == _lib.OK
        completed = torch.full((1, ), -1, dtype=torch.int32, device=cuda)
        rc = lib.tb200_selftest_wait(1_000_000, completed.data_ptr(), stream)   # 1 ms
        assert rc == _lib.OK, _lib.error_string(rc)
        torch.cuda.synchronize()
        assert int(completed.item()) == 0                      # the wait was abandoned, not completed
        word = lib.tb200_last_status_code()
        assert (word >> 16) == WAIT_SELFTEST and (word & 0xffff) == 0   # wait code, block 0
        assert lib.tb200_check(stream) == _lib.ERR_TIMEOUT    # reported ...
        assert lib.tb200_check(stream) == _lib.OK             # ... once, then cleared
        assert lib.tb200_last_status_code() == 0
        # the context is intact: a GEMM launched afterwards is correct
        g = torch.Generator().manual_seed(0)
        a = torch.randn(256, 256, generator=g).to(torch.bfloat16)
        b = torch.randn(256, 256, generator=g).to(torch.bfloat16)
        c = matmul(a.to(cuda), b.to(cuda))
        torch.testing.assert_close(c.cpu().float(), o_gemm.gemm_ref(a, b).float(), rtol=1e-2, atol=1e-2)
        _lib.sync_check(cuda)


def test_selftest_rejects_long_limits(lib):
    from triton_b200 import _lib
    assert lib.tb200_selftest_wait(0, None, None) == _lib.ERR_BAD_ARG
    assert lib.tb200_selftest_wait(2_000_000_000, None, None) == _lib.ERR_BAD_ARG
