"""Expert-parallel MoE layer on GPUs, both transports (peer stores through a SymmetricMemoryPool, NCCL
all-to-all through an EpGroup). World size 1 runs everywhere (the exchange degenerates to local row moves,
the fused combine to a one-entry peer table); the 2-rank cases run when the box has at least two GPUs, with
NVLS off and plain peer stores only."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe as o

pytestmark = pytest.mark.gpu


def _inputs(T, D, F, E, seed=4):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    w1 = (0.05 * torch.randn(E, D, 2 * F, generator=g)).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(E, F, D, generator=g)).to(torch.bfloat16)
    return x, logits, w1, w2


@pytest.mark.parametrize("shape", [(192, 16), (1536, 8)])  # 48 and 768 rows per expert: one CTA per block, CTA pairs
@pytest.mark.parametrize("transport", ["pool_fused", "pool", "nccl"])
def test_ep_layer_world_size_one_matches_oracle(cuda, transport, shape):
    from triton_b200 import _lib
    from triton_b200.triton_kernels.distributed import (EpGroup, Mesh, SymmetricMemoryPool, make_expt_assignment,
                                                        make_expt_dict_uniform, moe_layer_ep)
    (T, E), D, F, k = shape, 256, 128, 4
    x, logits, w1, w2 = _inputs(T, D, F, E)
    ea = make_expt_assignment(1, E, make_expt_dict_uniform(1, E), cuda)
    if transport == "nccl":
        ep = EpGroup()
    else:
        ep = SymmetricMemoryPool(Mesh())
        ep.initialize_matmul(T, D, D, k, E, torch.bfloat16, cuda)
    for _ in range(2):  # twice: the buffers are reused from call to call
        z = moe_layer_ep(x.to(cuda), logits.to(cuda), w1.to(cuda), w2.to(cuda), k, ea, ep,
                         fuse_combine=transport == "pool_fused")
    ref = o.moe_layer_ref(x, logits, w1, w2, k, 1.0, None)
    torch.testing.assert_close(z.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
    _lib.sync_check(cuda)
    if transport != "nccl":
        ep.close()


def test_dispatch_and_combine_are_inverse_permutations(cuda):
    """convert_dp_to_ep then convert_ep_to_dp through the pool (world size 1) returns every token row k times,
    bit for bit, and the dispatch buffer holds each token at its expert-sorted positions."""
    from triton_b200.triton_kernels.distributed import (Mesh, SymmetricMemoryPool, convert_dp_to_ep, convert_ep_to_dp,
                                                        make_expt_assignment, make_expt_dict_random)
    from triton_b200.triton_kernels.topk import topk
    T, D, E, k = 300, 128, 24, 3
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16).to(cuda)
    sm = topk(torch.randn(T, E, generator=g).to(cuda), k)
    mm = sm.mask_metadata
    ea = make_expt_assignment(1, E, make_expt_dict_random(1, E), cuda)
    pool = SymmetricMemoryPool(Mesh())
    pool.initialize_matmul(T, D, D, k, E, torch.bfloat16, cuda)
    y = convert_dp_to_ep(x, ea, sm.indx, mm.row_sorted_indx, pool)
    assert torch.equal(y, x[torch.div(mm.col_sorted_indx, k, rounding_mode="trunc").long()])
    back = convert_ep_to_dp(y, ea, sm.indx, mm.col_sorted_indx, pool)
    assert torch.equal(back.view(T, k, D), x[:, None, :].expand(T, k, D))
    pool.close()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from triton_b200 import _lib
        from triton_b200.triton_kernels.distributed import (EpGroup, Mesh, SymmetricMemoryPool, make_expt_assignment,
                                                            make_expt_dict_random, make_expt_dict_uniform,
                                                            moe_layer_ep)
        T, D, F, E, k = 256, 256, 128, 16, 4
        x, logits, w1, w2 = _inputs(T, D, F, E)
        tl = T // world
        ref = o.moe_layer_ref(x, logits, w1, w2, k, 1.0, None)[rank * tl:(rank + 1) * tl]
        pool = SymmetricMemoryPool(Mesh())
        pool.initialize_matmul(T, D, D, k, E, torch.bfloat16, dev)
        done = []
        for maker in (make_expt_dict_uniform, make_expt_dict_random):
            expt_dict = maker(world, E)
            ea = make_expt_assignment(world, E, expt_dict, dev)
            mine = sorted(expt_dict[rank])  # local expert i is the i-th smallest global id
            args = (x[rank * tl:(rank + 1) * tl].to(dev), logits[rank * tl:(rank + 1) * tl].to(dev),
                    w1[mine].to(dev), w2[mine].to(dev), k, ea)
            for name, ep, fuse in (("pool_fused", pool, True), ("pool", pool, False), ("nccl", EpGroup(), False)):
                for _ in range(2):
                    z = moe_layer_ep(*args, ep, fuse_combine=fuse)
                torch.testing.assert_close(z.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
                done.append(f"{maker.__name__}/{name}")
        _lib.sync_check(dev)
        pool.close()
        q.put((rank, "ok", done))
    except Exception as e:
        q.put((rank, f"error: {e!r}", []))
    finally:
        dist.destroy_process_group()


def test_ep_layer_two_ranks_all_transports(cuda):
    """Two ranks, uniform and random (interleaved) expert assignment, peer-store transport with and without
    the fused combine, and the NCCL all-to-all transport: every rank's slice equals the unsharded layer."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {r: (s, d) for r, s, d in (q.get(timeout=300) for _ in range(2))}
    for p in procs:
        p.join(timeout=60)
    assert results[0][0] == "ok" and results[1][0] == "ok", results
    assert len(results[0][1]) == 6


def _late_rank_worker(rank, world, port, q):
    """Rank 1 stays away from one barrier (it is alive and idle, its buffers stay mapped); rank 0's barrier kernel
    waits its 0.3 s, gives up and returns: the host reads the timeout, the context stays usable, and after rank 1
    makes up for the missed barrier both ranks meet again normally."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import ctypes
        from triton_b200 import _lib
        from triton_b200.triton_kernels.distributed import Mesh, SymmetricMemoryPool
        pool = SymmetricMemoryPool(Mesh())
        pool._reserve_region("signal", pool.SIGNAL_BYTES, 256, 0)
        pool._initialize(dev)
        stream = ctypes.c_void_p(_lib.current_stream_ptr(dev))
        l = _lib.lib()
        pool.hdl.barrier(channel=2)                      # both arrive: fine
        torch.cuda.synchronize()
        assert l.tb200_check(stream) == _lib.OK
        dist.barrier()
        if rank == 0:
            pool.hdl.barrier(channel=2, limit_ns=300_000_000)   # rank 1 never comes
            torch.cuda.synchronize()
            word = l.tb200_last_status_code()
            assert (word >> 16) == 10 and (word & 0xffff) == 1, hex(word)   # wait code "peer", the missing rank
            assert l.tb200_check(stream) == _lib.ERR_TIMEOUT
            assert l.tb200_check(stream) == _lib.OK
        dist.barrier()                                   # host-side: rank 0 has seen the timeout
        if rank == 1:
            pool.hdl.barrier(channel=2)                  # the missed one: rank 0's flag is there already
            torch.cuda.synchronize()
        dist.barrier()
        pool.hdl.barrier(channel=2)                      # and the ranks are in step again
        x = torch.full((4, ), float(rank + 1), device=dev)
        torch.cuda.synchronize()
        assert l.tb200_check(stream) == _lib.OK and float(x.sum()) == 4.0 * (rank + 1)
        pool.close()
        q.put((rank, "ok", []))
    except Exception as e:
        q.put((rank, f"error: {e!r}", []))
    finally:
        dist.destroy_process_group()


def test_barrier_wait_for_an_absent_rank_runs_out(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_late_rank_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = {r: s for r, s, _ in (q.get(timeout=300) for _ in range(2))}
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results
