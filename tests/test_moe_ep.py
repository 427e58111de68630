"""Expert-parallel MoE layer on GPUs. World size 1 runs everywhere (the exchange degenerates to the
local row moves); the 2-rank NCCL case runs when the box has at least two GPUs."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe as o

pytestmark = pytest.mark.gpu


def test_ep_layer_world_size_one_matches_oracle(cuda):
    from triton_b200.triton_kernels.distributed import (EpGroup, make_expt_assignment, make_expt_dict_uniform,
                                                        moe_layer_ep)
    T, D, F, E, k = 192, 256, 128, 16, 4
    g = torch.Generator().manual_seed(4)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    w1 = (0.05 * torch.randn(E, D, 2 * F, generator=g)).to(torch.bfloat16)
    w2 = (0.05 * torch.randn(E, F, D, generator=g)).to(torch.bfloat16)
    ea = make_expt_assignment(1, E, make_expt_dict_uniform(1, E), cuda)
    z = moe_layer_ep(x.to(cuda), logits.to(cuda), w1.to(cuda), w2.to(cuda), k, ea, EpGroup())
    ref = o.moe_layer_ref(x, logits, w1, w2, k, 1.0, None)
    torch.testing.assert_close(z.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)


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
        from triton_b200.triton_kernels.distributed import (EpGroup, make_expt_assignment, make_expt_dict_uniform,
                                                            moe_layer_ep)
        T, D, F, E, k = 256, 256, 128, 16, 4
        g = torch.Generator().manual_seed(4)
        x = torch.randn(T, D, generator=g).to(torch.bfloat16)
        logits = torch.randn(T, E, generator=g)
        w1 = (0.05 * torch.randn(E, D, 2 * F, generator=g)).to(torch.bfloat16)
        w2 = (0.05 * torch.randn(E, F, D, generator=g)).to(torch.bfloat16)
        ea = make_expt_assignment(world, E, make_expt_dict_uniform(world, E), dev)
        per, tl = E // world, T // world
        z = moe_layer_ep(x[rank * tl:(rank + 1) * tl].to(dev), logits[rank * tl:(rank + 1) * tl].to(dev),
                         w1[rank * per:(rank + 1) * per].to(dev), w2[rank * per:(rank + 1) * per].to(dev), k, ea,
                         EpGroup())
        ref = o.moe_layer_ref(x, logits, w1, w2, k, 1.0, None)[rank * tl:(rank + 1) * tl]
        torch.testing.assert_close(z.cpu().float(), ref.float(), rtol=2e-2, atol=2e-2)
        q.put((rank, "ok"))
    except Exception as e:
        q.put((rank, f"error: {e}"))
    finally:
        dist.destroy_process_group()


def test_ep_layer_two_ranks_nccl(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results
