"""Host-side logic of the expert-parallel path on CPU: expert assignment tables and the
all-to-all exchange plan, exercised by two `gloo` ranks (no GPU). The plan is pure index
arithmetic; the row movement that the product does with a CUDA kernel is done here with tensor
indexing inside the test, so what is checked is that the plan routes every row to the right rank
and position."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moe as o


def test_make_expt_assignment_tables():
    from triton_b200.triton_kernels.distributed import (make_expt_assignment, make_expt_dict_random,
                                                        make_expt_dict_uniform)
    for n_shard, n_tot, maker in [(8, 512, make_expt_dict_uniform), (16, 64, make_expt_dict_random),
                                  (4, 40, make_expt_dict_random)]:
        d = maker(n_shard, n_tot)
        ea = make_expt_assignment(n_shard, n_tot, d, "cpu")
        for shard in range(n_shard):
            words = ea.expt_bitmask[shard].numpy().view(np.uint32)
            experts = [j for j in range(n_tot) if (int(words[j >> 5]) >> (j & 31)) & 1]
            assert experts == sorted(d[shard])
            assert ea.expt_boolmask[shard].nonzero().flatten().tolist() == sorted(d[shard])
            emap = torch.full((n_tot, ), -1, dtype=torch.int32)
            emap[sorted(d[shard])] = torch.arange(len(d[shard]), dtype=torch.int32)
            assert torch.equal(emap, ea.expt_map[shard])
    with pytest.raises(ValueError):
        make_expt_assignment(2, 4, {0: [0, 1], 1: [1, 2, 3]}, "cpu")  # expert 1 owned twice
    with pytest.raises(ValueError):
        make_expt_assignment(2, 4, {0: [0, 1, 2, 3], 1: []}, "cpu")
    with pytest.raises(ValueError):
        make_expt_assignment(2, 4, {0: [0, 1], 1: [2]}, "cpu")         # expert 3 owned by nobody
    with pytest.raises(ValueError):
        make_expt_assignment(2, 4, {0: [0, 1], 2: [2, 3]}, "cpu")      # shard id out of range
    with pytest.raises(ValueError):
        make_expt_assignment(2, 4, {0: [0, 1], 1: [2, 4]}, "cpu")      # expert id out of range
    with pytest.raises(TypeError):
        make_expt_assignment(2, 4, {0: {0, 1}, 1: [2, 3]}, "cpu")


def test_make_expt_dict_random_is_the_reference_draw():
    """The seeded draw must give the reference's assignment (``make_expt_dict_random``,
    python/triton_kernels/triton_kernels/distributed.py:38-53); these three dicts are its outputs."""
    from triton_b200.triton_kernels.distributed import make_expt_dict_random
    assert make_expt_dict_random(2, 8) == {0: [4, 1, 5, 2], 1: [0, 3, 7, 6]}
    assert make_expt_dict_random(4, 16) == {0: [10, 14, 5], 1: [1, 9], 2: [2, 3, 11, 13, 7, 8, 4, 0], 3: [6, 15, 12]}
    assert make_expt_dict_random(3, 10) == {0: [7, 8, 1, 5], 1: [3, 4], 2: [2, 0, 9, 6]}


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_worker(rank, world, port, n_local, E, k, d, fail_rank, q, random_assignment=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from triton_b200.triton_kernels.distributed import (_expt_owner, make_ep_plan, make_expt_assignment,
                                                            make_expt_dict_random, make_expt_dict_uniform)
        g = torch.Generator().manual_seed(4)
        T = n_local * world
        x_global = torch.randn(T, d, generator=g)
        logits = torch.randn(T, E, generator=g)
        _, indx, _ = o.topk_ref(logits, k)
        md = o.bitmatrix_metadata_ref(indx.numpy(), E)
        rg = o.ragged_metadata_ref(md.col_sum, T * k)
        maker = make_expt_dict_random if random_assignment else make_expt_dict_uniform
        ea = make_expt_assignment(world, E, maker(world, E), "cpu")
        plan = make_ep_plan(indx, torch.from_numpy(md.row_sorted_indx), _expt_owner(ea), rank, world, n_local)
        # ---- dispatch
        x_local = x_global[rank * n_local:(rank + 1) * n_local]
        send = x_local[(plan.send_entries // k).long()]
        recv = torch.empty(sum(plan.recv_counts), d)
        dist.all_to_all_single(recv, send, plan.recv_counts, plan.send_counts)
        buf = torch.full((T * k, d), float("nan"))
        buf[plan.recv_positions.long()] = recv
        # every sorted position that belongs to one of my experts holds the row of its token
        combine = torch.from_numpy(md.col_sorted_indx).long()
        my_experts = ea.expt_boolmask[rank].nonzero().flatten().tolist()
        n_checked = 0
        for e in my_experts:
            lo, hi = int(rg.slice_offs[e]), int(rg.slice_offs[e + 1])
            assert torch.equal(buf[lo:hi], x_global[combine[lo:hi] // k])
            n_checked += hi - lo
        assert n_checked == sum(plan.recv_counts)
        # ---- "expert computation": scale every row by (expert id + 1), then combine
        y = buf.clone()
        for e in my_experts:
            lo, hi = int(rg.slice_offs[e]), int(rg.slice_offs[e + 1])
            y[lo:hi] *= (e + 1)
        back_send = y[plan.recv_positions.long()]
        back = torch.empty(sum(plan.send_counts), d)
        dist.all_to_all_single(back, back_send, plan.send_counts, plan.recv_counts)
        out = torch.zeros(n_local * k, d)
        out[plan.send_entries.long()] = back
        want = x_local.repeat_interleave(k, 0) * (indx[rank * n_local:(rank + 1) * n_local].reshape(-1, 1) + 1)
        assert torch.allclose(out, want)
        if rank == fail_rank:
            raise RuntimeError("injected host-side failure")
        q.put((rank, "ok"))
    except Exception as e:  # report instead of hanging the peer
        q.put((rank, f"error: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_local,E,k,random_assignment", [(48, 16, 4, False), (5, 8, 2, False), (40, 16, 4, True)])
def test_ep_plan_two_gloo_ranks(n_local, E, k, random_assignment):
    """Uniform blocks of experts per rank, and the reference's random assignment (a rank's experts interleave
    with the other rank's in expert order)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, n_local, E, k, 8, -1, q, random_assignment))
             for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert results == {0: "ok", 1: "ok"}, results


def test_ep_rank_failure_is_reported_on_the_host():
    """Failure detection without touching a GPU: one rank raises after the exchange; the test
    driver sees the error from that rank and a clean result from the other (no hang)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ep_worker, args=(r, 2, port, 8, 8, 2, 8, 1, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert results[0] == "ok" and results[1].startswith("error: injected")


def test_plan_of_an_interleaved_assignment():
    """Ranks owning alternating experts: rows are grouped by destination rank, by sorted position inside."""
    from triton_b200.triton_kernels.distributed import _expt_owner, make_ep_plan, make_expt_assignment
    E, k, T = 4, 1, 8
    indx = torch.arange(T).remainder(E).view(T, 1).to(torch.int32)
    md = o.bitmatrix_metadata_ref(indx.numpy(), E)
    ea = make_expt_assignment(2, E, {0: [0, 2], 1: [1, 3]}, "cpu")
    plan = make_ep_plan(indx, torch.from_numpy(md.row_sorted_indx), _expt_owner(ea), 0, 2, 4)
    # rank 0 holds tokens 0..3 (experts 0, 1, 2, 3): experts 0 and 2 stay, 1 and 3 go to rank 1
    assert plan.send_entries.tolist() == [0, 2, 1, 3] and plan.send_counts == [2, 2]
    # it receives the rows of experts 0 and 2 from both ranks; sorted positions: expert 0 -> 0, 1; expert 2 -> 4, 5
    assert plan.recv_positions.tolist() == [0, 4, 1, 5] and plan.recv_counts == [2, 2]
