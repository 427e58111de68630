"""Expert-parallel (EP) token exchange — counterpart of ``triton_kernels/distributed.py`` in the
reference (``ExptAssignment``, ``make_expt_dict_uniform/random``, ``make_expt_assignment``
``:9-95``; ``convert_dp_to_ep`` ``:176-211``; ``convert_ep_to_dp`` ``:257-283``).

The reference moves token rows with peer stores through symmetric memory; here the rows cross
NVLink with one NCCL ``all_to_all_single`` per direction (what the headline configuration names),
and the indexed row placement on either side is a CUDA row-mover kernel. The result layouts are the
reference's: ``convert_dp_to_ep`` returns a ``[n_tokens_global * k, d]`` buffer whose rows at the
*global* expert-sorted positions of this rank's experts are filled (the other rows are
unspecified), so ``remap_ragged_tensor_metadata(global_metadata, expt_map[rank])`` and ``matmul``
work on it unchanged; ``convert_ep_to_dp`` returns ``[n_tokens_local * k, d]`` in (token, slot)
order, ready for ``reduce(y.view(-1, k, d), dim=1)``.

All index bookkeeping (`make_ep_plan`) is device-agnostic tensor arithmetic on the routing
metadata that every rank holds after the top-k all-gather; it contains no data movement and is
covered on CPU with ``gloo`` ranks. Requirement of the all-to-all formulation: each rank's experts
occupy one contiguous range of expert-sorted rows, which holds for ``make_expt_dict_uniform`` (and
any assignment of contiguous expert blocks in rank order); other assignments raise.
"""
from __future__ import annotations

import ctypes
import random
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _lib
from .tensor import Bitmatrix, SparseMatrix


@dataclass
class ExptAssignment:
    # [n_expt_shard, ceil(n_expt_tot / 32)] int32: bit j%32 of word j//32 set iff shard i owns expert j
    expt_bitmask: torch.Tensor
    # [n_expt_shard, n_expt_tot] bool
    expt_boolmask: torch.Tensor
    # [n_expt_shard, n_expt_tot] int32: local id of expert j in shard i, or -1
    expt_map: torch.Tensor
    n_expts_per_shard: list


def make_expt_dict_uniform(n_expt_shard, n_expt_tot):
    """Shard i owns experts [i * (n_expt_tot // n_expt_shard), (i + 1) * (n_expt_tot // n_expt_shard))."""
    per = n_expt_tot // n_expt_shard
    return {i: list(range(per * i, per * (i + 1))) for i in range(n_expt_shard)}


def make_expt_dict_random(n_expt_shard, n_expt_tot):
    """Each shard owns a disjoint random, non-empty subset of the experts (seeded)."""
    rng = random.Random(0)
    perm = list(range(n_expt_tot))
    rng.shuffle(perm)
    cuts = [0] + sorted(rng.sample(range(1, n_expt_tot), n_expt_shard - 1)) + [n_expt_tot]
    return {i: perm[cuts[i]:cuts[i + 1]] for i in range(n_expt_shard)}


def make_expt_assignment(n_expt_shard, n_expt_tot, expt_dict, device) -> ExptAssignment:
    import numpy as np
    words = (n_expt_tot + 31) // 32
    bm = np.zeros((n_expt_shard, words), dtype=np.uint32)
    boolmask = torch.zeros((n_expt_shard, n_expt_tot), dtype=torch.bool)
    counts = [0] * n_expt_tot
    for shard, experts in expt_dict.items():
        if len(experts) == 0:
            raise ValueError(f"shard {shard} has no experts")
        if shard < 0 or shard >= n_expt_shard:
            raise ValueError(f"shard {shard} out of range [0, {n_expt_shard})")
        if not isinstance(experts, (list, tuple)):
            raise TypeError(f"expt_dict[{shard}] must be a list/tuple of ints")
        for e in experts:
            if not (0 <= e < n_expt_tot):
                raise ValueError(f"expert id {e} out of range [0, {n_expt_tot})")
            counts[e] += 1
            bm[shard, e >> 5] |= np.uint32(1) << np.uint32(e & 31)
            boolmask[shard, e] = True
    bitmask = torch.from_numpy(bm.view(np.int32).copy())
    if not all(c == 1 for c in counts):
        raise ValueError("each expert must be owned by exactly one shard")
    expt_map = torch.full((n_expt_shard, n_expt_tot), -1, dtype=torch.int32)
    for shard, experts in expt_dict.items():
        for local_id, global_id in enumerate(sorted(experts)):
            expt_map[shard, global_id] = local_id
    return ExptAssignment(bitmask.to(device), boolmask.to(device), expt_map.to(device),
                          [len(e) for e in expt_dict.values()])


# --------------------------------------------------------------------------- exchange plan


@dataclass
class EpPlan:
    """Everything a rank needs for the two all-to-alls, derived from global routing metadata."""
    send_entries: torch.Tensor    # int32 [n_send]: this rank's (token, slot) entry ids (local numbering), ordered by
                                  # global expert-sorted position == grouped by destination rank
    send_counts: list             # rows sent to each rank (dispatch) == rows received from it (combine)
    recv_positions: torch.Tensor  # int32 [n_recv]: global sorted position of every received row, in arrival order
    recv_counts: list             # rows received from each rank (dispatch) == rows sent to it (combine)


def make_ep_plan(expt_indx: torch.Tensor, dispatch_indx: torch.Tensor, slice_offs: torch.Tensor,
                 expt_boolmask: torch.Tensor, rank: int, world_size: int, n_tokens_local: int) -> EpPlan:
    """expt_indx: [n_tokens_global, k] expert of every (token, slot) (-1 = padded row);
    dispatch_indx: [n_tokens_global * k] global expert-sorted position of every entry (-1 = none);
    slice_offs: [E + 1] start of every expert in sorted order; expt_boolmask: [world, E]."""
    n_tok_global, k = expt_indx.shape
    dev = expt_indx.device
    owner_of_expert = torch.argmax(expt_boolmask.to(torch.int32), dim=0)  # [E]
    sizes = (slice_offs[1:] - slice_offs[:-1]).to(torch.int64)
    # contiguity check: experts listed in sorted order must have non-decreasing owners (ignoring empty ones)
    own_nz = owner_of_expert[sizes > 0]
    if own_nz.numel() > 1 and bool((own_nz[1:] < own_nz[:-1]).any()):
        raise NotImplementedError("EP all-to-all needs each rank's experts to be contiguous in expert order "
                                  "(make_expt_dict_uniform); got an interleaved assignment")
    flat_e = expt_indx.reshape(-1).to(torch.int64)
    valid = flat_e >= 0
    entry_owner = torch.where(valid, owner_of_expert[flat_e.clamp(min=0)], torch.full_like(flat_e, -1))
    pos = dispatch_indx.to(torch.int64)
    entry_src = torch.arange(n_tok_global * k, device=dev) // (n_tokens_local * k)  # DP rank holding the token
    # ---- what this rank sends: its own valid entries, ordered by sorted position
    lo, hi = rank * n_tokens_local * k, (rank + 1) * n_tokens_local * k
    mine = torch.arange(lo, hi, device=dev)
    mine = mine[valid[lo:hi] & (pos[lo:hi] >= 0)]
    order = torch.argsort(pos[mine], stable=True)
    send_global = mine[order]
    send_counts = torch.bincount(entry_owner[send_global], minlength=world_size)[:world_size]
    # ---- what this rank receives: all entries whose expert it owns, by source rank then sorted position
    theirs = torch.nonzero((entry_owner == rank) & (pos >= 0)).flatten()
    key = entry_src[theirs] * (n_tok_global * k + 1) + pos[theirs]
    theirs = theirs[torch.argsort(key, stable=True)]
    recv_counts = torch.bincount(entry_src[theirs], minlength=world_size)[:world_size]
    return EpPlan((send_global - lo).to(torch.int32), [int(c) for c in send_counts.tolist()],
                  pos[theirs].to(torch.int32), [int(c) for c in recv_counts.tolist()])


# --------------------------------------------------------------------------- row movement (CUDA)


def _move_rows(src: torch.Tensor, dst: torch.Tensor, indx: torch.Tensor, scatter: bool) -> None:
    if not src.is_cuda:
        raise RuntimeError("EP row movement needs CUDA tensors (there is no CPU path)")
    assert src.stride(1) == 1 and dst.stride(1) == 1 and src.shape[1] == dst.shape[1] and src.dtype == dst.dtype
    indx = indx.to(torch.int32).contiguous()
    esz = src.element_size()
    with torch.cuda.device(src.device):
        rc = _lib.lib().tb200_move_rows(src.data_ptr(), src.stride(0) * esz, dst.data_ptr(), dst.stride(0) * esz,
                                        indx.data_ptr(), indx.numel(), src.shape[1] * esz, 1 if scatter else 0,
                                        ctypes.c_void_p(_lib.current_stream_ptr(src.device)))
    _lib.check(rc, "tb200_move_rows")


@dataclass
class EpGroup:
    """Stands where the reference passes a ``SymmetricMemoryPool``: the process group plus the plan
    cache shared by the two conversions of one layer call."""
    group: object = None
    plan: EpPlan | None = None
    n_tokens_local: int = 0

    @property
    def rank(self):
        return dist.get_rank(self.group) if dist.is_initialized() else 0

    @property
    def world_size(self):
        return dist.get_world_size(self.group) if dist.is_initialized() else 1


def all_gather_topk(x_local: torch.Tensor, k: int, ep: EpGroup, apply_softmax: bool = True) -> SparseMatrix:
    """``topk(..., all_gather=True)`` of the reference (``topk.py:41-69``): local top-k, then every
    rank gets the values / indices of all ranks' tokens (rank-major), and the global routing
    metadata is built from them."""
    from .topk import topk_forward
    vals, indx, _ = topk_forward(x_local, k, apply_softmax)
    world = ep.world_size
    if world > 1:
        g_vals = torch.empty((world * vals.shape[0], k), dtype=vals.dtype, device=vals.device)
        g_indx = torch.empty((world * indx.shape[0], k), dtype=indx.dtype, device=indx.device)
        # gathered as raw bytes: NCCL has no int16
        dist.all_gather_into_tensor(g_vals.view(torch.uint8), vals.contiguous().view(torch.uint8), group=ep.group)
        dist.all_gather_into_tensor(g_indx.view(torch.uint8), indx.contiguous().view(torch.uint8), group=ep.group)
    else:
        g_vals, g_indx = vals, indx
    return SparseMatrix(vals=g_vals, indx=g_indx, mask=Bitmatrix(None, shape=[g_indx.shape[0], x_local.shape[1]]))


def convert_dp_to_ep(src, expt_assignment: ExptAssignment, expt_indx, gate_indx, symm_mem_pool: EpGroup,
                     slice_offs=None):
    """DP-local token rows -> expert-sorted rows on the ranks that own the experts.
    src: [n_tokens_local, d]; expt_indx: [n_tokens_global, k]; gate_indx: dispatch indices
    (``row_sorted_indx``) [n_tokens_global * k]. ``slice_offs`` (global ragged ``slice_offs``) is
    needed to check the contiguity requirement; it is recomputed from ``expt_indx`` when omitted."""
    ep = symm_mem_pool
    n_local, d = src.shape
    n_global, k = expt_indx.shape
    dev = src.device
    if slice_offs is None:
        e_tot = expt_assignment.expt_boolmask.shape[1]
        flat = expt_indx.reshape(-1).to(torch.int64)
        sizes = torch.bincount(flat[flat >= 0], minlength=e_tot)
        slice_offs = torch.cat([torch.zeros(1, dtype=torch.int64, device=dev), torch.cumsum(sizes, 0)])
    plan = make_ep_plan(expt_indx, gate_indx, slice_offs, expt_assignment.expt_boolmask, ep.rank, ep.world_size, n_local)
    ep.plan, ep.n_tokens_local = plan, n_local
    send = torch.empty((sum(plan.send_counts), d), dtype=src.dtype, device=dev)
    _move_rows(src, send, torch.div(plan.send_entries, k, rounding_mode="trunc"), scatter=False)
    recv = torch.empty((sum(plan.recv_counts), d), dtype=src.dtype, device=dev)
    if ep.world_size > 1:
        dist.all_to_all_single(recv, send, plan.recv_counts, plan.send_counts, group=ep.group)
    else:
        recv = send
    dst = torch.empty((n_global * k, d), dtype=src.dtype, device=dev)
    _move_rows(recv, dst, plan.recv_positions, scatter=True)
    return dst


def convert_ep_to_dp(src, expt_assignment: ExptAssignment, expt_indx, topk_indx, symm_mem_pool: EpGroup):
    """Expert-sorted output rows (global positions, valid where this rank owns the expert) -> rows in
    (token, slot) order on the DP rank that holds each token. Must follow ``convert_dp_to_ep`` on the
    same ``EpGroup`` (it reuses that exchange plan, reversed)."""
    ep = symm_mem_pool
    plan = ep.plan
    assert plan is not None, "convert_ep_to_dp needs the plan of the preceding convert_dp_to_ep"
    d = src.shape[1]
    dev = src.device
    k = expt_indx.shape[1]
    send = torch.empty((sum(plan.recv_counts), d), dtype=src.dtype, device=dev)
    _move_rows(src, send, plan.recv_positions, scatter=False)
    back = torch.empty((sum(plan.send_counts), d), dtype=src.dtype, device=dev)
    if ep.world_size > 1:
        dist.all_to_all_single(back, send, plan.send_counts, plan.recv_counts, group=ep.group)
    else:
        back = send
    out = torch.zeros((ep.n_tokens_local * k, d), dtype=src.dtype, device=dev)
    _move_rows(back, out, plan.send_entries, scatter=True)
    return out


def moe_layer_ep(x_local, logits_local, w1_local, w2_local, k, expt_assignment: ExptAssignment, ep: EpGroup,
                 alpha: float = 1.0, limit=None, gate_weighted: bool = True):
    """One expert-parallel MoE layer, wired as the reference's ``run_mlp``
    (``python/triton_kernels/bench/bench_mlp.py:60-96``): all-gathered top-k -> global routing
    metadata -> DP->EP exchange -> GEMM-1 (+SwiGLU) -> GEMM-2 (x gate weight) on the local experts
    -> EP->DP exchange -> sum over the k slots. Returns ``[n_tokens_local, d_model]``."""
    from .matmul import matmul, swiglu_activation
    from .reduce import reduce
    from .tensor import make_ragged_tensor_metadata, remap_ragged_tensor_metadata
    sm = all_gather_topk(logits_local, k, ep)
    mm = sm.mask_metadata
    n_entries = sm.indx.numel()
    rg = make_ragged_tensor_metadata(mm.col_sum, n_entries)
    y = convert_dp_to_ep(x_local, expt_assignment, sm.indx, mm.row_sorted_indx, ep, slice_offs=rg.slice_offs)
    rg_local = remap_ragged_tensor_metadata(rg, expt_assignment.expt_map[ep.rank])
    h = matmul(y, w1_local, None, rg_local, fused_activation=swiglu_activation(alpha, limit))
    gam = None
    if gate_weighted:
        gam = sm.vals.float().reshape(-1)[mm.col_sorted_indx.long().clamp(min=0)]
    o = matmul(h, w2_local, None, rg_local, gammas=gam)
    y_dp = convert_ep_to_dp(o, expt_assignment, sm.indx, mm.col_sorted_indx, ep)
    z, _ = reduce(y_dp.view(x_local.shape[0], k, -1), dim=1)
    return z
