"""Expert-parallel (EP) token exchange — counterpart of ``triton_kernels/distributed.py`` and
``distributed_details/mesh.py`` in the reference (``ExptAssignment``, ``make_expt_dict_uniform/random``,
``make_expt_assignment`` ``distributed.py:9-95``; ``convert_dp_to_ep`` ``:176-211``; ``convert_ep_to_dp``
``:257-283``; ``Mesh``, ``SymmetricMemoryPool`` ``mesh.py:13-166``).

Two transports, chosen by what is passed where the reference passes its ``symm_mem_pool``:

* ``SymmetricMemoryPool`` (the reference's scheme, the default of ``moe_layer_ep``): every rank maps every
  rank's buffer (CUDA IPC), token rows are stored straight into the owner rank's buffer by a CUDA kernel
  (plain 16-byte peer stores over NVLink), a small barrier kernel orders the steps, and the combine can be
  fused into GEMM-2's epilogue (``matmul(..., fused_comm=...)``). No host synchronisation anywhere in a
  layer call; any expert-to-rank assignment works.
* ``EpGroup``: the rows cross NVLink with one NCCL ``all_to_all_single`` per direction, with CUDA row-mover
  kernels on either side. The exchange plan needs the per-pair row counts on the host (one read-back per
  layer call). Kept as the baseline the fused path is measured against.

Result layouts are the reference's: ``convert_dp_to_ep`` returns a ``[n_tokens_global * k, d]`` buffer whose
rows at the *global* expert-sorted positions of this rank's experts are filled (the other rows are
unspecified), so ``remap_ragged_tensor_metadata(global_metadata, expt_map[rank])`` and ``matmul`` work on it
unchanged; ``convert_ep_to_dp`` returns ``[n_tokens_local * k, d]`` in (token, slot) order, ready for
``reduce(y.view(-1, k, d), dim=1)``.
"""
from __future__ import annotations

import ctypes
import random
from dataclasses import dataclass
from math import prod

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
    """Each shard owns a disjoint, non-empty random subset of the experts. The draw sequence (one shuffle of
    the expert list, then one sample of the cut points, both from ``random.Random(0)``) is the reference's
    (``distributed.py:38-53``), so the same arguments give the same assignment."""
    rng = random.Random(0)
    order = list(range(n_expt_tot))
    rng.shuffle(order)
    inner = sorted(rng.sample(range(1, n_expt_tot), n_expt_shard - 1))
    bounds = [0, *inner, n_expt_tot]
    return {shard: order[lo:hi] for shard, (lo, hi) in enumerate(zip(bounds[:-1], bounds[1:]))}


def make_expt_assignment(n_expt_shard, n_expt_tot, expt_dict, device) -> ExptAssignment:
    """Tables of an expert -> shard assignment given as ``{shard: [expert ids]}``. Every expert must be named
    exactly once and every listed shard must own at least one expert."""
    owner = torch.full((n_expt_tot, ), -1, dtype=torch.int64)
    for shard, experts in expt_dict.items():
        if not isinstance(experts, (list, tuple)):
            raise TypeError(f"experts of shard {shard}: expected a list or tuple, got {type(experts).__name__}")
        if not 0 <= shard < n_expt_shard:
            raise ValueError(f"shard id {shard} is outside 0..{n_expt_shard - 1}")
        if not experts:
            raise ValueError(f"shard {shard} owns no expert")
        ids = torch.as_tensor(list(experts), dtype=torch.int64)
        if int(ids.min()) < 0 or int(ids.max()) >= n_expt_tot:
            raise ValueError(f"shard {shard} names an expert outside 0..{n_expt_tot - 1}")
        if ids.unique().numel() != ids.numel() or bool((owner[ids] != -1).any()):
            raise ValueError("an expert is assigned more than once")
        owner[ids] = shard
    if bool((owner == -1).any()):
        raise ValueError(f"experts {(owner == -1).nonzero().flatten().tolist()} are assigned to no shard")
    shards = torch.arange(n_expt_shard)[:, None]
    boolmask = owner[None, :] == shards                                        # [shard, expert]
    # local id = rank of the expert among its shard's experts in increasing expert order
    local = torch.cumsum(boolmask.to(torch.int32), dim=1, dtype=torch.int32) - 1
    expt_map = torch.where(boolmask, local, torch.full_like(local, -1))
    words = (n_expt_tot + 31) // 32
    padded = torch.zeros((n_expt_shard, words * 32), dtype=torch.int64)
    padded[:, :n_expt_tot] = boolmask
    weights = torch.ones(32, dtype=torch.int64) << torch.arange(32)
    packed = (padded.view(n_expt_shard, words, 32) * weights).sum(-1)          # 0 .. 2^32 - 1
    bitmask = torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)
    return ExptAssignment(bitmask.to(device), boolmask.to(device), expt_map.to(device),
                          [len(e) for e in expt_dict.values()])


def _expt_owner(ea: ExptAssignment) -> torch.Tensor:
    """int32 [n_expt_tot]: the shard that owns each expert (derived once from ``expt_boolmask``)."""
    own = ea.__dict__.get("_owner")
    if own is None:
        own = torch.argmax(ea.expt_boolmask.to(torch.int32), dim=0).to(torch.int32).contiguous()
        ea.__dict__["_owner"] = own
    return own


# --------------------------------------------------------------------------- symmetric memory


class Mesh:
    """The ranks that exchange tokens (``mesh.py:13-18``)."""

    def __init__(self, process_group=None):
        self.process_group = process_group
        init = dist.is_initialized()
        self.world_size = dist.get_world_size(process_group) if init else 1
        self.local_rank = dist.get_rank(process_group) if init else 0


@dataclass
class _Region:
    base: int
    size: int


class PeerBuffer:
    """A view of another rank's symmetric buffer: address, shape and dtype, nothing else. Kernels of this
    library store to it; torch never touches it."""

    def __init__(self, ptr: int, shape, dtype):
        self._ptr, self.shape, self.dtype = int(ptr), tuple(shape), dtype

    def data_ptr(self) -> int:
        return self._ptr


class _DeviceArray:
    """CUDA-array-interface holder that lets torch view memory this library allocated."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes, ), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


class _Handle:
    """What the reference's ``symm_mem.rendezvous`` handle is used for: ``barrier(channel)``."""

    N_CHANNELS = 8
    CHANNEL_BYTES = 512
    LIMIT_NS = 20_000_000_000  # ranks may reach a barrier seconds apart (first launches, host work between steps)

    def __init__(self, pool):
        self._pool = pool
        self._arrays = {}

    def barrier(self, channel: int = 0, limit_ns: int | None = None):
        """All ranks of the mesh meet on the current stream. ``limit_ns`` bounds the device-side wait (default
        20 s): when a rank does not arrive the kernel gives up, and the next ``tb200_check`` / ``sync_check`` on
        this device reports ``TB200_ERR_TIMEOUT``. The limit covers the time between the first and the last
        rank's launch, host-side delays included."""
        pool = self._pool
        if pool.mesh.world_size == 1:
            return
        assert 0 <= channel < self.N_CHANNELS
        arr = self._arrays.get(channel)
        if arr is None:
            arr = _lib.pointer_array([b + channel * self.CHANNEL_BYTES for b in pool.base_ptrs])
            self._arrays[channel] = arr
        with _lib.device_guard(pool.device):
            rc = _lib.lib().tb200_symm_barrier(arr, pool.mesh.local_rank, pool.mesh.world_size, limit_ns or self.LIMIT_NS,
                                               ctypes.c_void_p(_lib.current_stream_ptr(pool.device)))
        _lib.check(rc, "tb200_symm_barrier")


class SymmetricMemoryPool:
    """One buffer per rank, mapped into every rank (``mesh.py:34-166``): regions are reserved by name, then
    ``make_empty`` hands out one view per rank of the same region. The reference builds it on
    ``torch.distributed._symmetric_memory``; here each rank allocates with ``tb200_symm_alloc``, the 64-byte
    CUDA IPC handles travel through ``torch.distributed.all_gather`` and ``tb200_symm_open`` maps the peers.
    The first 4 KB hold the barrier's signal blocks."""

    SIGNAL_BYTES = _Handle.N_CHANNELS * _Handle.CHANNEL_BYTES

    def __init__(self, mesh: Mesh):
        self._is_initialized = False
        self.mesh = mesh
        self.regions = {}
        self.size = 0
        self.buf = None
        self.base_ptrs = None
        self.device = None
        self.hdl = _Handle(self)
        self._own_ptr = None
        self._side = None

    @staticmethod
    def align_up(value: int, alignment: int) -> int:
        return value if alignment <= 1 else (value + alignment - 1) // alignment * alignment

    def _reserve_region(self, name: str, size: int, alignment: int, offset: int) -> int:
        if self._is_initialized:
            raise RuntimeError("regions are reserved before the pool is initialised")
        if name in self.regions:
            raise ValueError(f"region {name!r} is reserved already")
        base = self.align_up(offset, max(alignment, 1))
        size = self.align_up(size, max(alignment, 1))
        self.regions[name] = _Region(base, size)
        return base + size

    def _initialize(self, device) -> None:
        if self._is_initialized:
            return
        device = torch.device(device)
        self.device = device
        self.size = max(self.SIGNAL_BYTES, max((r.base + r.size for r in self.regions.values()), default=0))
        l = _lib.lib()
        world, rank = self.mesh.world_size, self.mesh.local_rank
        with _lib.device_guard(device):
            own = ctypes.c_void_p()
            _lib.check(l.tb200_symm_alloc(self.size, ctypes.byref(own)), "tb200_symm_alloc")
            self._own_ptr = own.value
            ptrs = [None] * world
            ptrs[rank] = own.value
            if world > 1:
                handle = (ctypes.c_uint8 * 64)()
                _lib.check(l.tb200_symm_export(own, handle), "tb200_symm_export")
                mine = torch.tensor(list(handle), dtype=torch.uint8, device=device)
                everyone = [torch.empty_like(mine) for _ in range(world)]
                dist.all_gather(everyone, mine, group=self.mesh.process_group)
                for r in range(world):
                    if r == rank:
                        continue
                    raw = (ctypes.c_uint8 * 64)(*everyone[r].cpu().tolist())
                    peer = ctypes.c_void_p()
                    _lib.check(l.tb200_symm_open(raw, ctypes.byref(peer)), "tb200_symm_open")
                    ptrs[r] = peer.value
                dist.barrier(group=self.mesh.process_group)  # every rank's buffer is zeroed and mapped
            self.base_ptrs = ptrs
            self.buf = torch.as_tensor(_DeviceArray(own.value, self.size), device=device)
        self._is_initialized = True

    def initialize_matmul(self, n_tokens_global: int, d_input: int, d_model: int, n_expts_act: int, n_expts_tot: int,
                          dtype: torch.dtype, device) -> None:
        """Reserves the regions one MoE layer needs (``mesh.py:138-166``): the dispatch buffer
        ``[n_tokens_global * k, d_input]``, the combine buffer ``[n_tokens_local * k, d_model]`` and the gathered
        top-k values and indices."""
        if self._is_initialized:
            return
        esz = torch.empty((), dtype=dtype).element_size()
        n_local = n_tokens_global // self.mesh.world_size
        off = self._reserve_region("signal", self.SIGNAL_BYTES, 256, 0)
        # gathered top-k: values (4 bytes at most) then int16 indices, [n_tokens_global, k] each
        off = self._reserve_region("topk", n_tokens_global * n_expts_act * 6, 256, off)
        off = self._reserve_region("ep_to_dp", n_local * n_expts_act * d_model * esz, 256, off)
        off = self._reserve_region("dp_to_ep", n_tokens_global * n_expts_act * d_input * esz, 256, off)
        self._initialize(device)

    def side_stream(self):
        """A second stream on the pool's device for work that may overlap the token exchange (created once)."""
        if self._side is None:
            self._side = torch.cuda.Stream(self.device)
        return self._side

    def make_empty(self, shape, dtype, region: str, region_offset: int = 0, clear: bool = False):
        """One view per rank of ``region`` (this rank's as a torch tensor, the others as ``PeerBuffer``)."""
        if not self._is_initialized:
            raise RuntimeError("SymmetricMemoryPool is not initialised")
        info = self.regions.get(region)
        if info is None:
            raise ValueError(f"unknown region {region!r}")
        esz = torch.empty((), dtype=dtype).element_size()
        nbytes = prod(shape) * esz
        start = info.base + region_offset
        if region_offset % esz or start + nbytes > info.base + info.size:
            raise ValueError(f"[{start}, {start + nbytes}) does not fit region {region!r}")
        mine = self.buf[start:start + nbytes].view(dtype).view(*shape)
        if clear:
            mine.zero_()
        rank = self.mesh.local_rank
        return tuple(mine if r == rank else PeerBuffer(self.base_ptrs[r] + start, shape, dtype)
                     for r in range(self.mesh.world_size))

    def close(self) -> None:
        """Unmaps the peers and frees this rank's buffer (collective: every rank calls it)."""
        if not self._is_initialized:
            return
        l = _lib.lib()
        with _lib.device_guard(self.device):
            torch.cuda.synchronize()
            if self.mesh.world_size > 1:
                dist.barrier(group=self.mesh.process_group)
            for r, p in enumerate(self.base_ptrs):
                if r != self.mesh.local_rank:
                    l.tb200_symm_close(ctypes.c_void_p(p))
            self.buf = None
            l.tb200_symm_free(ctypes.c_void_p(self._own_ptr))
        self._is_initialized = False


# --------------------------------------------------------------------------- NCCL exchange plan


@dataclass
class EpPlan:
    """Everything a rank needs for the two all-to-alls, derived from global routing metadata."""
    send_entries: torch.Tensor    # int32 [n_send]: this rank's (token, slot) entry ids (local numbering), grouped by
                                  # destination rank, by expert-sorted position within a destination
    send_counts: list             # rows sent to each rank (dispatch) == rows received from it (combine)
    recv_positions: torch.Tensor  # int32 [n_recv]: global sorted position of every received row, in arrival order
    recv_counts: list             # rows received from each rank (dispatch) == rows sent to it (combine)


def make_ep_plan(expt_indx: torch.Tensor, dispatch_indx: torch.Tensor, expt_owner: torch.Tensor, rank: int,
                 world_size: int, n_tokens_local: int) -> EpPlan:
    """expt_indx: [n_tokens_global, k] expert of every (token, slot) (-1 = padded row);
    dispatch_indx: [n_tokens_global * k] global expert-sorted position of every entry (-1 = none);
    expt_owner: [E] rank owning each expert (any assignment). Device-agnostic tensor arithmetic; the
    counts are read back to the host in one transfer."""
    n_tok_global, k = expt_indx.shape
    assert n_tok_global == world_size * n_tokens_local, "every rank must hold n_tokens_local tokens"
    dev = expt_indx.device
    n = n_tok_global * k
    flat_e = expt_indx.reshape(-1).to(torch.int64)
    pos = dispatch_indx.to(torch.int64)
    valid = (flat_e >= 0) & (pos >= 0)
    owner = torch.where(valid, expt_owner.to(torch.int64)[flat_e.clamp(min=0)], torch.full_like(flat_e, -1))
    src = torch.arange(n, device=dev) // (n_tokens_local * k)          # DP rank holding the entry's token
    # what this rank sends: its own valid entries by (destination, sorted position)
    lo = rank * n_tokens_local * k
    mine = torch.arange(lo, lo + n_tokens_local * k, device=dev)
    mine = mine[valid[mine]]
    mine = mine[torch.argsort(owner[mine] * (n + 1) + pos[mine], stable=True)]
    # what it receives: every entry whose expert it owns, by (source, sorted position) = the senders' orders
    theirs = torch.nonzero(owner == rank).flatten()
    theirs = theirs[torch.argsort(src[theirs] * (n + 1) + pos[theirs], stable=True)]
    counts = torch.stack([torch.bincount(owner[mine], minlength=world_size)[:world_size],
                          torch.bincount(src[theirs], minlength=world_size)[:world_size]]).tolist()
    return EpPlan((mine - lo).to(torch.int32), [int(c) for c in counts[0]], pos[theirs].to(torch.int32),
                  [int(c) for c in counts[1]])


def _move_rows(src: torch.Tensor, dst: torch.Tensor, indx: torch.Tensor, scatter: bool) -> None:
    if not src.is_cuda:
        raise RuntimeError("EP row movement needs CUDA tensors (there is no CPU path)")
    assert src.stride(1) == 1 and dst.stride(1) == 1 and src.shape[1] == dst.shape[1] and src.dtype == dst.dtype
    indx = indx.to(torch.int32).contiguous()
    esz = src.element_size()
    with _lib.device_guard(src.device):
        rc = _lib.lib().tb200_move_rows(src.data_ptr(), src.stride(0) * esz, dst.data_ptr(), dst.stride(0) * esz,
                                        indx.data_ptr(), indx.numel(), src.shape[1] * esz, 1 if scatter else 0,
                                        dst.shape[0] if scatter else src.shape[0],
                                        ctypes.c_void_p(_lib.current_stream_ptr(src.device)))
    _lib.check(rc, "tb200_move_rows")


@dataclass
class EpGroup:
    """NCCL transport: the process group plus the plan shared by the two conversions of one layer call."""
    group: object = None
    plan: EpPlan | None = None
    n_tokens_local: int = 0

    @property
    def rank(self):
        return dist.get_rank(self.group) if dist.is_initialized() else 0

    @property
    def world_size(self):
        return dist.get_world_size(self.group) if dist.is_initialized() else 1


def _transport(pool):
    """(rank, world_size, process group) of either transport."""
    if isinstance(pool, SymmetricMemoryPool):
        return pool.mesh.local_rank, pool.mesh.world_size, pool.mesh.process_group
    return pool.rank, pool.world_size, pool.group


def all_gather_topk(x_local: torch.Tensor, k: int, ep, apply_softmax: bool = True) -> SparseMatrix:
    """``topk(..., all_gather=True)`` of the reference (``topk.py:41-69``): local top-k, then every rank gets
    the values / indices of all ranks' tokens (rank-major), and the global routing metadata is built from them.
    With a ``SymmetricMemoryPool`` each rank stores its block into every rank's ``topk`` region (peer stores,
    then a barrier), as the reference does; with an ``EpGroup`` it is one NCCL all-gather of the packed bytes."""
    from .topk import topk_forward
    vals, indx, _ = topk_forward(x_local, k, apply_softmax)
    rank, world, group = _transport(ep)
    n, vb = vals.shape[0], vals.element_size()
    if world == 1:
        g_vals, g_indx = vals, indx
    elif isinstance(ep, SymmetricMemoryPool) and "topk" in ep.regions and (n * k * 2) % 16 == 0:
        dev = vals.device
        all_vals = ep.make_empty((world * n, k), vals.dtype, region="topk")
        all_indx = ep.make_empty((world * n, k), torch.int16, region="topk", region_offset=world * n * k * 4)
        l = _lib.lib()
        with _lib.device_guard(dev):
            stream = ctypes.c_void_p(_lib.current_stream_ptr(dev))
            for src, bufs, esz in ((vals, all_vals, vb), (indx, all_indx, 2)):
                slots = _lib.pointer_array([b.data_ptr() + rank * n * k * esz for b in bufs])
                _lib.check(l.tb200_symm_put(src.data_ptr(), n * k * esz, slots, world, stream), "tb200_symm_put")
        ep.hdl.barrier(channel=1)
        g_vals, g_indx = all_vals[rank], all_indx[rank]
    else:
        packed = torch.empty((n, k * (vb + 2)), dtype=torch.uint8, device=vals.device)
        packed[:, :k * vb] = vals.contiguous().view(torch.uint8).view(n, k * vb)
        packed[:, k * vb:] = indx.contiguous().view(torch.uint8).view(n, k * 2)
        gathered = torch.empty((world * n, k * (vb + 2)), dtype=torch.uint8, device=vals.device)
        dist.all_gather_into_tensor(gathered, packed, group=group)
        g_vals = gathered[:, :k * vb].contiguous().view(vals.dtype).view(world * n, k)
        g_indx = gathered[:, k * vb:].contiguous().view(torch.int16).view(world * n, k)
    return SparseMatrix(vals=g_vals, indx=g_indx, mask=Bitmatrix(None, shape=[g_indx.shape[0], x_local.shape[1]]))


def _indx_arg(expt_indx):
    assert expt_indx.dtype in (torch.int16, torch.int32) and expt_indx.is_contiguous()
    return expt_indx.data_ptr(), 1 if expt_indx.dtype == torch.int16 else 0


def convert_dp_to_ep(src, expt_assignment: ExptAssignment, expt_indx, gate_indx, symm_mem_pool):
    """DP-local token rows -> expert-sorted rows on the ranks that own the experts.
    src: [n_tokens_local, d]; expt_indx: [n_tokens_global, k]; gate_indx: dispatch indices
    (``row_sorted_indx``) [n_tokens_global * k]."""
    n_local, d = src.shape
    n_global, k = expt_indx.shape
    dev = src.device
    rank, world, group = _transport(symm_mem_pool)
    owner = _expt_owner(expt_assignment)
    if isinstance(symm_mem_pool, SymmetricMemoryPool):
        pool = symm_mem_pool
        assert n_local * world <= n_global
        peer_bufs = pool.make_empty((n_global * k, d), src.dtype, region="dp_to_ep")
        dst_local = peer_bufs[rank]
        if src.stride(1) != 1:
            src = src.contiguous()
        esz = src.element_size()
        args = _lib.EpDispatchArgs()
        args.x, args.x_pitch_bytes = src.data_ptr(), src.stride(0) * esz
        args.expt_indx, args.indx_is_int16 = _indx_arg(expt_indx)
        args.dispatch_indx, args.expt_owner = gate_indx.data_ptr(), owner.data_ptr()
        args.dst_peers = _lib.pointer_array([b.data_ptr() for b in peer_bufs])
        args.dst_pitch_bytes, args.dst_rows, args.row_bytes = d * esz, n_global * k, d * esz
        args.n_tokens_local, args.token_offset = n_local, rank * n_local
        args.k, args.n_experts, args.world = k, owner.shape[0], world
        with _lib.device_guard(dev):
            rc = _lib.lib().tb200_ep_dispatch(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
        _lib.check(rc, "tb200_ep_dispatch")
        pool.hdl.barrier(channel=0)
        return dst_local
    ep = symm_mem_pool
    plan = make_ep_plan(expt_indx, gate_indx, owner, rank, world, n_local)
    ep.plan, ep.n_tokens_local = plan, n_local
    send = torch.empty((sum(plan.send_counts), d), dtype=src.dtype, device=dev)
    _move_rows(src, send, torch.div(plan.send_entries, k, rounding_mode="trunc"), scatter=False)
    recv = torch.empty((sum(plan.recv_counts), d), dtype=src.dtype, device=dev)
    if world > 1:
        dist.all_to_all_single(recv, send, plan.recv_counts, plan.send_counts, group=group)
    else:
        recv = send
    dst = torch.empty((n_global * k, d), dtype=src.dtype, device=dev)
    _move_rows(recv, dst, plan.recv_positions, scatter=True)
    return dst


def convert_ep_to_dp(src, expt_assignment: ExptAssignment, expt_indx, topk_indx, symm_mem_pool):
    """Expert-sorted output rows (global positions, valid where this rank owns the expert) -> rows in
    (token, slot) order on the DP rank that holds each token. src: [n_tokens_global * k, d]; topk_indx:
    combine indices (``col_sorted_indx``). With an ``EpGroup`` it must follow ``convert_dp_to_ep`` on the same
    group (it reuses that exchange plan, reversed)."""
    d = src.shape[1]
    dev = src.device
    k = expt_indx.shape[1]
    rank, world, group = _transport(symm_mem_pool)
    if isinstance(symm_mem_pool, SymmetricMemoryPool):
        pool = symm_mem_pool
        rows_per_rank = src.shape[0] // world
        peer_bufs = pool.make_empty((rows_per_rank, d), src.dtype, region="ep_to_dp")
        owner = _expt_owner(expt_assignment)
        esz = src.element_size()
        args = _lib.EpCombineArgs()
        args.src, args.src_pitch_bytes = src.data_ptr(), src.stride(0) * esz
        args.expt_indx, args.indx_is_int16 = _indx_arg(expt_indx)
        args.combine_indx, args.expt_owner = topk_indx.data_ptr(), owner.data_ptr()
        args.dst_peers = _lib.pointer_array([b.data_ptr() for b in peer_bufs])
        args.dst_pitch_bytes, args.row_bytes = d * esz, d * esz
        args.n_rows, args.rows_per_rank = src.shape[0], rows_per_rank
        args.n_experts, args.world, args.rank = owner.shape[0], world, rank
        with _lib.device_guard(dev):
            rc = _lib.lib().tb200_ep_combine(ctypes.byref(args), ctypes.c_void_p(_lib.current_stream_ptr(dev)))
        _lib.check(rc, "tb200_ep_combine")
        pool.hdl.barrier(channel=0)
        return peer_bufs[rank]
    ep = symm_mem_pool
    plan = ep.plan
    assert plan is not None, "convert_ep_to_dp needs the plan of the preceding convert_dp_to_ep"
    send = torch.empty((sum(plan.recv_counts), d), dtype=src.dtype, device=dev)
    _move_rows(src, send, plan.recv_positions, scatter=False)
    back = torch.empty((sum(plan.send_counts), d), dtype=src.dtype, device=dev)
    if world > 1:
        dist.all_to_all_single(back, send, plan.send_counts, plan.recv_counts, group=group)
    else:
        back = send
    out = torch.zeros((ep.n_tokens_local * k, d), dtype=src.dtype, device=dev)
    _move_rows(back, out, plan.send_entries, scatter=True)
    return out


def moe_layer_ep(x_local, logits_local, w1_local, w2_local, k, expt_assignment: ExptAssignment, ep,
                 alpha: float = 1.0, limit=None, gate_weighted: bool = True, fuse_combine: bool = True):
    """One expert-parallel MoE layer, wired as the reference's ``run_mlp``
    (``python/triton_kernels/bench/bench_mlp.py:60-96``): all-gathered top-k -> global routing metadata ->
    DP->EP exchange -> GEMM-1 (+SwiGLU) -> GEMM-2 (x gate weight) on the local experts -> EP->DP exchange ->
    sum over the k slots. ``ep`` is a ``SymmetricMemoryPool`` (peer stores; with ``fuse_combine`` GEMM-2's
    epilogue writes each row straight into the buffer of the rank that holds the token) or an ``EpGroup``
    (NCCL all-to-all). Returns ``[n_tokens_local, d_model]``."""
    from .matmul import FusedComm, matmul, swiglu_activation
    from .reduce import reduce
    from .tensor import make_ragged_tensor_metadata, remap_ragged_tensor_metadata
    rank, world, _ = _transport(ep)
    sm = all_gather_topk(logits_local, k, ep)
    mm = sm.mask_metadata
    n_entries = sm.indx.numel()
    if isinstance(ep, SymmetricMemoryPool) and world > 1:
        # the ragged metadata is needed by the GEMMs only: derive it on a second stream while the token rows cross
        # NVLink (under graph capture the two become parallel branches)
        cur = torch.cuda.current_stream(x_local.device)
        side = ep.side_stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            rg = make_ragged_tensor_metadata(mm.col_sum, n_entries)
            rg_local = remap_ragged_tensor_metadata(rg, expt_assignment.expt_map[rank])
        y = convert_dp_to_ep(x_local, expt_assignment, sm.indx, mm.row_sorted_indx, ep)
        cur.wait_stream(side)
    else:
        rg = make_ragged_tensor_metadata(mm.col_sum, n_entries)
        rg_local = remap_ragged_tensor_metadata(rg, expt_assignment.expt_map[rank])
        y = convert_dp_to_ep(x_local, expt_assignment, sm.indx, mm.row_sorted_indx, ep)
    # The GEMMs see buffers sized for the worst case, so the tiling is chosen here from what balanced routing gives
    # a rank: CTA pairs when the experts average 256 rows or more (the rule the library applies to the row count
    # it is given), else the library's own choice.
    n_expts_tot = expt_assignment.expt_map.shape[-1]
    tile_mode = 2 if n_entries >= 256 * n_expts_tot else 0
    h = matmul(y, w1_local, None, rg_local, fused_activation=swiglu_activation(alpha, limit), _tile_mode=tile_mode)
    n_local = x_local.shape[0]
    if isinstance(ep, SymmetricMemoryPool) and fuse_combine:
        d_out = w2_local.shape[-1]
        peer_bufs = ep.make_empty((n_local * k, d_out), h.dtype, region="ep_to_dp")
        # the gate weight of an output row is the top-k value of its (token, slot): looked up by the epilogue
        matmul(h, w2_local, None, rg_local, gammas=sm.vals if gate_weighted else None, scatter_indx=mm.col_sorted_indx, _tile_mode=tile_mode,
               fused_comm=FusedComm(peer_bufs, n_local * k, d_out), _gammas_by_out_row=True)
        ep.hdl.barrier(channel=0)
        y_dp = peer_bufs[rank]
    else:
        gam = None
        if gate_weighted:
            gam = sm.vals.float().reshape(-1)[mm.col_sorted_indx.long().clamp(min=0)]
        o = matmul(h, w2_local, None, rg_local, gammas=gam, _tile_mode=tile_mode)
        y_dp = convert_ep_to_dp(o, expt_assignment, sm.indx, mm.col_sorted_indx, ep)
    z, _ = reduce(y_dp.view(n_local, k, -1), dim=1)
    return z


class EpLayerGraph:
    """One expert-parallel layer call captured into a CUDA graph (the reference tests its EP layer under graph
    replay too, ``tests/test_distributed.py:248-340``). At 8 GPUs a rank's share of the layer is a few hundred
    microseconds of GPU work issued by some thirty launches; replaying a graph takes the host out of the
    critical path. Needs the ``SymmetricMemoryPool`` transport (nothing in it touches the host; the barrier
    keeps its epoch on the device, so a replay is a valid next barrier). Every rank must build and replay it the
    same number of times. ``x_local`` / ``logits_local`` are the static inputs: copy new data into them, then
    ``replay()``; the result tensor is reused from replay to replay."""

    def __init__(self, x_local, logits_local, w1_local, w2_local, k, expt_assignment, pool: SymmetricMemoryPool, **kw):
        assert isinstance(pool, SymmetricMemoryPool), "graph capture needs the peer-store transport"
        self.x, self.logits = x_local, logits_local
        args = (x_local, logits_local, w1_local, w2_local, k, expt_assignment, pool)
        cur = torch.cuda.current_stream(x_local.device)
        side = torch.cuda.Stream(x_local.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(2):  # first calls load kernels and cache per-device state: keep them out of the capture
                moe_layer_ep(*args, **kw)
        cur.wait_stream(side)
        torch.cuda.synchronize(x_local.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.out = moe_layer_ep(*args, **kw)

    def replay(self):
        self.graph.replay()
        return self.out
