"""Oracle for the MoE path: routing metadata (bit-exact integer work, numpy) and the grouped
GEMM / SwiGLU / k-way reduce (fp32 torch-CPU). Test infrastructure only.

Each function restates the torch twin that the reference's own tests use as ground truth
(paths are inside python/triton_kernels/triton_kernels/ of the reference):
  topk_ref                   <- topk_torch                          topk.py:144-185
  bitmatrix_metadata_ref     <- make_bitmatrix_metadata_torch        tensor_details/bitmatrix.py:157-168
  ragged_metadata_ref        <- make_ragged_tensor_metadata_torch    tensor_details/ragged_tensor.py:217-253
  n_blocks / max_n_blocks    <- RaggedTensorMetadata.n_blocks        tensor_details/ragged_tensor.py:73-81
  remap_ragged_metadata_ref  <- remap_ragged_tensor_metadata_torch   tensor_details/ragged_tensor.py:388-433
  swiglu_ref                 <- swiglu_torch                         swiglu.py:89-100
  grouped_matmul_ref         <- matmul_torch                         matmul.py:823-914
  reduce_ref                 <- reduce_torch                         reduce.py:1173-1206
  moe_layer_ref              <- mixture_of_expt_nosharded            tests/test_distributed.py:201-218
                                (plus the gate-weighted combine of the MoE benchmark configuration)
  batched_matmul_ref         <- matmul_torch, batched inputs          matmul.py:864-898
  ragged_k_matmul_ref        <- matmul_torch, b_ragged_metadata       matmul.py:836-861
  flex_actual_scale_ref      <- compute_actual_scale                  matmul.py:810-820
  quantize_mxfp8_ref         <- downcast_to_mxfp_torch (fp8, e8m0,   numerics_details/mxfp.py:212-318
                                ROUND_UP), the twin of the quantize_mxfp8_fn matmul epilogue
  dequantize_mxfp8_ref       <- upcast_from_mxfp_torch (fp8)         numerics_details/mxfp.py:384-449
"""
from dataclasses import dataclass

import numpy as np
import torch

BLOCK_SIZES = (16, 32, 64, 128)  # RaggedTensorMetadata.block_sizes() on CUDA: 2**4 .. 2**7


# ----------------------------------------------------------------------------- top-k

def topk_ref(x: torch.Tensor, k: int, apply_softmax: bool = True, n_rows=None):
    """Returns (vals [rows, k] in x.dtype, indx int32 [rows, k], bitmatrix uint32 [rows, ceil(cols/32)]).

    Selection: the k largest per row, ties to the smaller column index (stable argsort of -x);
    softmax over the k selected values in fp32, rounded to x.dtype; values (and their indices)
    sorted in descending order, stable. Rows >= n_rows carry indx -1 and no mask bits.
    """
    x = x.detach().cpu()
    rows, cols = x.shape
    if n_rows is None:
        n_rows = rows
    indx = torch.argsort(-x.float(), dim=1, stable=True)[:, :k]
    vals = torch.take_along_dim(x[:n_rows], indx[:n_rows], dim=1)
    vals = torch.cat([vals, x[n_rows:, :k]], dim=0)
    if apply_softmax:
        vals = torch.softmax(vals.float(), dim=-1).to(x.dtype)
    vals_sorted, order = torch.sort(vals.float(), dim=1, descending=True, stable=True)
    indx = torch.gather(indx, 1, order).to(torch.int32)
    indx[n_rows:] = -1
    words = (cols + 31) // 32
    bits = np.zeros((rows, words), dtype=np.uint32)
    ind = indx.numpy()
    for j in range(k):
        c = ind[:n_rows, j].astype(np.int64)
        np.bitwise_or.at(bits, (np.arange(n_rows), c // 32), (np.uint32(1) << (c % 32).astype(np.uint32)))
    return vals_sorted.to(x.dtype), indx, torch.from_numpy(bits.view(np.int32))


# ----------------------------------------------------------------------------- bitmatrix metadata

@dataclass
class BitmatrixMetadataRef:
    col_sum: np.ndarray          # int32 [n_cols]: entries per column (tokens per expert)
    col_sorted_indx: np.ndarray  # int32 [n]: row-major entry ids grouped by column ("combine" order)
    row_sorted_indx: np.ndarray  # int32 [n]: position of each row-major entry in column order ("dispatch")


def bitmatrix_metadata_ref(nonzero_indx, n_cols: int) -> BitmatrixMetadataRef:
    flat = np.asarray(nonzero_indx).reshape(-1).astype(np.int32)
    n = flat.shape[0]
    valid = flat != -1
    col_sorted = np.argsort(flat[valid], kind="stable").astype(np.int32)
    col_sorted = np.concatenate([col_sorted, np.full(n - col_sorted.shape[0], -1, np.int32)])
    cvalid = col_sorted != -1
    row_sorted = np.argsort(col_sorted[cvalid], kind="stable").astype(np.int32)
    row_sorted = np.concatenate([row_sorted, np.full(n - row_sorted.shape[0], -1, np.int32)])
    col_sum = np.bincount(flat[valid], minlength=n_cols).astype(np.int32)[:n_cols]
    return BitmatrixMetadataRef(col_sum, col_sorted, row_sorted)


# ----------------------------------------------------------------------------- ragged metadata

def n_blocks(n_slices: int, n_total_rows: int, block_size: int) -> int:
    if n_total_rows <= n_slices:
        return n_total_rows
    return n_slices - 1 - ((n_slices - n_total_rows - 1) // block_size)


def max_n_blocks(n_slices: int, n_total_rows: int) -> int:
    return n_blocks(n_slices, n_total_rows, min(BLOCK_SIZES))


@dataclass
class RaggedMetadataRef:
    slice_sizes: np.ndarray          # int32 [E]
    slice_offs: np.ndarray           # int32 [E+1]
    block_offs_data: np.ndarray      # int32 [4, E+1]
    block_schedule_data: np.ndarray  # int32 [4, max_n_blocks]; (block_in_slice << 16) | slice, -1 padded


def ragged_metadata_ref(slice_sizes, n_total_rows: int) -> RaggedMetadataRef:
    ss = np.asarray(slice_sizes).astype(np.int32)
    E = ss.shape[0]
    mnb = max_n_blocks(E, n_total_rows)
    slice_offs = np.concatenate([[0], np.cumsum(ss)]).astype(np.int32)
    offs = np.zeros((len(BLOCK_SIZES), E + 1), np.int32)
    sched = np.full((len(BLOCK_SIZES), mnb), -1, np.int32)
    for i, bs in enumerate(BLOCK_SIZES):
        nb = (ss + bs - 1) // bs
        offs[i, 1:] = np.cumsum(nb)
        pos = 0
        for e in range(E):
            for blk in range(int(nb[e])):
                if pos < mnb:
                    sched[i, pos] = (blk << 16) | e
                pos += 1
    return RaggedMetadataRef(ss, slice_offs, offs, sched)


def remap_ragged_metadata_ref(md: RaggedMetadataRef, slice_map) -> RaggedMetadataRef:
    """Metadata of the ragged tensor that keeps slice i iff slice_map[i] != -1, renumbered to
    slice_map[i]; dropped entries are compacted to the end as -1."""
    sm = np.asarray(slice_map).astype(np.int64)
    E = md.slice_sizes.shape[0]
    keep = sm != -1
    keep1 = np.concatenate([keep, [False]])

    def compact(vals, cond):
        return np.concatenate([vals[cond], np.full(int((~cond).sum()), -1, vals.dtype)])

    ss = compact(md.slice_sizes, keep)
    so = compact(md.slice_offs, keep1)
    bo, bs = [], []
    for i in range(md.block_offs_data.shape[0]):
        o = compact(md.block_offs_data[i], keep1)
        sch = md.block_schedule_data[i]
        sid = sch & 0xFFFF
        valid = sid != 0xFFFF
        cond = np.zeros_like(valid)
        cond[valid] = sm[sid[valid]] != -1
        s2 = compact(sch, cond)
        sid2 = s2 & 0xFFFF
        v2 = sid2 != 0xFFFF
        out = s2.copy()
        out[v2] = ((s2[v2].astype(np.int64) & 0xFFFF0000) | sm[sid2[v2]]).astype(np.int32)
        first = int(np.nonzero(o == -1)[0][0])
        o[first] = int((out != -1).sum())
        bo.append(o)
        bs.append(out)
    return RaggedMetadataRef(ss, so, np.stack(bo), np.stack(bs))


# ----------------------------------------------------------------------------- fp parts

def swiglu_ref(a: torch.Tensor, alpha: float, limit=None) -> torch.Tensor:
    """Interleaved gate/linear columns: even columns are the gate g, odd the linear part l.
    out = g * sigmoid(alpha * g) * (l + 1), with g clamped to <= limit and l to [-limit, limit]."""
    g = a[..., ::2]
    l = a[..., 1::2]
    if limit is not None:
        g = g.clamp(max=limit)
        l = l.clamp(min=-limit, max=limit)
    return g * torch.sigmoid(alpha * g) * (l + 1)


def grouped_matmul_ref(a, w, bias=None, slice_sizes=None, gather_indx=None, scatter_indx=None, gammas=None,
                       swiglu=None, out_dtype=None):
    """Per-slice (expert) GEMM with optional row gather on the input, per-row scale, fused SwiGLU
    and row scatter on the output.

    a: [rows_in, K]; w: [E, K, N]; slice_sizes: int [E] rows per expert in expert-sorted order;
    gather_indx: int [R] (row of `a` feeding sorted row r); gammas: fp32 [R] applied after bias and
    activation; swiglu: None or (alpha, limit); scatter_indx: int [R], sorted row r is written to
    output row scatter_indx[r] (-1 = dropped; untouched rows are zero).
    """
    a32 = a.detach().cpu().float()
    w32 = w.detach().cpu().float()
    out_dtype = out_dtype or a.dtype
    E = w32.shape[0]
    R = a32.shape[0] if gather_indx is None else int(np.asarray(gather_indx).shape[0])
    if slice_sizes is None:
        assert E == 1
        offs = [(0, R)]
    else:
        ss = np.asarray(slice_sizes).astype(np.int64)
        cs = np.concatenate([[0], np.cumsum(ss)])
        offs = [(int(cs[i]), int(cs[i + 1])) for i in range(E)]
    n_out = w32.shape[-1] // (2 if swiglu is not None else 1)
    y = torch.zeros(R, n_out, dtype=torch.float32)
    gi = None if gather_indx is None else torch.as_tensor(np.asarray(gather_indx)).long()
    for e, (lo, hi) in enumerate(offs):
        if hi <= lo:
            continue
        idx = torch.arange(lo, hi) if gi is None else gi[lo:hi]
        out = a32[idx] @ w32[e]
        if bias is not None:
            out = out + bias[e].detach().cpu().float()
        if swiglu is not None:
            out = swiglu_ref(out, swiglu[0], swiglu[1])
        if gammas is not None:
            out = out * gammas.detach().cpu().float()[lo:hi, None]
        y[lo:hi] = out
    y = y.to(out_dtype)
    if scatter_indx is None:
        return y
    si = torch.as_tensor(np.asarray(scatter_indx)).long()
    out = torch.zeros(si.shape[0], n_out, dtype=out_dtype)
    msk = si != -1
    out[si[msk]] = y[msk]
    return out


def batched_matmul_ref(a, w, bias=None, swiglu=None, out_dtype=None) -> torch.Tensor:
    """[B, M, K] x [B, K, N] (+ bias [B, N]) -> [B, M, N]: one independent product per batch entry."""
    a32, w32 = a.detach().cpu().float(), w.detach().cpu().float()
    y = torch.matmul(a32, w32)
    if bias is not None:
        y = y + bias.detach().cpu().float()[:, None, :]
    if swiglu is not None:
        y = swiglu_ref(y, swiglu[0], swiglu[1])
    return y.to(out_dtype or a.dtype)


def ragged_k_matmul_ref(a, w, slice_sizes, a_slice_offs=None, w_slice_offs=None, out_dtype=None) -> torch.Tensor:
    """Ragged K: out[e] = a[:, xo_e : xo_e + k_e] @ w[wo_e : wo_e + k_e, :] for every slice e (zeros for an empty
    slice). a: [M, K_total]; w: [K_total, N]; the offsets default to the cumulative slice sizes."""
    a32, w32 = a.detach().cpu().float(), w.detach().cpu().float()
    ss = np.asarray(slice_sizes).astype(np.int64)
    cum = np.concatenate([[0], np.cumsum(ss)])
    xo = cum if a_slice_offs is None else np.asarray(a_slice_offs).astype(np.int64)
    wo = cum if w_slice_offs is None else np.asarray(w_slice_offs).astype(np.int64)
    out = torch.zeros(len(ss), a32.shape[0], w32.shape[1], dtype=torch.float32)
    for e, k in enumerate(ss):
        if k:
            out[e] = a32[:, int(xo[e]):int(xo[e] + k)] @ w32[int(wo[e]):int(wo[e] + k), :]
    return out.to(out_dtype or a.dtype)


def reduce_ref(x: torch.Tensor, dim: int, mask=None, scale=None) -> torch.Tensor:
    x32 = x.detach().cpu().float()
    if scale is not None:
        x32 = x32 * scale.detach().cpu().float()
    if mask is not None:
        x32 = torch.where(mask.detach().cpu().bool(), x32, torch.zeros(()))
    return x32.sum(dim=dim).to(x.dtype)


def moe_layer_ref(x, logits, w1, w2, k: int, alpha: float = 1.0, limit=None, gate_weighted: bool = True):
    """Whole single-GPU MoE layer: top-k routing -> gather GEMM-1 (+SwiGLU) -> GEMM-2 (x gate
    weight) scattered back to (token, slot) order -> sum over the k slots."""
    vals, indx, _ = topk_ref(logits, k, apply_softmax=True)
    E = w1.shape[0]
    md = bitmatrix_metadata_ref(indx.numpy(), E)
    combine = md.col_sorted_indx
    gather = combine // k
    h = grouped_matmul_ref(x, w1, None, md.col_sum, gather_indx=gather, swiglu=(alpha, limit))
    gammas = None
    if gate_weighted:
        gammas = vals.float().reshape(-1)[torch.as_tensor(combine).long()]
    y = grouped_matmul_ref(h, w2, None, md.col_sum, scatter_indx=combine, gammas=gammas)
    return reduce_ref(y.view(-1, k, y.shape[-1]), dim=1)


# ----------------------------------------------------------------------------- MX-quantised activations / outputs


def quantize_mxfp8_ref(x: torch.Tensor, dtype=torch.float8_e4m3fn):
    """MXFP8 quantisation along the last axis: every 32 consecutive values (the last block may be short) share
    the e8m0 scale 2^ceil(log2(amax / max_finite)), computed on the bits as (bits(amax / max_finite) + 0x7FFFFF)
    & 0x7F800000; values are multiplied by the reciprocal of the scale (by 0 when the scale is 0), clamped to the
    finite range and converted with round to nearest even. Returns (values as ``dtype``, scales uint8)."""
    x = x.detach().cpu().float()
    max_q = 448.0 if dtype == torch.float8_e4m3fn else 57344.0
    n = x.shape[-1]
    pad = (-n) % 32
    xp = torch.nn.functional.pad(x, (0, pad))
    valid = torch.nn.functional.pad(torch.ones_like(x, dtype=torch.bool), (0, pad))
    groups = xp.reshape(*xp.shape[:-1], -1, 32)
    amax = torch.where(valid.reshape(groups.shape), groups.abs(), torch.full((), -1.0)).amax(dim=-1, keepdim=True)
    bits = ((amax / max_q).view(torch.int32) + 0x007FFFFF) & 0x7F800000
    scale = bits.view(torch.float32)
    inv = torch.where(scale == 0, torch.zeros(()), 1.0 / scale)
    q = (groups * inv).reshape(xp.shape)[..., :n].clamp(-max_q, max_q).to(dtype)
    return q, (bits >> 23).to(torch.uint8).squeeze(-1)


def dequantize_mxfp8_ref(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp8 values x 2^(scale - 127) per block of 32 along the last axis, in fp32."""
    q32 = q.detach().cpu().float()
    s = torch.pow(2.0, scale.detach().cpu().float() - 127.0).repeat_interleave(32, dim=-1)[..., :q32.shape[-1]]
    return q32 * s


def flex_actual_scale_ref(y: torch.Tensor, dtype=torch.float8_e4m3fn) -> float:
    """The flexpoint scale a kernel reports for its (unscaled) result: max |y| / max_finite(dtype)."""
    max_finite = {torch.float8_e5m2: 57344.0, torch.float8_e4m3fn: 448.0, torch.float16: 65504.0}[dtype]
    return float(y.detach().cpu().float().abs().max()) / max_finite
