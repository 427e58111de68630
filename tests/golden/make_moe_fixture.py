"""Generates ``moe_cases.npz``: seeded inputs and the outputs of the reference's own torch twins for the
MoE path, executed here as they stand in the reference checkout given as argv[1]
(paths inside python/triton_kernels/triton_kernels/):

  topk_torch                            topk.py:144-185
  make_bitmatrix_metadata_torch         tensor_details/bitmatrix.py:157-168
  make_ragged_tensor_metadata_torch     tensor_details/ragged_tensor.py:217-253  (+ RaggedTensorMetadata :12-94)
  remap_ragged_tensor_metadata_torch    tensor_details/ragged_tensor.py:388-433
  matmul_torch (+ apply_precision, scale, compute_actual_scale)   matmul.py:755-914
  swiglu_torch                          swiglu.py:89-100
  reduce_torch                          reduce.py:1173-1206

The reference package cannot be imported here (its modules import the fork's own triton build), so the
definitions of these pure-torch functions are cut out of the reference files with ``ast`` and executed
unchanged in a namespace that supplies the few names they look up (dataclass holders, a precision
config with every scale unset). Two environment shims, because this box has no GPU: ``matmul_torch``
builds an unused index tensor with ``device="cuda"``, so ``torch.arange`` is wrapped to place it on the
CPU; and ``torch.histc`` has no integer CPU kernel, so it is handed the same values as floats.

Run once where the reference is available: ``python tests/golden/make_moe_fixture.py /path/to/reference``.
The committed ``moe_cases.npz`` is what ``tests/test_oracle.py`` and the GPU tests read.
"""
import ast
import itertools
import sys
import types
from dataclasses import dataclass
from typing import Callable, Optional

import numpy as np
import torch

ref_root = sys.argv[1]
TK = ref_root + "/python/triton_kernels/triton_kernels/"


def cut(path, names):
    tree = ast.parse(open(path).read())
    body = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in names]
    assert {n.name for n in body} == set(names), (path, names)
    return compile(ast.Module(body=body, type_ignores=[]), path, "exec")


class _Torch:
    """torch, with arange(device="cuda") mapped to the CPU and histc fed floats (see the module docstring)."""

    def __getattr__(self, name):
        return getattr(torch, name)

    @staticmethod
    def arange(*a, **kw):
        if kw.get("device") == "cuda":
            kw["device"] = "cpu"
        return torch.arange(*a, **kw)

    @staticmethod
    def histc(x, **kw):
        return torch.histc(x.float(), **kw)


class _Holder:
    def __init__(self, **kw):
        self.__dict__.update(kw)


# ---------------------------------------------------------------- namespaces for the cut-out code
ns_topk = {"torch": torch, "Optional": Optional, "Tensor": type("Tensor", (), {}), "BIT": None,
           "wrap_torch_tensor": lambda data, dtype=None, shape=None: data,
           "SparseMatrix": lambda vals, indx, mask: _Holder(vals=vals, indx=indx, mask=mask)}
exec(cut(TK + "topk.py", ["topk_torch"]), ns_topk)
topk_torch = ns_topk["topk_torch"]

ns_bm = {"torch": _Torch(),
         "BitmatrixMetadata": lambda col_sum, col_sorted_indx, row_sorted_indx: _Holder(
             col_sum=col_sum, col_sorted_indx=col_sorted_indx, row_sorted_indx=row_sorted_indx)}
exec(cut(TK + "tensor_details/bitmatrix.py", ["make_bitmatrix_metadata_torch"]), ns_bm)
make_bitmatrix_metadata_torch = ns_bm["make_bitmatrix_metadata_torch"]

ns_rg = {"torch": torch, "dataclass": dataclass, "is_hip": lambda: False}
exec(cut(TK + "tensor_details/ragged_tensor.py",
         ["RaggedTensorMetadata", "make_ragged_tensor_metadata_torch", "remap_ragged_tensor_metadata_torch"]), ns_rg)
make_ragged_tensor_metadata_torch = ns_rg["make_ragged_tensor_metadata_torch"]
remap_ragged_tensor_metadata_torch = ns_rg["remap_ragged_tensor_metadata_torch"]

# apply_precision does `from .tensor_details import layout` and `from .numerics_details.mxfp import
# upcast_from_mxfp` before looking at the config; neither is used when no MX scale is set.
pkg = types.ModuleType("tkstub")
pkg.__path__ = []
td = types.ModuleType("tkstub.tensor_details")
td.layout = types.SimpleNamespace()
nd = types.ModuleType("tkstub.numerics_details")
nd.__path__ = []
mx = types.ModuleType("tkstub.numerics_details.mxfp")
mx.upcast_from_mxfp = None
sys.modules.update({"tkstub": pkg, "tkstub.tensor_details": td, "tkstub.numerics_details": nd,
                    "tkstub.numerics_details.mxfp": mx})
no_flex = _Holder(lhs_data=_Holder(scale=None), rhs_data=_Holder(scale=None),
                  out_data=_Holder(actual_scale=None, expected_scale=None))
PLAIN = _Holder(flex_ctx=no_flex, a_mx_scale=None, b_mx_scale=None, out_dtype=None)
ns_mm = {"torch": _Torch(), "itertools": itertools, "__package__": "tkstub", "__name__": "tkstub.matmul",
         "RaggedTensorMetadata": ns_rg["RaggedTensorMetadata"], "PrecisionConfig": lambda: PLAIN,
         "convert_layout": None, "compute_actual_scale": None}
exec(cut(TK + "matmul.py", ["apply_precision", "scale", "matmul_torch"]), ns_mm)
matmul_torch = ns_mm["matmul_torch"]

ns_sw = {"torch": torch}
exec(cut(TK + "swiglu.py", ["swiglu_torch"]), ns_sw)
swiglu_torch = ns_sw["swiglu_torch"]

tk = types.ModuleType("triton_kernels")
tk.__path__ = []
tknd = types.ModuleType("triton_kernels.numerics_details")
tknd.__path__ = []
tkmx = types.ModuleType("triton_kernels.numerics_details.mxfp")
tkmx.downcast_to_mxfp_torch = tkmx.upcast_from_mxfp_torch = None
sys.modules.update({"triton_kernels": tk, "triton_kernels.numerics_details": tknd,
                    "triton_kernels.numerics_details.mxfp": tkmx})
ns_rd = {"torch": torch, "Optional": Optional, "Callable": Callable, "InFlexData": lambda: None,
         "OutFlexData": lambda: None, "compute_actual_scale": None}
exec(cut(TK + "reduce.py", ["reduce_torch"]), ns_rd)
reduce_torch = ns_rd["reduce_torch"]

# ---------------------------------------------------------------- cases
g = torch.Generator().manual_seed(21)
out = {}


def put(key, t):
    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        t = t.float()
    if t.dtype == torch.uint32:
        t = t.view(torch.int32)
    out[key] = t.contiguous().numpy()


# -- top-k: plain, heavy ties (values on a 5-point grid), padded rows, no softmax, provided indices
E, K = 128, 4
topk_inputs = {
    "plain": (torch.randn(37, E, generator=g), dict()),
    "ties": (torch.randint(0, 5, (40, E), generator=g).float() * 0.5, dict()),
    "padded": (torch.randn(64, E, generator=g), dict(n_rows=50)),
    "nosoftmax": (torch.randn(33, 96, generator=g), dict(apply_softmax=False)),
    "bf16": (torch.randn(48, E, generator=g).to(torch.bfloat16), dict()),
}
for name, (x, kw) in topk_inputs.items():
    sm = topk_torch(x, K, **kw)
    put(f"topk_{name}_x", x)
    put(f"topk_{name}_vals", sm.vals)
    put(f"topk_{name}_indx", sm.indx)
    put(f"topk_{name}_bits", sm.mask)
    out[f"topk_{name}_kw"] = np.array([kw.get("n_rows", x.shape[0]), int(kw.get("apply_softmax", True)),
                                       int(x.dtype == torch.bfloat16)])
x = torch.randn(20, E, generator=g)
given = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(20)]).to(torch.int16)
sm = topk_torch(x, K, y_indx=given)
put("topk_given_x", x), put("topk_given_yin", given), put("topk_given_vals", sm.vals), put("topk_given_indx", sm.indx)
put("topk_given_bits", sm.mask)

# -- bitmatrix metadata from routing indices (with a padded tail of -1 rows)
for name in ("plain", "ties", "padded"):
    indx = torch.from_numpy(out[f"topk_{name}_indx"])
    bm = torch.zeros(indx.shape[0], E)  # only .shape[1] is read
    md = make_bitmatrix_metadata_torch(indx, bm)
    put(f"bm_{name}_col_sum", md.col_sum), put(f"bm_{name}_col_sorted", md.col_sorted_indx)
    put(f"bm_{name}_row_sorted", md.row_sorted_indx)

# -- ragged metadata (docstring example, zeros, many small slices) and its remap
ragged_inputs = {
    "doc": torch.tensor([15, 17, 0, 127], dtype=torch.int32),
    "mixed": torch.tensor([0, 300, 1, 128, 129, 0, 16, 5], dtype=torch.int32),
    "routing": torch.from_numpy(out["bm_plain_col_sum"]).int(),
    "empty": torch.zeros(6, dtype=torch.int32),
}
for name, ss in ragged_inputs.items():
    tot = int(ss.sum())
    md = make_ragged_tensor_metadata_torch(ss, tot)
    put(f"rg_{name}_slice_sizes", ss), put(f"rg_{name}_slice_offs", md.slice_offs)
    put(f"rg_{name}_block_offs", md.block_offs_data), put(f"rg_{name}_block_sched", md.block_schedule_data)
    if name in ("mixed", "routing"):
        n = ss.shape[0]
        keep = torch.randperm(n, generator=g)[: n // 2].sort().values
        smap = torch.full((n, ), -1, dtype=torch.int32)
        smap[keep] = torch.arange(keep.shape[0], dtype=torch.int32)
        rm = remap_ragged_tensor_metadata_torch(md, smap)
        put(f"rg_{name}_map", smap), put(f"rg_{name}_re_slice_sizes", rm.slice_sizes)
        put(f"rg_{name}_re_slice_offs", rm.slice_offs), put(f"rg_{name}_re_block_offs", rm.block_offs_data)
        put(f"rg_{name}_re_block_sched", rm.block_schedule_data)


# -- grouped matmul: fp32 tensors holding bf16-representable values, so the twin's result is exact fp32
def bf(t):
    return t.to(torch.bfloat16).float()


Eg, Kd, Nd, T = 5, 64, 48, 24
sizes = torch.tensor([7, 0, 40, 1, 16], dtype=torch.int32)  # one empty expert
R = int(sizes.sum())
a = bf(torch.randn(T, Kd, generator=g))
w = bf(torch.randn(Eg, Kd, Nd, generator=g) * 0.2)
bias = torch.randn(Eg, Nd, generator=g)
gam = torch.rand(R, generator=g)
gather = torch.randint(0, T, (R, ), generator=g, dtype=torch.int32)
scatter = torch.randperm(R, generator=g).to(torch.int32)
scatter[torch.randperm(R, generator=g)[:6]] = -1
rg = make_ragged_tensor_metadata_torch(sizes, R)
put("mm_a", a), put("mm_w", w), put("mm_bias", bias), put("mm_gammas", gam), put("mm_sizes", sizes)
put("mm_gather", gather), put("mm_scatter", scatter)
a_sorted = a[gather.long()]
put("mm_y_plain", matmul_torch(a_sorted, w, None, rg, precision_config=PLAIN))
put("mm_y_gather", matmul_torch(a, w, None, rg, gather_indx=gather.long(), precision_config=PLAIN))
put("mm_y_bias_gamma", matmul_torch(a_sorted, w, bias, rg, gammas=gam, precision_config=PLAIN))
put("mm_y_scatter", matmul_torch(a_sorted, w, None, rg, scatter_indx=scatter.long(), gammas=gam, precision_config=PLAIN))
put("mm_y_all", matmul_torch(a, w, bias, rg, gather_indx=gather.long(), scatter_indx=scatter.long(), gammas=gam,
                             precision_config=PLAIN))
for limit in (None, 1.4):
    y = matmul_torch(a, w, bias, rg, gather_indx=gather.long(), precision_config=PLAIN)
    put(f"mm_y_swiglu_{limit}", swiglu_torch(y, 1.1, _Holder(limit=limit)))
# the same in bf16 (the dtype the kernels run in): the twin rounds each expert's block to bf16
put("mm_y_all_bf16", matmul_torch(a.to(torch.bfloat16), w.to(torch.bfloat16), bias, rg, gather_indx=gather.long(),
                                  scatter_indx=scatter.long(), gammas=gam, precision_config=PLAIN))

# -- swiglu
xs = torch.randn(9, 64, generator=g) * 3
put("sw_x", xs)
put("sw_y_None", swiglu_torch(xs, 1.702, _Holder(limit=None)))
put("sw_y_limit", swiglu_torch(xs, 1.702, _Holder(limit=2.0)))

# -- reduce over the k slots, with mask and scale
xr = bf(torch.randn(11, 4, 32, generator=g))
mask = torch.rand(11, 4, 1, generator=g) > 0.3
sc = torch.rand(11, 4, 1, generator=g)
put("rd_x", xr), put("rd_mask", mask.to(torch.uint8)), put("rd_scale", sc)
put("rd_y_plain", reduce_torch(xr, 1, x_flex=None, y_flex=None)[0])
put("rd_y_mask", reduce_torch(xr, 1, mask=mask, x_flex=None, y_flex=None)[0])
put("rd_y_scale", reduce_torch(xr, 1, scale=sc, x_flex=None, y_flex=None)[0])
put("rd_y_both", reduce_torch(xr, 1, mask=mask, scale=sc, x_flex=None, y_flex=None)[0])
put("rd_y_both_bf16", reduce_torch(xr.to(torch.bfloat16), 1, mask=mask, scale=sc, x_flex=None, y_flex=None)[0])

# -- batched matmul: [B, M, K] x [B, K, N] + bias [B, N] (matmul.py:864-868, 893-898)
Bb, Mb, Kb, Nb = 3, 10, 32, 24
ab = bf(torch.randn(Bb, Mb, Kb, generator=g))
wb = bf(torch.randn(Bb, Kb, Nb, generator=g) * 0.2)
biasb = torch.randn(Bb, Nb, generator=g)
put("bt_a", ab), put("bt_w", wb), put("bt_bias", biasb)
put("bt_y", matmul_torch(ab, wb, biasb, precision_config=PLAIN))

# -- ragged K: out[e] = a[:, ks_e] @ b[ks_e, :] with one empty slice (matmul.py:836-861)
ks = torch.tensor([16, 0, 40, 8], dtype=torch.int32)
Ktot, Mr, Nr = int(ks.sum()), 12, 20
ar = bf(torch.randn(Mr, Ktot, generator=g))
wr = bf(torch.randn(Ktot, Nr, generator=g) * 0.2)
rgk = make_ragged_tensor_metadata_torch(ks, Ktot)
put("rk_a", ar), put("rk_w", wr), put("rk_sizes", ks)
put("rk_y", matmul_torch(ar, wr, None, rgk, rgk, precision_config=PLAIN))

# -- fp8 x fp8 with flexpoint scales, grouped (matmul.py:755-800: the operands are multiplied by lhs / rhs scale;
#    :909-914: actual_scale = max |out| / max_finite(out dtype), the result divided by expected_scale)
ns_num = {}
for node in ast.parse(open(TK + "numerics.py").read()).body:
    if isinstance(node, ast.Assign) and all(isinstance(t, ast.Name) and t.id.startswith("MAX_FINITE") for t in node.targets):
        exec(compile(ast.Module(body=[node], type_ignores=[]), TK + "numerics.py", "exec"), {"torch": torch}, ns_num)
tknum = types.ModuleType("triton_kernels.numerics")
tknum.__dict__.update(ns_num)
sys.modules["triton_kernels.numerics"] = tknum
ns_cs = {"torch": torch}
exec(cut(TK + "matmul.py", ["compute_actual_scale"]), ns_cs)
ns_mm["compute_actual_scale"] = ns_cs["compute_actual_scale"]
Ef, Kf, Nf = 3, 48, 40
sizes_f = torch.tensor([9, 0, 22], dtype=torch.int32)
Rf = int(sizes_f.sum())
af = (torch.randn(Rf, Kf, generator=g)).to(torch.float8_e5m2)
wf = (torch.randn(Ef, Kf, Nf, generator=g) * 0.5).to(torch.float8_e5m2)
gam_f = torch.rand(Rf, generator=g)
ls, rs, es = torch.tensor(0.5), torch.tensor(0.25), torch.tensor(0.03125)
actual = torch.zeros(())
FLEX = _Holder(flex_ctx=_Holder(lhs_data=_Holder(scale=ls), rhs_data=_Holder(scale=rs),
                                out_data=_Holder(actual_scale=actual, expected_scale=es)),
               a_mx_scale=None, b_mx_scale=None, out_dtype=torch.float8_e5m2)
rgf = make_ragged_tensor_metadata_torch(sizes_f, Rf)
put("f8_a", af.view(torch.uint8)), put("f8_w", wf.view(torch.uint8)), put("f8_sizes", sizes_f), put("f8_gammas", gam_f)
put("f8_scales", torch.stack([ls, rs, es]))
put("f8_y", matmul_torch(af, wf, None, rgf, gammas=gam_f, precision_config=FLEX))
put("f8_actual", actual.reshape(1))

np.savez_compressed(__file__.rsplit("/", 1)[0] + "/moe_cases.npz", **out)
print("wrote", len(out), "arrays")
