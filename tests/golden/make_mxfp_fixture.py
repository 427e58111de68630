"""Generates ``mxfp_cases.npz``: inputs and the outputs of the reference's own torch implementations
``downcast_to_mxfp_torch`` / ``upcast_from_mxfp_torch``
(python/triton_kernels/triton_kernels/numerics_details/mxfp.py:212, :384), imported from the reference
checkout given as argv[1]. Run once where the reference is available; the
committed fixture is what the tests read."""
import sys

import numpy as np
import torch

import ast
import math
import types

ref_root = sys.argv[1]  # path of the reference checkout
ref_file = ref_root + "/python/triton_kernels/triton_kernels/numerics_details/mxfp.py"
# The module's import line pulls in the fork's own triton build; only the pure-torch functions are needed,
# so their definitions are taken from the reference file and executed as they stand.
wanted = {"DequantScaleRoundingMode", "right_shift_unsigned", "get_max_quant_val", "downcast_to_mxfp_torch",
          "cvt_e2m1_to_fp32", "upcast_from_mxfp_torch"}
tree = ast.parse(open(ref_file).read())
body = [n for n in tree.body if isinstance(n, (ast.FunctionDef, ast.ClassDef)) and n.name in wanted]
assert {n.name for n in body} == wanted
import enum  # noqa: E402
import torch.nn.functional as F  # noqa: E402


class _Const:  # the reference reads MXFP_BLOCK_SIZE.value / NVFP_BLOCK_SIZE.value
    def __init__(self, v):
        self.value = v


ns = {"torch": torch, "F": F, "math": math, "Enum": enum.Enum, "MXFP_BLOCK_SIZE": _Const(32), "NVFP_BLOCK_SIZE": _Const(16),
      "triton": types.SimpleNamespace(cdiv=lambda a, b: (a + b - 1) // b)}
exec(compile(ast.Module(body=body, type_ignores=[]), ref_file, "exec"), ns)
DequantScaleRoundingMode = ns["DequantScaleRoundingMode"]
downcast_to_mxfp_torch = ns["downcast_to_mxfp_torch"]
upcast_from_mxfp_torch = ns["upcast_from_mxfp_torch"]

g = torch.Generator().manual_seed(11)
out = {}
cases = {
    "normal": torch.randn(6, 96, generator=g),
    "wide": torch.randn(4, 64, generator=g) * torch.pow(2.0, torch.randint(-20, 20, (4, 64), generator=g).float()),
    # every e2m1 tie (midpoints of the value grid) and the saturation edge, scaled so the block scale is 1
    "ties": torch.tensor([[6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, 5.9,
                           0.2499, 0.2501, 0.7499, 0.7501, 2.4999, 2.5001, 4.9999, 5.0001, 0.0, -0.0, 1e-8, -6.0, 3.0, 4.0, 1.0,
                           0.5]]),
    "zeros": torch.zeros(2, 32),
    "axis0": torch.randn(64, 5, generator=g),
}
for name, x in cases.items():
    axis = 0 if name == "axis0" else -1
    x = x.to(torch.bfloat16).to(torch.float32) if name != "ties" else x
    out[f"{name}_x"] = x.numpy()
    for mode in (DequantScaleRoundingMode.ROUND_UP, DequantScaleRoundingMode.ROUND_DOWN):
        for qname, qt in (("fp4", torch.uint8), ("e4m3", torch.float8_e4m3fn)):
            v, s = downcast_to_mxfp_torch(x, qt, axis, DEQUANT_SCALE_ROUNDING_MODE=mode)
            key = f"{name}_{qname}_{mode.name}"
            out[key + "_v"] = v.contiguous().view(torch.uint8).numpy()
            out[key + "_s"] = s.contiguous().numpy()
            out[key + "_up"] = upcast_from_mxfp_torch(v, s, torch.float32, axis).numpy()
np.savez_compressed(__file__.rsplit("/", 1)[0] + "/mxfp_cases.npz", **out)
print("wrote", len(out), "arrays")
