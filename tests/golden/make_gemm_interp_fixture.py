"""Generates ``gemm_interp_512.npz``: outputs of the REFERENCE's own tutorial GEMM kernel
(``python/tutorials/03-matrix-multiplication.py:228-320`` in the reference checkout) run on CPU
under ``TRITON_INTERPRET=1`` for the 512^3 configuration.

Run it where the reference checkout is mounted:
    python tests/golden/make_gemm_interp_fixture.py /path/to/reference
The kernel source is read from the checkout at run time and written to a temporary module
(the interpreter needs a real file for ``inspect.getsource``); nothing of it is stored in this
repository. Launch parameters follow the tutorial's smallest autotune config because the
autotuner itself needs a GPU driver: BLOCK_SIZE_M=64, BLOCK_SIZE_N=64, BLOCK_SIZE_K=32,
GROUP_SIZE_M=8, ACTIVATION="". The interpreter's ``tl.dot`` mishandles bf16 (it multiplies the
raw uint16 payloads), so the inputs are the fp16 roundings of the seed-0 N(0,1) matrices; the
kernel's output dtype is fp16.

Stored: rows 0, 17, 255 and 511 of C (fp16), the float64 sum of C and of |C|, and the input seed.
"""
import hashlib
import importlib.util
import os
import re
import sys
import tempfile

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch

ROWS = [0, 17, 255, 511]


def load_kernel(ref_root):
    path = os.path.join(ref_root, "python", "tutorials", "03-matrix-multiplication.py")
    src = open(path).read()
    m = re.search(r"@triton\.jit\ndef matmul_kernel\(.*?(?=\n# We can fuse `leaky_relu`)", src, re.S)
    assert m, "kernel not found in the tutorial"
    lr = re.search(r"@triton\.jit\ndef leaky_relu\(x\):\n.*?\n\n", src, re.S)
    body = "import triton\nimport triton.language as tl\n\n" + m.group(0) + "\n\n" + lr.group(0)
    d = tempfile.mkdtemp()
    p = os.path.join(d, "ref_tutorial03_kernel.py")
    open(p, "w").write(body)
    spec = importlib.util.spec_from_file_location("ref_tutorial03_kernel", p)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.matmul_kernel


def main():
    ref_root = sys.argv[1]  # path of the reference checkout
    kernel = load_kernel(ref_root)
    M = N = K = 512
    torch.manual_seed(0)
    a = torch.randn(M, K).to(torch.float16)
    b = torch.randn(K, N).to(torch.float16)
    c = torch.empty(M, N, dtype=torch.float16)
    BM, BN, BK, G = 64, 64, 32, 8
    grid = ((M // BM) * (N // BN), )
    kernel[grid](a, b, c, M, N, K, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1),
                 BLOCK_SIZE_M=BM, BLOCK_SIZE_N=BN, BLOCK_SIZE_K=BK, GROUP_SIZE_M=G, ACTIVATION="")
    ref = (a.float() @ b.float())
    err = (c.float() - ref).abs().max().item()
    print("max |interp - torch fp32| =", err)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "gemm_interp_512.npz")
    np.savez_compressed(out, rows=np.array(ROWS), c_rows=c[ROWS].numpy(), c_sum=np.float64(c.double().sum().item()),
                        c_abs_sum=np.float64(c.double().abs().sum().item()), seed=0,
                        a_sha=hashlib.sha256(a.numpy().tobytes()).hexdigest(),
                        b_sha=hashlib.sha256(b.numpy().tobytes()).hexdigest())
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
