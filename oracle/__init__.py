"""CPU oracle — TEST INFRASTRUCTURE ONLY.

Plain CPU restatements (numpy for integer/byte work, torch-CPU fp32 for floating point) of the
reference's own torch twins for every function on the hot path. Only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / ``--impl reference`` legs may import
this package; nothing under ``triton_b200/`` does, and the product has no CPU path.

Parity pins (how the restatements themselves are checked, see ``tests/test_oracle.py``):
  * GEMM: outputs of the reference's tutorial-03 kernel run under ``TRITON_INTERPRET=1`` in the
    build container (``tests/golden/gemm_interp_512.npz`` + the script that made it).
  * routing metadata: the literal known-answer examples in the reference's docstrings
    (``tensor_details/bitmatrix.py:10-19``, ``tensor_details/ragged_tensor.py:14-30``,
    ``RaggedTensorMetadata.n_blocks`` ``:73-77``).
  * attention / MXFP8 / scaled_mm / MoE GEMM: the reference tests compare against torch
    expressions (``F.scaled_dot_product_attention``, dequantise-then-matmul, ``matmul_torch``);
    the restatements here are those expressions. The MXFP8 *quantiser* the reference's tests use
    is torchao's ``MXTensor.to_mx`` (third-party, unpinned ``git+https://github.com/pytorch/ao``
    HEAD, not in the checkout): parity of the quantiser is UNPINNED; parity of the GEMM on given
    quantised inputs is pinned by the dequantise-then-matmul expression.
"""
