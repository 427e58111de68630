"""Drop-in counterparts of the reference's ``triton_kernels`` MoE entry points
(``python/triton_kernels/triton_kernels`` in the reference): ``topk``, ``SparseMatrix``,
``make_bitmatrix_metadata``, ``make_ragged_tensor_metadata``, ``matmul`` (ragged / gather / scatter /
gammas / fused SwiGLU), ``swiglu``, ``reduce`` and the expert-parallel token exchange. Same function
names, argument names and result field names; CUDA kernels underneath, no Triton."""
