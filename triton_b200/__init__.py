"""triton_b200 — hand-written sm_100a (B200) kernels behind the call signatures of the reference's
TLX tutorials and ``triton_kernels`` MoE path. Python here is plumbing (tensors, streams); the
work is done by ``libtriton_b200.so`` through the C ABI in ``include/triton_b200.h``.
There is no CPU or PyTorch fallback: a missing library or a failed launch raises.
"""
__version__ = "0.1.0"
