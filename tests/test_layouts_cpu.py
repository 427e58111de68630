"""Host-side layout conversions of the MoE weight path, checked on the CPU against element-by-element restatements
of the layouts the kernels read (``include/triton_b200.h``, tb200_moe_gemm_mx4_args): the blocked MXFP4 values
``[E][ceil(N/256)][ceil(K/128)][256][64]``, the 512-byte scale atoms ``[E][ceil(N/128)][ceil(K/128)][n%32][n/32%4][k/32%4]``
and the padding of K and N tails (zero codes, scale 1.0 = 127)."""
import numpy as np
import pytest
import torch


@pytest.mark.parametrize("E,K,N", [(2, 256, 256), (1, 96, 48), (3, 832, 400)])
def test_mxfp4_value_layout_blocks_and_pads(E, K, N):
    from triton_b200.triton_kernels.tensor import FP4, convert_layout, wrap_torch_tensor
    from triton_b200.triton_kernels.tensor_details.layout import make_default_matmul_mxfp4_w_layout
    g = torch.Generator().manual_seed(1)
    v = torch.randint(0, 256, (E, K // 2, N), generator=g).to(torch.uint8)
    out = convert_layout(wrap_torch_tensor(v, dtype=FP4), make_default_matmul_mxfp4_w_layout(mx_axis=1))
    tiles, ksteps = (N + 255) // 256, (K + 127) // 128
    blocked = out.data.numpy()
    assert blocked.shape == (E, tiles, ksteps, 256, 64) and out.shape == (E, K, N)
    ref = np.zeros((E, tiles, ksteps, 256, 64), dtype=np.uint8)
    vn = v.numpy()
    for e in range(E):
        for n in range(N):
            for kb in range(K // 2):
                ref[e, n // 256, kb // 64, n % 256, kb % 64] = vn[e, kb, n]
    assert np.array_equal(blocked, ref)


@pytest.mark.parametrize("E,K,N", [(2, 256, 256), (1, 96, 48), (3, 832, 400)])
def test_mx_scale_layout_atoms_and_pads(E, K, N):
    from triton_b200.triton_kernels.tensor import convert_layout, wrap_torch_tensor
    from triton_b200.triton_kernels.tensor_details.layout import make_default_matmul_mxfp4_w_scale_layout
    g = torch.Generator().manual_seed(2)
    s = torch.randint(100, 140, (E, K // 32, N), generator=g).to(torch.uint8)
    out = convert_layout(wrap_torch_tensor(s), make_default_matmul_mxfp4_w_scale_layout(mx_axis=1))
    nb, ksteps = (N + 127) // 128, (K // 32 + 3) // 4
    atoms = out.data.numpy().reshape(E, nb, ksteps, 32, 4, 4)
    ref = np.full((E, nb, ksteps, 32, 4, 4), 127, dtype=np.uint8)
    sn = s.numpy()
    for e in range(E):
        for n in range(N):
            for kb in range(K // 32):
                ref[e, n // 128, kb // 4, n % 32, (n // 32) % 4, kb % 4] = sn[e, kb, n]
    assert np.array_equal(atoms, ref)


@pytest.mark.parametrize("E,K,N", [(2, 128, 128), (1, 416, 400)])
def test_fp8_weight_layout_and_scale_atoms(E, K, N):
    """fp8 weights: [E, N, K] bytes with K contiguous (a view when the caller's tensor already is), MXFP8 scales as
    atoms with 127 past N and K."""
    from triton_b200.triton_kernels.matmul import _fp8_weight_kernel_layout
    g = torch.Generator().manual_seed(3)
    w = torch.randn(E, K, N, generator=g).to(torch.float8_e4m3fn)
    s = torch.randint(100, 140, (E, (K + 31) // 32, N), generator=g).to(torch.uint8)
    wk, atoms, dims = _fp8_weight_kernel_layout(w, s, None)
    assert dims == (E, K, N) and wk.shape == (E, N, K) and wk.is_contiguous()
    assert torch.equal(wk.view(torch.uint8), w.transpose(1, 2).contiguous().view(torch.uint8))
    col_major = w.transpose(1, 2).contiguous().transpose(1, 2)      # K contiguous: no copy is made
    wk2, _, _ = _fp8_weight_kernel_layout(col_major, None, None)
    assert wk2.data_ptr() == col_major.data_ptr()
    nb, ksteps = (N + 127) // 128, (K + 127) // 128
    a = atoms.numpy().reshape(E, nb, ksteps, 32, 4, 4)
    ref = np.full((E, nb, ksteps, 32, 4, 4), 127, dtype=np.uint8)
    sn = s.numpy()
    for e in range(E):
        for n in range(N):
            for kb in range(sn.shape[1]):
                ref[e, n // 128, kb // 4, n % 32, (n // 32) % 4, kb % 4] = sn[e, kb, n]
    assert np.array_equal(a, ref)
    with pytest.raises(NotImplementedError):
        _fp8_weight_kernel_layout(torch.zeros(1, 72, 16).to(torch.float8_e4m3fn), None, None)
