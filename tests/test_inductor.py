"""The torch.compile hook-up (triton_b200.inductor): the graph rewrite on fake tensors (no GPU needed) and, on a
GPU, a compiled module whose matmuls and attention run through this library's kernels."""
import pytest
import torch


def _fx(fn, *args):
    from torch.fx.experimental.proxy_tensor import make_fx
    return make_fx(fn)(*args)


def test_rewrite_picks_eligible_matmuls_only():
    from torch._subclasses.fake_tensor import FakeTensorMode
    from triton_b200 import inductor as ind
    with FakeTensorMode():
        a = torch.empty(256, 512, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(1024, 512, dtype=torch.bfloat16, device="cuda")
        small = torch.empty(4, 8, dtype=torch.bfloat16, device="cuda")
        f32 = torch.empty(256, 512, device="cuda")
        odd = torch.empty(256, 510, dtype=torch.bfloat16, device="cuda")[:, :508]   # row pitch not 16-byte aligned

        def f(a, w, small, f32, odd):
            return torch.relu(a @ w.t()), small @ small.t(), f32 @ f32.t(), odd @ odd.t()
        g = _fx(f, a, w, small, f32, odd)
        assert ind.rewrite_graph(g.graph) == 1
        targets = [str(n.target) for n in g.graph.nodes if n.op == "call_function"]
        assert targets.count("triton_b200.mm.default") == 1 and targets.count("aten.mm.default") == 3
        g.graph.lint()


def test_rewrite_replaces_inference_flash_attention():
    from torch._subclasses.fake_tensor import FakeTensorMode
    from triton_b200 import inductor as ind
    with FakeTensorMode():
        q = torch.empty(2, 4, 512, 128, dtype=torch.bfloat16, device="cuda")
        q256 = torch.empty(2, 4, 512, 256, dtype=torch.bfloat16, device="cuda")

        def h(q, q256):
            a = torch.ops.aten._scaled_dot_product_flash_attention.default(q, q, q, 0.0, True)[0]
            b = torch.ops.aten._scaled_dot_product_flash_attention.default(q256, q256, q256, 0.0, False)[0]  # head dim 256: kept
            c = torch.ops.aten._scaled_dot_product_flash_attention.default(q, q, q, 0.0, False)
            return a * 2, b, c[0] + c[1].unsqueeze(-1).to(c[0].dtype)   # the log-sum-exp is read: kept
        g = _fx(h, q, q256)
        assert ind.rewrite_graph(g.graph) == 1
        g.graph.lint()
        targets = [str(n.target) for n in g.graph.nodes if n.op == "call_function"]
        assert targets.count("triton_b200.attention.default") == 1
        assert targets.count("aten._scaled_dot_product_flash_attention.default") == 2
        new = next(n for n in g.graph.nodes if str(n.target) == "triton_b200.attention.default")
        assert new.args[3] == pytest.approx(128 ** -0.5) and new.args[4] is True


def test_enable_and_disable_restore_the_inductor_hook():
    import torch._inductor.config as cfg
    from triton_b200 import inductor as ind
    before = cfg.post_grad_custom_post_pass
    ind.enable()
    assert cfg.post_grad_custom_post_pass is not before
    ind.enable()  # idempotent
    ind.disable()
    assert cfg.post_grad_custom_post_pass is before


@pytest.mark.gpu
def test_compiled_module_runs_on_the_library_kernels(cuda):
    """A bf16 MLP block with attention under torch.compile: with the hook enabled its matmuls and its attention go
    through triton_b200::mm / ::attention (the call counters move) and the result matches eager within bf16 tolerance."""
    from triton_b200 import _lib, inductor as ind

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = torch.nn.Linear(256, 3 * 256, bias=False)
            self.up = torch.nn.Linear(256, 1024, bias=False)
            self.down = torch.nn.Linear(1024, 256, bias=False)

        def forward(self, x):                       # x [B, S, 256], 2 heads of 128
            B, S, _ = x.shape
            q, k, v = self.qkv(x).view(B, S, 3, 2, 128).permute(2, 0, 3, 1, 4)
            a = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + a.transpose(1, 2).reshape(B, S, 256)
            return x + self.down(torch.nn.functional.gelu(self.up(x)))

    torch.manual_seed(0)
    m = Block().to(cuda).to(torch.bfloat16).eval()
    x = torch.randn(2, 384, 256, device=cuda, dtype=torch.bfloat16)
    with torch.no_grad():
        want = m(x)
    ind.enable()
    try:
        torch._dynamo.reset()
        before = dict(ind.calls)
        try:
            compiled = torch.compile(m)
            with torch.no_grad():
                got = compiled(x)
        except Exception as e:  # no working Inductor tool chain on this box
            pytest.skip(f"torch.compile unavailable here: {type(e).__name__}")
    finally:
        ind.disable()
        torch._dynamo.reset()
    assert ind.calls["mm"] - before["mm"] >= 3
    torch.testing.assert_close(got.float(), want.float(), rtol=3e-2, atol=3e-2)
    _lib.sync_check(cuda)


@pytest.mark.gpu
def test_operators_have_gradients(cuda):
    from triton_b200 import inductor as ind  # noqa: F401  (registers the operators)
    g = torch.Generator(device=cuda).manual_seed(3)
    a = (torch.randn(256, 128, device=cuda, generator=g) * 0.1).to(torch.bfloat16).requires_grad_()
    b = (torch.randn(128, 192, device=cuda, generator=g) * 0.1).to(torch.bfloat16).requires_grad_()
    c = torch.ops.triton_b200.mm(a, b)
    c.float().square().sum().backward()
    a2, b2 = a.detach().float().requires_grad_(), b.detach().float().requires_grad_()
    (a2 @ b2).square().sum().backward()
    torch.testing.assert_close(a.grad.float(), a2.grad, rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(b.grad.float(), b2.grad, rtol=3e-2, atol=3e-2)
    q, k, v = ((torch.randn(1, 2, 256, 128, device=cuda, generator=g) * 0.5).to(torch.bfloat16).requires_grad_() for _ in range(3))
    o, _ = torch.ops.triton_b200.attention(q, k, v, 128 ** -0.5, True)
    o.float().sum().backward()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, is_causal=True).sum().backward()
    for got, want in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        torch.testing.assert_close(got.float(), want, rtol=3e-2, atol=3e-2)
