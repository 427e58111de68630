"""``torch.compile`` hook-up — counterpart of ``third_party/tlx/language/tlx/inductor/`` in the reference
(``registry.py``: shape heuristics and the patches that make Inductor consider the TLX kernels;
``mm_templates.py`` / ``flex_attention_templates.py``: the GEMM and attention templates and their choice
injection ``append_tlx`` / ``append_tlx_flex``).

The reference injects jinja templates of its kernels into Inductor's autotuned choices. The kernels of this
library are precompiled, so the hook-up has two parts:

1. Custom operators (``torch.library``): ``triton_b200::mm`` and ``triton_b200::attention``, each with a fake
   (meta) implementation and autograd, so that Dynamo and AOTAutograd trace through them and Inductor calls
   them as extern kernels (the role the template objects play in the reference).
2. ``enable()`` installs a post-grad graph pass in Inductor (the role of ``append_tlx``): ``aten.mm`` nodes on
   2-D bf16 / fp16 CUDA operands that satisfy the kernel's alignment rules become ``triton_b200::mm``, and
   inference-time flash-attention nodes (``aten._scaled_dot_product_flash_attention`` whose only used result is
   the output) with head dim 64 or 128 become ``triton_b200::attention``. ``use_for_mm(M, N, K)`` is the shape
   rule that decides, as ``get_heuristic_config`` / the choice filter do in the reference. ``disable()`` removes
   the pass.

Nothing here runs a kernel on the CPU: the operators raise on non-CUDA tensors, as every entry point of the
library does.
"""
from __future__ import annotations

import torch

_LIB = "triton_b200"
calls = {"mm": 0, "attention": 0}  # how often the operators ran (tests use it to see that a graph was rewritten)


# ------------------------------------------------------------------------------------------ operators


@torch.library.custom_op(f"{_LIB}::mm", mutates_args=())
def mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b`` for 2-D bf16 / fp16 operands (each contiguous or the transpose of a contiguous matrix)."""
    from .tutorials.blackwell_gemm_ws import matmul
    calls["mm"] += 1
    return matmul(a, b)


@mm.register_fake
def _mm_fake(a, b):
    return a.new_empty((a.shape[0], b.shape[1]))


def _mm_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _mm_backward(ctx, grad):
    a, b = ctx.saved_tensors
    grad = grad.contiguous()
    return mm(grad, b.t()), mm(a.t(), grad)


mm.register_autograd(_mm_backward, setup_context=_mm_setup)


@torch.library.custom_op(f"{_LIB}::attention", mutates_args=())
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sm_scale: float,
              causal: bool) -> tuple[torch.Tensor, torch.Tensor]:
    """Flash-attention forward: (o, base-2 log-sum-exp). q, k, v ``[B, H, S, D]`` bf16 / fp16."""
    from .tutorials.blackwell_fa_ws_pipelined_persistent import attention_with_lse
    calls["attention"] += 1
    return attention_with_lse(q.contiguous(), k.contiguous(), v.contiguous(), sm_scale, causal)


@attention.register_fake
def _attention_fake(q, k, v, sm_scale, causal):
    return torch.empty_like(q, memory_format=torch.contiguous_format), q.new_empty(q.shape[:3], dtype=torch.float32)


@torch.library.custom_op(f"{_LIB}::attention_bwd", mutates_args=())
def attention_bwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                  d_o: torch.Tensor, sm_scale: float, causal: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    from .tutorials.blackwell_fa_ws_pipelined_persistent import attention_backward
    return attention_backward(q, k, v, o, lse, d_o.contiguous(), sm_scale, causal)


@attention_bwd.register_fake
def _attention_bwd_fake(q, k, v, o, lse, d_o, sm_scale, causal):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _attention_setup(ctx, inputs, output):
    q, k, v, sm_scale, causal = inputs
    o, lse = output
    ctx.save_for_backward(q, k, v, o, lse)
    ctx.sm_scale, ctx.causal = sm_scale, causal


def _attention_backward(ctx, d_o, d_lse):
    q, k, v, o, lse = ctx.saved_tensors
    dq, dk, dv = attention_bwd(q, k, v, o, lse, d_o, ctx.sm_scale, ctx.causal)
    return dq, dk, dv, None, None


attention.register_autograd(_attention_backward, setup_context=_attention_setup)


# ------------------------------------------------------------------------------------------ the choice


def use_for_mm(M: int, N: int, K: int) -> bool:
    """Shape rule of the rewrite: every GEMM the kernel accepts except the ones too small to fill a tile row
    (left to the library kernel Inductor would pick itself)."""
    return M >= 1 and N >= 8 and K >= 16 and M * N * K >= 128 * 128 * 64


def _static(shape):
    return all(isinstance(d, int) for d in shape)


def _operand_ok(t) -> bool:
    """A 2-D operand the GEMM kernel reads in place: contiguous or transposed-contiguous, 16-byte aligned pitch."""
    if t.dim() != 2 or not _static(t.shape) or not _static(t.stride()):
        return False
    r, c = t.shape
    esz = t.element_size()
    if t.stride(1) == 1 and t.stride(0) >= c:
        return (t.stride(0) * esz) % 16 == 0
    if t.stride(0) == 1 and t.stride(1) >= r:
        return (t.stride(1) * esz) % 16 == 0
    return False


def _mm_eligible(a, b) -> bool:
    if a is None or b is None or not isinstance(a, torch.Tensor) or not isinstance(b, torch.Tensor):
        return False
    if a.device.type != "cuda" or a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        return False
    if not (_operand_ok(a) and _operand_ok(b)):
        return False
    return use_for_mm(a.shape[0], b.shape[1], a.shape[1])


def rewrite_graph(graph: torch.fx.Graph) -> int:
    """Rewrites eligible nodes of a post-grad (ATen-level) FX graph in place; returns how many were rewritten."""
    aten = torch.ops.aten
    n = 0
    for node in list(graph.nodes):
        if node.op != "call_function":
            continue
        if node.target is aten.mm.default:
            a, b = node.args
            if _mm_eligible(a.meta.get("val"), b.meta.get("val")):
                node.target = torch.ops.triton_b200.mm.default
                n += 1
        elif node.target is aten._scaled_dot_product_flash_attention.default:
            q, k, v = node.args[:3]
            qv = q.meta.get("val")
            kw = dict(node.kwargs)
            dropout = node.args[3] if len(node.args) > 3 else kw.get("dropout_p", 0.0)
            causal = node.args[4] if len(node.args) > 4 else kw.get("is_causal", False)
            scale = kw.get("scale", None)
            users = list(node.users)
            # results other than the output may be picked out of the tuple as long as nothing reads them
            only_out = all(u.op == "call_function" and getattr(u.target, "__name__", "") == "getitem"
                           and (u.args[1] == 0 or len(u.users) == 0) for u in users)
            if (qv is None or qv.dim() != 4 or qv.device.type != "cuda" or qv.dtype not in (torch.bfloat16, torch.float16)
                    or qv.shape[-1] not in (64, 128) or dropout != 0.0 or not only_out or not _static(qv.shape)):
                continue
            kv = k.meta.get("val")
            if causal and kv is not None and kv.shape[2] != qv.shape[2]:
                continue
            sm_scale = float(scale) if scale is not None else float(qv.shape[-1]) ** -0.5
            with graph.inserting_before(node):
                new = graph.call_function(torch.ops.triton_b200.attention.default, (q, k, v, sm_scale, bool(causal)))
            new.meta["val"] = (node.meta["val"][0], node.meta["val"][1]) if "val" in node.meta else None
            for u in users:
                if u.args[1] == 0:
                    u.replace_input_with(node, new)
                else:
                    graph.erase_node(u)
            graph.erase_node(node)
            n += 1
    return n


try:
    from torch._inductor.custom_graph_pass import CustomGraphPass

    class _Pass(CustomGraphPass):
        def __call__(self, graph: torch.fx.Graph) -> None:
            rewrite_graph(graph)

        def uuid(self):
            return "triton_b200.inductor.rewrite.v1"
except Exception:  # an Inductor without CustomGraphPass: a plain callable (the FX graph cache is then bypassed)
    class _Pass:  # type: ignore[no-redef]
        def __call__(self, graph):
            rewrite_graph(graph)


_previous = None
_enabled = False


def enable() -> None:
    """Makes ``torch.compile`` (Inductor) use this library's GEMM and attention for eligible nodes."""
    global _previous, _enabled
    import torch._inductor.config as cfg
    if _enabled:
        return
    _previous = cfg.post_grad_custom_post_pass
    prev = _previous

    class _Chained(_Pass):
        def __call__(self, graph):
            if prev is not None:
                prev(graph)
            rewrite_graph(graph)

    cfg.post_grad_custom_post_pass = _Chained()
    _enabled = True


def disable() -> None:
    global _previous, _enabled
    import torch._inductor.config as cfg
    if _enabled:
        cfg.post_grad_custom_post_pass = _previous
        _previous, _enabled = None, False
