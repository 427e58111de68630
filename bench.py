#!/usr/bin/env python
"""Benchmark driver.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--no-configs]

Headline workload (the configuration the metric is quoted on): the bf16 persistent warp-specialised GEMM,
M=N=K=8192, A row-major, B supplied K-major, entries N(0,1)/sqrt(K) from seed 1, fp32 accumulation, bf16
output. One "step" is one GEMM over resident inputs. With N GPUs every rank owns one 8192-column block of a
K x (8192*N) B (no collective on the data path; weak scaling) and the reported value is the whole job's
TFLOP/s with the time taken as the max over ranks.

One JSON line is printed by rank 0. Keys beyond the base contract:
  roofline      tensor-pipe roofline of the GEMM kernel: achieved = 2MNK / mean CUDA-event duration of the
                launches in the timed region, peak = measured cuBLAS bf16 figure from MEASURED_PEAKS.json (burst
                when the timed region is shorter than 0.5 s, else sustained), traffic = DRAM bytes per launch
                from an ncu capture of the same kernel, or null.
  e2e           same metric through the public Python entry point with HOST (pinned) inputs and a host result:
                H2D copies of A and B and the D2H copy of C are inside the timed region.
  cpu_baseline  the CPU oracle (torch CPU fp32 matmul, all host threads) timed on a bounded sample.
  sustained     at least 2 s of back-to-back headline GEMMs with the clock sampler running.
  clocks        SM clock / throttle reasons sampled through NVML during the timed region.
  configs       every other configuration of the metric, measured in the same run (a few steps each): the
                attention, FP8 / MXFP8, MoE, skinny and sweep workloads as per-GPU replicas, plus the two sharded
                ones - `gemm_strong` (the one 8192^3 problem split into N column blocks) and `moe_ep` (the
                16384-token MoE layer with experts and tokens sharded over the N GPUs, token exchange inside the
                timed region, parity-checked against the CPU oracle on the live ranks before it is timed). Each
                entry: tflops, ms, roofline, e2e (host buffers) and, at N = 1, a cpu_baseline on a stated
                down-scaled sample.

`--workload NAME` measures one of those workloads alone (more steps; what the ncu summaries were taken from).
`--impl reference` times the reference's CPU path for the headline workload (the oracle port: the reference's own
kernels need a GPU and its compiler, which cannot be built offline) with all host threads.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M = N = K = 8192
WORKLOAD = "bf16 GEMM M=N=K=8192, A row-major, B K-major (transposed), N(0,1)/sqrt(K) seed 1, fp32 acc, bf16 out"
CONFIG = {"workload": WORKLOAD, "sharding": "one 8192-column block of B per GPU, no collective",
          "l2": "inputs (256 MiB) and output (128 MiB) exceed the 126 MB L2; no flush"}

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of each workload's dominant kernel, from
# ncu captures of `python bench.py --workload NAME`; None where no capture of the current kernel exists.
NCU_TRAFFIC = {
    "gemm": 1.037e9,
    "gemm_skinny": 0.140e9,  # the kernel with the split-K partial sums reduced inside a cluster
    "attn": 16.04e9,         # the tile order re-reads K / V for every query tile; kernel unchanged since the capture
    "attn_causal": 8.16e9,
    "fp8": 0.509e9,
    "fp8_blockwise": 0.587e9,
    "mxfp8": 0.565e9,
}

L2_BYTES = 126e6


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_burst": float(p["bf16_tflops"]), "bf16_sustained": float(p["bf16_tflops_sustained"]),
                "hbm": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_burst": 1590.0, "bf16_sustained": 1400.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """Polls NVML for SM clock and throttle reasons while the timed region runs (read-only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def sample(self):
        if not self.nv:
            return
        try:
            nv = self.nv
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(
                nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                     0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}
            for bit, name in names.items():
                if r & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self.sample()
            time.sleep(0.005)

    def start(self):
        if self.nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr:
            self._thr.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------ workloads


class Workload:
    """One measurable configuration: `step()` runs it on resident device inputs; `inputs` are the device tensors
    a step reads (the e2e leg refills them from pinned host copies every step); `cpu()` times the CPU oracle on a
    down-scaled sample and returns (TFLOP/s, description)."""

    def __init__(self, step, flops, hbm_bytes, desc, kernel, bound, inputs, dtype="bf16", launches=1, cpu=None,
                 sharded=False, peak="bf16", footprint=None, parity=None):
        self.step, self.flops, self.hbm_bytes, self.desc, self.kernel, self.bound = step, flops, hbm_bytes, desc, kernel, bound
        self.inputs, self.dtype, self.launches, self.cpu, self.sharded, self.peak = inputs, dtype, launches, cpu, sharded, peak
        self.footprint = footprint if footprint is not None else sum(t.numel() * t.element_size() for t in inputs)
        self.parity = parity


def _cpu_time(fn, flops, what):
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
    fn()  # warm the thread pool
    t0 = time.perf_counter()
    fn()
    dt = time.perf_counter() - t0
    return flops / dt / 1e12, what


def cpu_gemm(s=2048):
    import torch
    from oracle import gemm as o_gemm
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(s, s, generator=g) / s ** 0.5).to(torch.bfloat16)
    w = (torch.randn(s, s, generator=g) / s ** 0.5).to(torch.bfloat16)
    return _cpu_time(lambda: o_gemm.gemm_ref(a, w.t()), 2.0 * s ** 3,
                     f"torch CPU fp32 matmul of bf16 inputs, M=N=K={s} (down-scaled), all host threads")


def cpu_attn(causal):
    import torch
    from oracle import attention as o_attn
    B, H, S, D = 1, 4, 1024, 128
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16) for _ in range(3))
    fl = 4.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S)
    return _cpu_time(lambda: o_attn.attention_ref(q, k, v, D ** -0.5, causal), fl,
                     f"fp32 softmax(QK^T)V on CPU, [B={B},H={H},S={S},D={D}] (down-scaled), causal={causal}, all host threads")


def cpu_mxfp8(s=1024):
    import torch
    from oracle import mxfp8 as o_mx
    g = torch.Generator().manual_seed(3)
    qa, sa = o_mx.make_mxfp8_operand(s, s, g)
    qb, sb = o_mx.make_mxfp8_operand(s, s, g)
    return _cpu_time(lambda: o_mx.mxfp8_gemm_ref(qa, qb, sa, sb), 2.0 * s ** 3,
                     f"dequantise + fp32 matmul on CPU, M=N=K={s} (down-scaled), all host threads")


def cpu_fp8(s=2048):
    import torch
    from oracle import gemm as o_gemm
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(s, s, generator=g) * 0.1).to(torch.float8_e4m3fn)
    b = (torch.randn(s, s, generator=g) * 0.1).to(torch.float8_e4m3fn)
    one = torch.ones(1)
    return _cpu_time(lambda: o_gemm.scaled_mm_tensorwise_ref(a, b, one, one), 2.0 * s ** 3,
                     f"fp32 matmul of e4m3 inputs on CPU, M=N=K={s} (down-scaled), all host threads")


def cpu_moe():
    import torch
    from oracle import moe as o_moe
    T, D, F, E, k = 512, 1024, 384, 16, 4
    g = torch.Generator().manual_seed(4)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, generator=g)
    w1 = (0.02 * torch.randn(E, D, 2 * F, generator=g)).to(torch.bfloat16)
    w2 = (0.02 * torch.randn(E, F, D, generator=g)).to(torch.bfloat16)
    fl = 2.0 * T * k * D * 2 * F + 2.0 * T * k * F * D
    return _cpu_time(lambda: o_moe.moe_layer_ref(x, logits, w1, w2, k), fl,
                     f"CPU oracle MoE layer, {T} tokens, d_model {D}, E={E}, top-{k}, W1 [{D},{2*F}] W2 [{F},{D}] "
                     "(down-scaled), all host threads")


def _dev_randn(shape, dev, seed, scale=1.0, dtype=None):
    import torch
    g = torch.Generator(device=dev).manual_seed(seed)
    t = torch.randn(shape, generator=g, device=dev)
    if scale != 1.0:
        t *= scale
    return t.to(dtype) if dtype is not None else t


def build_workload(name: str, rank: int, world: int, dev):
    """Builds one workload on `dev`. Inputs are drawn on the device from seeded generators (the configs'
    distributions; seeds offset per rank) so that set-up costs seconds, not minutes."""
    import torch
    bf = torch.bfloat16
    if name in ("attn_mxfp8", "attn_mxfp8_causal"):
        from triton_b200.triton_kernels.numerics_details.mxfp import downcast_to_mxfp
        from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent_mxfp8 import attention as mx_attention
        from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent_mxfp8 import swizzle_block_scales
        causal = name.endswith("causal")
        B, H, S, D = 4, 32, 8192, 128
        ops = []
        for i in range(3):  # N(0,1) bf16 tensors quantised to MXFP8: Q, K along D; V (transposed) along the sequence
            x = _dev_randn((B * H * S, D), dev, 2 + 1000 * rank + i, dtype=bf)
            val, s8 = downcast_to_mxfp(x if i < 2 else x.t().contiguous(), torch.float8_e4m3fn, axis=1)
            ops.append((val if i < 2 else val.t()).reshape(B, H, S, D).contiguous())
            ops.append(swizzle_block_scales(s8))
            del x, val, s8
        q, qs, k, ks, v, vs = ops
        sc = 1.0 / math.sqrt(D)
        fl = 4.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S)
        return Workload(lambda: mx_attention(q, k, v, qs, ks, vs, sc, causal), fl, 3.0 * B * H * S * D + 2.0 * B * H * S * D,
                        f"MXFP8 flash-attention fwd [B={B},H={H},S={S},D={D}] causal={causal}, N(0,1) quantised per 32, seed 2",
                        "attention_mxfp8_fwd_kernel", "tensor", [q, k, v], dtype="e4m3", peak="fp8")
    if name.startswith("attn") and "bwd" not in name:
        from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_with_lse
        causal = name.endswith("causal")
        B, H, S, D = (32, 32, 1024, 128) if "short" in name else (4, 32, 8192, 128)
        if "d256" in name:  # head dim 256 with the same flop count: half the heads
            H, D = H // 2, 256
        q, k, v = (_dev_randn((B, H, S, D), dev, 2 + 1000 * rank + i, dtype=bf) for i in range(3))
        sc = 1.0 / math.sqrt(D)
        fl = 4.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S)
        return Workload(lambda: attention_with_lse(q, k, v, sc, causal)[0], fl, 4.0 * B * H * S * D * 2,
                        f"flash-attention fwd bf16 [B={B},H={H},S={S},D={D}] causal={causal}, seed 2",
                        f"attention_fwd_kernel<{D}>", "tensor", [q, k, v],
                        cpu=None if D == 256 else (lambda: cpu_attn(causal)))
    if name in ("attn_bwd", "attn_bwd_causal", "attn_bwd_ref_shape", "attn_bwd_ref_shape_causal"):
        from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_backward, attention_with_lse
        causal = name.endswith("causal")
        # "ref_shape": Z=4, H=16, N=2048, the first shape of the reference's published backward table
        B, H, S, D = (4, 16, 2048, 128) if "ref_shape" in name else (4, 32, 8192, 128)
        q, k, v, do = (_dev_randn((B, H, S, D), dev, 2 + 1000 * rank + i, dtype=bf) for i in range(4))
        sc = 1.0 / math.sqrt(D)
        o, lse = attention_with_lse(q, k, v, sc, causal)
        fl = 10.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S)  # five S x S x D products
        return Workload(lambda: attention_backward(q, k, v, o, lse, do, sc, causal)[0], fl, 8.0 * B * H * S * D * 2,
                        f"flash-attention bwd bf16 [B={B},H={H},S={S},D={D}] causal={causal} (delta + main + dq kernels), seed 2",
                        "attention_bwd_kernel", "tensor", [q, k, v, do], launches=3)
    if name == "gemm_skinny":
        from triton_b200.tutorials.blackwell_gemm_ws import matmul
        m, n = 128, 8192
        a = _dev_randn((m, n), dev, 1 + 1000 * rank, n ** -0.5, bf)
        ws = [_dev_randn((n, n), dev, 10 + 1000 * rank + i, n ** -0.5, bf) for i in range(4)]
        turn = [0]

        def step():  # four weight matrices in turn: 512 MiB, so none of them stays in the 126 MB L2
            turn[0] = (turn[0] + 1) & 3
            return matmul(a, ws[turn[0]].t())
        return Workload(step, 2.0 * m * n * n, 2.0 * (n * n + m * n + m * n),
                        "bf16 GEMM M=128, N=K=8192 (the skinny case), B K-major, four weight matrices in turn",
                        "gemm_kernel (K split in a cluster)", "hbm", [a], launches=1, cpu=cpu_gemm, footprint=4 * n * n * 2)
    if name.startswith("gemm_") and name[5:].isdigit():
        from triton_b200.tutorials.blackwell_gemm_ws import matmul
        s = int(name[5:])
        a = _dev_randn((s, s), dev, 1 + 1000 * rank, s ** -0.5, bf)
        w = _dev_randn((s, s), dev, 2 + 1000 * rank, s ** -0.5, bf)
        return Workload(lambda: matmul(a, w.t()), 2.0 * s ** 3, 6.0 * s * s,
                        f"bf16 GEMM M=N=K={s} (sweep point of config 2), B K-major, seed 1", "gemm_kernel", "tensor",
                        [a, w], cpu=cpu_gemm, footprint=6 * s * s)
    if name == "gemm_strong":
        from triton_b200.tutorials.blackwell_gemm_ws import matmul
        n_loc = N // world
        a = _dev_randn((M, K), dev, 1, K ** -0.5, bf)                     # A replicated (same seed on every rank)
        w = _dev_randn((n_loc, K), dev, 100 + rank, K ** -0.5, bf)       # this rank's column block of B
        return Workload(lambda: matmul(a, w.t()), 2.0 * M * n_loc * K, 2.0 * (M * K + n_loc * K + M * n_loc),
                        f"the one bf16 8192^3 GEMM split into {world} column block(s) of {n_loc} columns, A replicated, "
                        "no collective; strong scaling", "gemm_kernel", "tensor", [a, w], cpu=cpu_gemm, sharded=True)
    if name in ("fp8", "fp8_blockwise", "mxfp8"):
        n = 8192
        a = _dev_randn((n, n), dev, 3 + 1000 * rank, 0.1).to(torch.float8_e4m3fn)
        b = _dev_randn((n, n), dev, 4 + 1000 * rank, 0.1).to(torch.float8_e4m3fn)
        g = torch.Generator(device="cpu").manual_seed(3 + 1000 * rank)
        if name == "fp8":
            from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
            sa, sb = torch.rand(1, generator=g).to(dev), torch.rand(1, generator=g).to(dev)
            return Workload(lambda: blackwell_scaled_mm_ws(a, b, sa, sb, scale_mode="tensorwise"), 2.0 * n ** 3, 4.0 * n * n,
                            "per-tensor-scaled e4m3 GEMM 8192^3, bf16 out", "gemm_kernel<256,4,pair,f8>", "tensor",
                            [a, b], dtype="e4m3", cpu=cpu_fp8, peak="fp8")
        if name == "fp8_blockwise":
            from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
            sa = torch.rand(n, n // 128, generator=g).t().contiguous().t().to(dev)
            sb = torch.rand(n // 128, n // 128, generator=g).to(dev)
            return Workload(lambda: blackwell_scaled_mm_ws(a, b, sa, sb, scale_mode="blockwise"), 2.0 * n ** 3, 4.0 * n * n,
                            "blockwise-scaled (128-wide K groups) e4m3 GEMM 8192^3, bf16 out", "gemm_fp8_blockwise_kernel",
                            "tensor", [a, b], dtype="e4m3", cpu=cpu_fp8, peak="fp8")
        from triton_b200.tutorials.blackwell_gemm_ws_mxfp8 import matmul as mx_matmul
        u = torch.randint(-4, 5, (n * n // 32, ), generator=g)
        sc = (u + 127).to(torch.uint8).to(dev).view(torch.float8_e8m0fnu)
        return Workload(lambda: mx_matmul(a, b, sc, sc), 2.0 * n ** 3, 4.0 * n * n + 2 * n * n / 32,
                        "MXFP8 block-scaled GEMM 8192^3 (e8m0 scales 2^u, u in [-4,4]), bf16 out", "gemm_mxfp8_kernel",
                        "tensor", [a, b], dtype="e4m3", cpu=cpu_mxfp8, peak="fp8")
    if name in ("moe", "moe_decode", "moe_small"):
        from triton_b200.triton_kernels.matmul import matmul as moe_matmul, swiglu_activation
        from triton_b200.triton_kernels.reduce import reduce
        from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
        from triton_b200.triton_kernels.topk import topk
        T, D, F, E, k = (64 if name == "moe_decode" else 16384), 4096, 1536, 128, 4
        if name == "moe_small":  # the layer down-scaled to 16 experts (the same rows per expert): the case profiled under ncu
            T, E = 2048, 16
        x = _dev_randn((T, D), dev, 4 + 1000 * rank, dtype=bf)
        logits = _dev_randn((T, E), dev, 5 + 1000 * rank)
        w1 = _dev_randn((E, D, 2 * F), dev, 6 + 1000 * rank, 0.02, bf)
        w2 = _dev_randn((E, F, D), dev, 7 + 1000 * rank, 0.02, bf)
        act = swiglu_activation(1.0, None)
        y = torch.empty(T * k, D, dtype=bf, device=dev)

        def step():
            sm = topk(logits, k)
            mm = sm.mask_metadata
            rg = make_ragged_tensor_metadata(mm.col_sum, T * k)
            combine = mm.col_sorted_indx
            gather = torch.div(combine, k, rounding_mode="trunc")
            gam = sm.vals.float().reshape(-1)[combine.long()]
            h = moe_matmul(x, w1, None, rg, gather_indx=gather, fused_activation=act)
            moe_matmul(h, w2, None, rg, scatter_indx=combine, gammas=gam, c=y)
            return reduce(y.view(T, k, D), dim=1)[0]
        R = T * k
        fl = 2.0 * R * D * 2 * F + 2.0 * R * F * D
        active = int((topk(logits, k).mask_metadata.col_sum > 0).sum().item())  # experts that get any row
        by = active * (D * 2 * F + F * D) * 2.0 + R * (D + F) * 2.0 + R * (F + D) * 2.0
        return Workload(step, fl, by, f"MoE layer: {T} tokens, d_model {D}, E={E}, top-{k}, W1 [{D},{2*F}] SwiGLU W2 "
                        f"[{F},{D}], gate-weighted combine, seed 4", "moe_gemm_kernel",
                        "hbm" if name == "moe_decode" else "tensor", [x, logits], launches=9, cpu=cpu_moe,
                        footprint=(w1.numel() + w2.numel()) * 2)
    if name in ("moe_mx4", "moe_mx4_decode", "moe_bf16_mx4", "moe_fp8"):
        from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul as moe_matmul, swiglu_activation
        from triton_b200.triton_kernels.numerics_details.mxfp import downcast_to_mxfp
        from triton_b200.triton_kernels.reduce import reduce
        from triton_b200.triton_kernels.tensor import FP4, convert_layout, make_ragged_tensor_metadata, wrap_torch_tensor
        from triton_b200.triton_kernels.tensor_details.layout import (make_default_matmul_mxfp4_w_layout,
                                                                      make_default_matmul_mxfp4_w_scale_layout)
        from triton_b200.triton_kernels.topk import topk
        T = 64 if name == "moe_mx4_decode" else 16384
        D, F, E, k = 4096, 1536, 128, 4
        x = _dev_randn((T, D), dev, 4 + 1000 * rank)
        x = x.to(bf) if name == "moe_bf16_mx4" else x.to(torch.float8_e4m3fn)
        logits = _dev_randn((T, E), dev, 5 + 1000 * rank)

        def prep(w):
            v, s = downcast_to_mxfp(w, torch.uint8, axis=1)
            return (convert_layout(wrap_torch_tensor(v, dtype=FP4), make_default_matmul_mxfp4_w_layout(mx_axis=1)),
                    convert_layout(wrap_torch_tensor(s), make_default_matmul_mxfp4_w_scale_layout(mx_axis=1)))
        if name == "moe_fp8":  # plain fp8 weights, K contiguous (how the reference stores 8-bit weights)
            def prep(w):
                return w.to(torch.float8_e4m3fn).transpose(1, 2).contiguous().transpose(1, 2), None
        w1, s1 = prep(_dev_randn((E, D, 2 * F), dev, 6 + 1000 * rank, 0.02, bf))
        w2, s2 = prep(_dev_randn((E, F, D), dev, 7 + 1000 * rank, 0.02, bf))
        bf16_act = name == "moe_bf16_mx4"
        # fp8 activations: GEMM 1 writes fp8 (the default: the activations' dtype), GEMM 2 bf16 for the combine
        pc1 = PrecisionConfig(b_mx_scale=s1)
        pc2 = PrecisionConfig(b_mx_scale=s2) if bf16_act else PrecisionConfig(b_mx_scale=s2, out_dtype=bf)
        act = swiglu_activation(1.0, None)

        def step():
            sm = topk(logits, k)
            mm = sm.mask_metadata
            rg = make_ragged_tensor_metadata(mm.col_sum, T * k)
            combine = mm.col_sorted_indx
            gather = torch.div(combine, k, rounding_mode="trunc")
            gam = sm.vals.float().reshape(-1)[combine.long()]
            h = moe_matmul(x, w1, None, rg, gather_indx=gather, precision_config=pc1, fused_activation=act)
            y = moe_matmul(h, w2, None, rg, scatter_indx=combine, gammas=gam, precision_config=pc2)
            return reduce(y.view(T, k, D), dim=1)[0]
        R = T * k
        fl = 2.0 * R * D * 2 * F + 2.0 * R * F * D
        if bf16_act:
            return Workload(step, fl, 0.0, "MoE layer, bf16 activations x MXFP4 weights (upcast pass + 16-bit grouped "
                            f"GEMM per call): {T} tokens, d_model {D}, E={E}, top-{k}, seed 4", "moe_gemm_kernel",
                            "tensor", [x, logits], launches=11)
        active = int((topk(logits, k).mask_metadata.col_sum > 0).sum().item())
        if name == "moe_fp8":
            by = active * (D * 2 * F + F * D) * 1.0 + R * (D + F) * 1.0 + R * (F * 1.0 + D * 2.0)
            return Workload(step, fl, by, f"MoE layer, fp8 activations x fp8 weights: {T} tokens, d_model {D}, E={E}, "
                            f"top-{k}, W1 [{D},{2*F}] SwiGLU W2 [{F},{D}], gate-weighted combine, seed 4",
                            "moe_gemm_mx4_kernel", "tensor", [x, logits], dtype="e4m3", launches=9, peak="fp8",
                            footprint=E * (D * 2 * F + F * D))
        by = active * (D * 2 * F + F * D) * (0.5 + 1.0 / 32) + R * (D + F) * 1.0 + R * (F * 1.0 + D * 2.0)
        return Workload(step, fl, by, f"MoE layer, fp8 activations x MXFP4 weights: {T} tokens, d_model {D}, E={E}, "
                        f"top-{k}, W1 [{D},{2*F}] SwiGLU W2 [{F},{D}], gate-weighted combine, seed 4",
                        "moe_gemm_mx4_kernel", "hbm" if name == "moe_mx4_decode" else "tensor", [x, logits], dtype="e4m3",
                        launches=9, peak="fp8", footprint=int(E * (D * 2 * F + F * D) * (0.5 + 1.0 / 32)))
    if name == "mxfp4_upcast":
        from triton_b200.triton_kernels.matmul import upcast_mxfp4_weight
        from triton_b200.triton_kernels.tensor import FP4, convert_layout, wrap_torch_tensor
        from triton_b200.triton_kernels.tensor_details.layout import (make_default_matmul_mxfp4_w_layout,
                                                                      make_default_matmul_mxfp4_w_scale_layout)
        E, Kd, Nd = 128, 4096, 3072
        g = torch.Generator(device=dev).manual_seed(4 + 1000 * rank)
        v = torch.randint(0, 256, (E, Kd // 2, Nd), generator=g, dtype=torch.uint8, device=dev)
        s = torch.randint(118, 130, (E, Kd // 32, Nd), generator=g, dtype=torch.uint8, device=dev)
        wv = convert_layout(wrap_torch_tensor(v, dtype=FP4), make_default_matmul_mxfp4_w_layout(mx_axis=1))
        ws = convert_layout(wrap_torch_tensor(s), make_default_matmul_mxfp4_w_scale_layout(mx_axis=1))
        del v, s
        by = E * Kd * Nd * (0.5 + 1.0 / 32 + 2.0)
        return Workload(lambda: upcast_mxfp4_weight(wv, ws, bf), 0.0, by,
                        f"MXFP4 -> bf16 weight upcast: E={E} matrices [{Kd},{Nd}] (W1 of the MoE layer), random codes, seed 4",
                        "mxfp4_upcast_kernel", "hbm", [wv.data])
    if name in ("moe_ep", "moe_ep_eager", "moe_ep_nccl", "moe_ep_unfused"):
        return build_moe_ep(name, rank, world, dev)
    raise SystemExit(f"unknown workload {name}")


def build_moe_ep(name, rank, world, dev):
    """The 16384-token MoE layer (config 5) with tokens and experts sharded over the ranks: strong scaling. The
    exchange (top-k all-gather, dispatch, combine) is inside every step. `moe_ep`: peer stores with the combine
    fused into GEMM-2's epilogue, the whole layer replayed as one CUDA graph; `moe_ep_eager`: the same, launched
    call by call; `moe_ep_unfused`: peer stores by separate dispatch / combine kernels; `moe_ep_nccl`: NCCL
    all-to-all. Before anything is timed a small layer is run on the live ranks and each rank's slice is compared
    with the CPU oracle."""
    import torch
    import torch.distributed as dist
    from triton_b200.triton_kernels.distributed import (EpGroup, EpLayerGraph, Mesh, SymmetricMemoryPool,
                                                        make_expt_assignment, make_expt_dict_uniform, moe_layer_ep)
    bf = torch.bfloat16
    T, D, F, E, k = 16384, 4096, 1536, 128, 4
    tl, per = T // world, E // world
    fuse = name in ("moe_ep", "moe_ep_eager")
    ea = make_expt_assignment(world, E, make_expt_dict_uniform(world, E), dev)
    if name == "moe_ep_nccl":
        ep = EpGroup()
    else:
        ep = SymmetricMemoryPool(Mesh())
        ep.initialize_matmul(T, D, D, k, E, bf, dev)

    # ---- parity on the live ranks: a small layer through the same transport against the CPU oracle
    from oracle import moe as o_moe
    pT, pD, pF = 64 * world, 256, 128
    g = torch.Generator().manual_seed(4)
    px = torch.randn(pT, pD, generator=g).to(bf)
    pl = torch.randn(pT, E, generator=g)
    pw1 = (0.05 * torch.randn(E, pD, 2 * pF, generator=g)).to(bf)
    pw2 = (0.05 * torch.randn(E, pF, pD, generator=g)).to(bf)
    ptl = pT // world
    sl, es = slice(rank * ptl, (rank + 1) * ptl), slice(rank * per, (rank + 1) * per)
    z = moe_layer_ep(px[sl].to(dev), pl[sl].to(dev), pw1[es].to(dev), pw2[es].to(dev), k, ea, ep, fuse_combine=fuse)
    ref = o_moe.moe_layer_ref(px, pl, pw1, pw2, k)[sl].float()
    err = float((z.cpu().float() - ref).abs().max())
    if world > 1:
        t = torch.tensor([err], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err = float(t.item())
    if not err <= 2e-2:
        raise SystemExit(f"{name}: parity check against the CPU oracle failed on the live ranks (max abs err {err})")
    if world > 1:
        dist.barrier()  # the CPU oracle above takes a different time on every rank: meet on the host before the next layer call
    parity = {"checked": True, "max_abs_err": err, "tolerance": 2e-2,
              "case": f"{pT} tokens, d_model {pD}, E={E}, top-{k} through the same transport, each rank's slice vs the CPU oracle"}

    x = _dev_randn((tl, D), dev, 4 + 1000 * rank, dtype=bf)
    logits = _dev_randn((tl, E), dev, 5 + 1000 * rank)
    w1 = _dev_randn((per, D, 2 * F), dev, 6 + 1000 * rank, 0.02, bf)
    w2 = _dev_randn((per, F, D), dev, 7 + 1000 * rank, 0.02, bf)
    R = T * k
    fl = (2.0 * R * D * 2 * F + 2.0 * R * F * D) / world  # per rank; the line reports world * this
    how = {"moe_ep": "peer stores over NVLink, combine fused into GEMM-2's epilogue, one CUDA graph per layer call",
           "moe_ep_eager": "peer stores over NVLink, combine fused into GEMM-2's epilogue, launched call by call",
           "moe_ep_unfused": "peer stores over NVLink by dispatch / combine kernels",
           "moe_ep_nccl": "NCCL all_to_all_single dispatch / combine"}[name]
    step = lambda: moe_layer_ep(x, logits, w1, w2, k, ea, ep, fuse_combine=fuse)  # noqa: E731
    if name == "moe_ep":
        eager = step().clone()
        graph = EpLayerGraph(x, logits, w1, w2, k, ea, ep, fuse_combine=True)
        parity["graph_equals_eager"] = bool(torch.equal(graph.replay(), eager))
        step = graph.replay
    return Workload(step, fl, 0.0,
                    f"expert-parallel MoE layer: {T} tokens total ({tl}/GPU), E={E} ({per}/GPU), top-{k}, d_model {D}; "
                    f"{how}; exchange inside the timed region; strong scaling", "moe_gemm_kernel", "tensor",
                    [x, logits], launches=12, cpu=cpu_moe, sharded=True, footprint=(w1.numel() + w2.numel()) * 2,
                    parity=parity)


def measure_fp8_peak(dev):
    """e4m3 tensor-core peak measured the way MEASURED_PEAKS.json measures the bf16 one: the vendor library's
    GEMM (torch._scaled_mm, e4m3 x e4m3 -> bf16) at 8192^3, best of 10, CUDA events. Denominator only."""
    import torch
    n = 8192
    a = _dev_randn((n, n), dev, 91, 0.1).to(torch.float8_e4m3fn)
    b = _dev_randn((n, n), dev, 92, 0.1).to(torch.float8_e4m3fn)
    one = torch.ones((), device=dev)
    try:
        for _ in range(3):
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        best = float("inf")
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return {"fp8_tflops": 2.0 * n ** 3 / (best * 1e-3) / 1e12,
                "how": "torch._scaled_mm e4m3 8192^3 -> bf16, best of 10, CUDA events, this run"}
    except Exception as e:  # no library kernel for this dtype: fall back to twice the bf16 figure, labelled
        return {"fp8_tflops": None, "how": f"torch._scaled_mm unavailable ({type(e).__name__}); 2 x bf16 burst used"}


def time_workload(wl, steps, warmup, dev, world, flush):
    """Device-resident timing of wl.step(): `warmup` untimed steps, then `steps` timed ones. When the working set
    fits the L2 a 256 MiB buffer is rewritten before every timed step and each step gets its own event pair."""
    import torch
    import torch.distributed as dist
    for _ in range(warmup):
        wl.step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if flush is not None:
        total = 0.0
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            wl.step()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        ms = total / steps
    else:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            wl.step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def time_e2e(wl, steps, dev, world):
    """The same step through the public Python entry point with HOST buffers: every step copies the workload's
    inputs from pinned host memory to the device, runs, and copies the result to pinned host memory."""
    import torch
    import torch.distributed as dist
    pins = [t.cpu().pin_memory() if t.dtype != torch.float8_e4m3fn else t.view(torch.uint8).cpu().pin_memory()
            for t in wl.inputs]
    views = [t if t.dtype != torch.float8_e4m3fn else t.view(torch.uint8) for t in wl.inputs]
    out = wl.step()
    out_pin = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def one():
        for d, p in zip(views, pins):
            d.copy_(p, non_blocking=True)
        out_pin.copy_(wl.step(), non_blocking=True)
    one()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        dist.barrier()
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    h2d = sum(p.numel() * p.element_size() for p in pins)
    d2h = out_pin.numel() * out_pin.element_size()
    return ms, h2d, d2h


def measure_config(name, rank, world, dev, steps, warmup, peaks, fp8_peak, flush, with_cpu):
    """One entry of `configs` (or the body of a `--workload` line)."""
    import torch
    wl = build_workload(name, rank, world, dev)
    need_flush = wl.footprint < 2 * L2_BYTES
    ms = time_workload(wl, steps, warmup, dev, world, flush if need_flush else None)
    tf = world * wl.flops / (ms * 1e-3) / 1e12
    if wl.bound == "hbm":
        ach, peak, unit, kind = wl.hbm_bytes / (ms * 1e-3) / 1e9, peaks["hbm"], "GB/s", "copy bandwidth, " + peaks["source"]
    elif wl.peak == "fp8":
        ach, unit = wl.flops / (ms * 1e-3) / 1e12, "TFLOP/s"
        if fp8_peak.get("fp8_tflops"):
            peak, kind = fp8_peak["fp8_tflops"], "torch._scaled_mm e4m3 8192^3 best of 10, measured in this run"
        else:
            peak, kind = 2 * peaks["bf16_burst"], "2 x burst cuBLAS bf16 (no fp8 library figure), " + peaks["source"]
    else:
        ach, peak, unit, kind = wl.flops / (ms * 1e-3) / 1e12, peaks["bf16_burst"], "TFLOP/s", "burst cuBLAS bf16, " + peaks["source"]
    e2e_ms, h2d, d2h = time_e2e(wl, max(2, min(steps, 3)), dev, world)
    out = {"tflops": tf, "ms": ms, "workload": wl.desc, "dtype": wl.dtype,
           "scaling": "strong" if wl.sharded else "weak (one replica per GPU)",
           "l2": "256 MiB buffer rewritten before every timed step" if need_flush else "working set exceeds the 126 MB L2; no flush",
           "roofline": {"bound": wl.bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                        "traffic": NCU_TRAFFIC.get(name), "kernel": wl.kernel, "peak_kind": kind},
           "e2e": {"value": world * wl.flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": e2e_ms,
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
           "gpu_launches_per_step": wl.launches}
    if wl.parity is not None:
        out["parity"] = wl.parity
    if with_cpu and wl.cpu is not None:
        val, what = wl.cpu()
        out["cpu_baseline"] = {"value": val, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": what}
    del wl
    torch.cuda.empty_cache()
    return out


CONFIG_NAMES = ["gemm_1024", "gemm_2048", "gemm_4096", "gemm_16384", "gemm_skinny", "gemm_strong", "attn", "attn_causal",
                "attn_short", "attn_short_causal", "fp8", "mxfp8", "moe", "moe_decode", "moe_ep"]


def run_single_workload(args, rank, local_rank, world):
    """`--workload NAME`: one JSON line for that workload alone, same keys as an entry of `configs` lifted to the
    top level."""
    import torch
    import torch.distributed as dist
    from triton_b200 import _lib
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = read_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    wl_probe = args.workload
    fp8_peak = measure_fp8_peak(dev) if wl_probe in ("fp8", "fp8_blockwise", "mxfp8", "moe_mx4", "moe_mx4_decode", "moe_fp8") else {}
    sampler = ClockSampler(local_rank)
    sampler.start()
    res = measure_config(args.workload, rank, world, dev, max(args.steps, 1), max(args.warmup, 3), peaks, fp8_peak, flush,
                         with_cpu=(world == 1 and not args.no_cpu_baseline))
    clocks = sampler.stop()
    _lib.sync_check(dev)
    if rank == 0:
        line = {"metric": f"{args.workload} throughput", "value": res["tflops"], "unit": "TFLOP/s", "n_gpus": world,
                "steps": max(args.steps, 1), "warmup": max(args.warmup, 3), "ms_per_step": res["ms"],
                "higher_is_better": True, "scaling": "strong" if res["scaling"] == "strong" else "weak",
                "vs_baseline": None, "dtype": res["dtype"], "data": "synthetic",
                "config": {"workload": res["workload"], "l2": res["l2"]},
                "roofline": res["roofline"], "e2e": res["e2e"],
                "gpu_launches": max(args.steps, 1) * world * res["gpu_launches_per_step"], "clocks": clocks}
        for key in ("parity", "cpu_baseline"):
            if key in res:
                line[key] = res[key]
        if fp8_peak:
            line["peaks_measured_here"] = fp8_peak
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def make_inputs(rank: int):
    import torch
    g = torch.Generator(device="cpu").manual_seed(1 + 1000 * rank)
    a = (torch.randn(M, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    return a, w


def cpu_baseline(budget_s: float = 20.0):
    """Times the CPU oracle (torch fp32 matmul, all threads) on the largest cube of the workload's family that
    fits the time budget; returns the cpu_baseline object."""
    import torch
    from oracle import gemm as o_gemm
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1)
    best = None
    rate = None
    for s in (1024, 2048, 4096, 8192):
        flops = 2.0 * s ** 3
        if rate is not None and flops / rate > budget_s:
            break
        a = (torch.randn(s, s, generator=g) / s ** 0.5).to(torch.bfloat16)
        w = (torch.randn(s, s, generator=g) / s ** 0.5).to(torch.bfloat16)
        o_gemm.gemm_ref(a[:256], w.t())  # warm the thread pool
        t0 = time.perf_counter()
        o_gemm.gemm_ref(a, w.t())
        dt = time.perf_counter() - t0
        rate = flops / dt
        best = (s, rate)
    s, rate = best
    return {"value": rate / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"torch CPU fp32 matmul of bf16 inputs, M=N=K={s} (one pass, all host threads)"}


def run_reference(args, rank: int, world: int):
    """Reference arm: the CPU path of the headline workload (the oracle port, torch CPU fp32 matmul) with all host
    threads, the same step count as the GPU arm and the full 8192^3 problem per step. Only when the whole run
    would take more than about four minutes is a step cut to a band of rows of A (stated in `sample`)."""
    if rank != 0:
        return
    import torch
    from oracle import gemm as o_gemm
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    warmup, steps = max(args.warmup, 0), max(args.steps, 1)
    a, w = make_inputs(0)
    t0 = time.perf_counter()
    o_gemm.gemm_ref(a[:1024], w.t())
    est_full = (time.perf_counter() - t0) * (M / 1024)
    rows = M
    budget = 240.0
    if est_full * (steps + warmup) > budget:
        rows = max(256, int(M * budget / (est_full * (steps + warmup))) // 256 * 256)
    a = a[:rows]
    for _ in range(warmup):
        o_gemm.gemm_ref(a, w.t())
    t0 = time.perf_counter()
    for _ in range(steps):
        o_gemm.gemm_ref(a, w.t())
    dt = (time.perf_counter() - t0) / steps
    val = 2.0 * rows * N * K / dt / 1e12
    sample = ("the full 8192^3 GEMM per step" if rows == M else f"a {rows}-row band of A against the full B per step "
              f"(the full problem would not fit {budget:.0f} s on these cores)") + \
        f", torch CPU fp32 matmul (the oracle port of the reference's check), {cores} threads"
    print(json.dumps({
        "impl": "reference", "metric": "bf16 GEMM throughput", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": CONFIG,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="headline GEMM only (skip the `configs` object)")
    ap.add_argument("--configs", default="", help="comma-separated subset of the configs to measure")
    ap.add_argument("--workload", default="gemm",
                    help="gemm (headline + configs, default) | " + " | ".join(CONFIG_NAMES) + " | attn_bwd | attn_bwd_causal | "
                         "attn_d256[_causal] | attn_bwd_ref_shape[_causal] | fp8_blockwise | moe_mx4 | moe_mx4_decode | moe_bf16_mx4 | moe_fp8 | mxfp4_upcast | "
                         "moe_ep_unfused | moe_ep_nccl | moe_small | attn_mxfp8 | attn_mxfp8_causal")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload != "gemm":
        run_single_workload(args, rank, local_rank, world)
        return

    import torch
    import torch.distributed as dist
    from triton_b200 import _lib
    from triton_b200.tutorials.blackwell_gemm_ws import matmul

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: triton_b200 has no CPU path")
    _lib.lib()  # fail loudly if the extension is missing
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    a_h, w_h = make_inputs(rank)
    a_pin, w_pin = a_h.pin_memory(), w_h.pin_memory()
    a = a_pin.to(dev, non_blocking=True)
    w = w_pin.to(dev, non_blocking=True)
    b = w.t()  # logical (K, N), K-major in memory
    c_pin = torch.empty(M, N, dtype=torch.bfloat16).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-resident timing
    for _ in range(warmup):
        c = matmul(a, b)
    barrier()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    sampler = ClockSampler(local_rank)
    sampler.start()
    t_all0 = torch.cuda.Event(enable_timing=True)
    t_all1 = torch.cuda.Event(enable_timing=True)
    t_all0.record()
    for i in range(steps):
        starts[i].record()
        c = matmul(a, b)
        ends[i].record()
    t_all1.record()
    sampler.sample()
    barrier()
    clocks = sampler.stop()
    _lib.sync_check(dev)
    total_ms = t_all0.elapsed_time(t_all1)
    kernel_ms = statistics.mean(s.elapsed_time(e) for s, e in zip(starts, ends))

    # ---------------------------------------------------------------- sustained leg (>= 2 s back to back)
    sus = None
    if rank == 0 or world > 1:
        n_sus = max(200, int(2.2e3 / max(kernel_ms, 1e-3)))
        sampler2 = ClockSampler(local_rank)
        barrier()
        sampler2.start()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(n_sus):
            matmul(a, b)
        s1.record()
        barrier()
        ck = sampler2.stop()
        sus_ms = s0.elapsed_time(s1)
        sus = {"launches": n_sus, "seconds": sus_ms / 1e3, "tflops": 2.0 * M * N * K * n_sus / (sus_ms * 1e-3) / 1e12,
               "clocks": ck}

    # ---------------------------------------------------------------- end to end (host buffers)
    # Every step copies its A and W from pinned host memory, multiplies, and copies its C back to pinned host
    # memory. The three legs run on three streams with two sets of device buffers, so step i's read-back overlaps
    # step i+1's upload and product (PCIe is full duplex); a step's own legs stay ordered by events.
    e2e_steps = max(3, min(steps, 10))
    s_cmp = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    a_d = [torch.empty_like(a) for _ in range(2)]
    w_d = [torch.empty_like(w) for _ in range(2)]
    c_d = [None, None]
    c_pins = [c_pin, torch.empty(M, N, dtype=torch.bfloat16).pin_memory()]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        j = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[j])          # the product that last read these input buffers is done
            a_d[j].copy_(a_pin, non_blocking=True)
            w_d[j].copy_(w_pin, non_blocking=True)
            ev_in[j].record(s_in)
        s_cmp.wait_event(ev_in[j])
        s_cmp.wait_event(ev_out[j])             # the read-back of the output this slot held is done
        c_d[j] = matmul(a_d[j], w_d[j].t())
        ev_cmp[j].record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[j])
            c_pins[j].copy_(c_d[j], non_blocking=True)
            ev_out[j].record(s_out)

    for i in range(2):
        e2e_step(i)
    s_cmp.wait_stream(s_out)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    s_in.wait_event(e0)
    for i in range(e2e_steps):
        e2e_step(i)
    s_cmp.wait_stream(s_out)
    s_cmp.wait_stream(s_in)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    e2e_check = torch.equal(c_pins[(e2e_steps - 1) & 1], c.cpu())  # the pipelined result is the resident one
    del a_d, w_d, c_d

    if world > 1:
        t = torch.tensor([total_ms, kernel_ms, e2e_ms, sus["seconds"]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, kernel_ms, e2e_ms, sus_s = t.tolist()
        sus["tflops"] *= sus["seconds"] / sus_s
        sus["seconds"] = sus_s

    # ---------------------------------------------------------------- every other configuration of the metric
    peaks = read_peaks()
    configs = {}
    fp8_peak = {}
    headline = {}  # filled below; the watchdog prints it if a multi-rank config never returns

    def emit(extra_note=None):
        if rank != 0 or not headline:
            return
        out = dict(headline)
        if configs:
            out["configs"] = dict(configs)
        if fp8_peak:
            out["peaks_measured_here"] = fp8_peak
        if extra_note:
            out["note"] = extra_note
        print(json.dumps(out), flush=True)

    # A config that involves other ranks (gemm_strong, moe_ep) can only hang if a peer is lost; the headline must
    # not be lost with it: after this many seconds without finishing, rank 0 prints what it has and every rank exits.
    watchdog = None
    if world > 1 and not args.no_configs:
        def give_up():
            emit("a multi-rank config did not return within the watchdog limit; the line holds what was measured before")
            os._exit(0)
        watchdog = threading.Timer(420.0, give_up)
        watchdog.daemon = True
    if rank == 0:
        flops = 2.0 * M * N * K
        ms_per_step = total_ms / steps
        value = world * flops / (ms_per_step * 1e-3) / 1e12
        sustained = total_ms > 500.0
        peak = peaks["bf16_sustained"] if sustained else peaks["bf16_burst"]
        achieved = flops / (kernel_ms * 1e-3) / 1e12
        headline.update({
            "metric": "bf16 GEMM throughput", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": CONFIG,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC["gemm"],
                         "peak_kind": ("sustained" if sustained else "burst") + " cuBLAS bf16, " + peaks["source"],
                         "frac_of_nominal_2250": achieved / 2250.0, "kernel": "gemm_kernel<256,4,PAIR,bf16> (256x512 tile per CTA pair)"},
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": 2 * M * K * 2, "d2h_bytes_per_step": M * N * 2, "steps": e2e_steps,
                    "pipeline": "3 streams (upload | product | read-back), 2 buffer sets", "matches_resident": e2e_check},
            "gpu_launches": steps * world,
            "clocks": clocks,
        })
        if sus is not None:
            mhz, mx = sus["clocks"]["sm_mhz"], sus["clocks"]["sm_max_mhz"]
            per_gpu = sus["tflops"]
            headline["sustained"] = {
                "tflops": world * per_gpu, "tflops_per_gpu": per_gpu, "seconds": sus["seconds"], "launches": sus["launches"],
                "sm_mhz_median": mhz, "sm_max_mhz": mx, "reasons": sus["clocks"]["reasons"],
                "tflops_per_gpu_at_max_clock": per_gpu * mx / mhz if mhz and mx else None,
                "peak": peaks["bf16_sustained"], "frac": per_gpu / peaks["bf16_sustained"],
                "peak_kind": "sustained cuBLAS bf16 (4 s back to back), " + peaks["source"]}
        if world == 1 and not args.no_cpu_baseline:
            headline["cpu_baseline"] = cpu_baseline()
    if watchdog is not None:
        watchdog.start()
    if not args.no_configs:
        names = [n for n in (args.configs.split(",") if args.configs else CONFIG_NAMES) if n]
        del a, w, b, c
        torch.cuda.empty_cache()
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        if any(n in ("fp8", "mxfp8", "fp8_blockwise") for n in names):
            fp8_peak = measure_fp8_peak(dev)
        for name in names:
            # a config that cannot run must not take the headline down with it: its entry then says why
            try:
                configs[name] = measure_config(name, rank, world, dev, 10, 3, peaks, fp8_peak, flush,
                                               with_cpu=(world == 1 and rank == 0 and not args.no_cpu_baseline))
                _lib.sync_check(dev)
            except Exception as e:  # noqa: BLE001
                configs[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.empty_cache()

    if watchdog is not None:
        watchdog.cancel()
    emit()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
