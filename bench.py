#!/usr/bin/env python
"""Benchmark driver.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (the configuration the headline metric is quoted on): the bf16 persistent
warp-specialised GEMM, M=N=K=8192, A row-major, B supplied K-major, entries N(0,1)/sqrt(K) from
seed 1, fp32 accumulation, bf16 output. One "step" is one GEMM over resident inputs. With N GPUs
every rank owns one 8192-column block of a K x (8192*N) B (no collective on the data path; weak
scaling) and the reported value is the whole job's TFLOP/s with the time taken as the max over
ranks.

One JSON line is printed by rank 0. Keys beyond the base contract:
  roofline      tensor-pipe roofline of the GEMM kernel: achieved = 2MNK / mean CUDA-event duration
                of the launches in the timed region, peak = measured cuBLAS bf16 figure from
                MEASURED_PEAKS.json (burst figure when the timed region is shorter than 0.5 s,
                else the sustained one), traffic = DRAM bytes per launch from the committed ncu
                capture (profiles/), or null.
  e2e           same metric through the public Python entry point with HOST (pinned) inputs and a
                host result: H2D copies of A and B and the D2H copy of C are inside the timed region.
  cpu_baseline  the CPU oracle (torch CPU fp32 matmul, all host threads) timed on a bounded sample.
  clocks        SM clock / throttle reasons sampled through NVML during the timed region.

`--impl reference` times the reference's CPU path for this workload (the oracle port: the
reference's own kernels need a GPU and its compiler, which cannot be built offline) on a bounded
sample per step with all host threads.
"""
from __future__ import annotations

import argparse
import json
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

# DRAM bytes per launch of gemm_kernel<256,4> at 8192^3 from the committed ncu capture
# (profiles/gemm_bf16_8192.md); None until a capture exists.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1.04e9


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
            time.sleep(0.01)

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


def build_workload(name: str, rank: int, dev):
    """Returns (step, flops_per_step, hbm_bytes_per_step, description, kernel, bound) for an extra
    workload (`--workload`); the default GEMM workload is handled in main()."""
    import math
    import torch
    g = torch.Generator(device="cpu").manual_seed(2 + 1000 * rank)
    if name in ("attn", "attn_causal", "attn_short", "attn_short_causal"):
        from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_with_lse
        causal = name.endswith("causal")
        B, H, S, D = (32, 32, 1024, 128) if "short" in name else (4, 32, 8192, 128)
        q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(3))
        sc = 1.0 / math.sqrt(D)
        fl = 4.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S)
        return (lambda: attention_with_lse(q, k, v, sc, causal), fl, 4.0 * B * H * S * D * 2,
                f"flash-attention fwd bf16 [B={B},H={H},S={S},D={D}] causal={causal}, seed 2", "attention_fwd_kernel<128>",
                "tensor")
    if name in ("attn_bwd", "attn_bwd_causal", "attn_bwd_ref_shape", "attn_bwd_ref_shape_causal"):
        from triton_b200.tutorials.blackwell_fa_ws_pipelined_persistent import attention_backward, attention_with_lse
        causal = name.endswith("causal")
        # "ref_shape": Z=4, H=16, N=2048, the first shape of the reference's published backward table
        B, H, S, D = (4, 16, 2048, 128) if "ref_shape" in name else (4, 32, 8192, 128)
        q, k, v, do = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).to(dev) for _ in range(4))
        sc = 1.0 / math.sqrt(D)
        o, lse = attention_with_lse(q, k, v, sc, causal)
        fl = 10.0 * B * H * D * (S * (S + 1) / 2 if causal else S * S)  # five S x S x D products
        return (lambda: attention_backward(q, k, v, o, lse, do, sc, causal), fl, 8.0 * B * H * S * D * 2,
                f"flash-attention bwd bf16 [B={B},H={H},S={S},D={D}] causal={causal} (delta + main + dq kernels), seed 2",
                "attention_bwd_kernel", "tensor")
    if name == "gemm_skinny":
        from triton_b200.tutorials.blackwell_gemm_ws import matmul
        m, n = 128, 8192
        a = (torch.randn(m, n, generator=g) / n ** 0.5).to(torch.bfloat16).to(dev)
        ws = [(torch.randn(n, n, generator=g) / n ** 0.5).to(torch.bfloat16).to(dev) for _ in range(4)]
        turn = [0]

        def step():  # four weight matrices in turn: 512 MiB, so none of them stays in the 126 MB L2
            turn[0] = (turn[0] + 1) & 3
            return matmul(a, ws[turn[0]].t())
        return (step, 2.0 * m * n * n, 2.0 * (n * n + m * n + m * n),
                "bf16 GEMM M=128, N=K=8192 (the skinny case), B K-major, four weight matrices in turn", "gemm_kernel<128,6> + splitk_reduce_kernel",
                "hbm")
    if name in ("fp8", "fp8_blockwise", "mxfp8"):
        n = 8192
        a = (torch.randn(n, n, generator=g) * 0.1).to(torch.float8_e4m3fn).to(dev)
        b = (torch.randn(n, n, generator=g) * 0.1).to(torch.float8_e4m3fn).to(dev)
        if name == "fp8":
            from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
            sa, sb = torch.rand(1, generator=g).to(dev), torch.rand(1, generator=g).to(dev)
            return (lambda: blackwell_scaled_mm_ws(a, b, sa, sb, scale_mode="tensorwise"), 2.0 * n ** 3, 3.0 * n * n,
                    "per-tensor-scaled e4m3 GEMM 8192^3, bf16 out", "gemm_kernel<256,4,pair,f8>", "tensor")
        if name == "fp8_blockwise":
            from triton_b200.tutorials.blackwell_scaled_mm_ws import blackwell_scaled_mm_ws
            sa = torch.rand(n, n // 128, generator=g).t().contiguous().t().to(dev)
            sb = torch.rand(n // 128, n // 128, generator=g).to(dev)
            return (lambda: blackwell_scaled_mm_ws(a, b, sa, sb, scale_mode="blockwise"), 2.0 * n ** 3, 3.0 * n * n,
                    "blockwise-scaled (128-wide K groups) e4m3 GEMM 8192^3, bf16 out", "gemm_fp8_blockwise_kernel",
                    "tensor")
        from triton_b200.tutorials.blackwell_gemm_ws_mxfp8 import matmul as mx_matmul
        u = torch.randint(-4, 5, (n * n // 32, ), generator=g)
        sc = (u + 127).to(torch.uint8).to(dev).view(torch.float8_e8m0fnu)
        return (lambda: mx_matmul(a, b, sc, sc), 2.0 * n ** 3, 3.0 * n * n + 2 * n * n / 32,
                "MXFP8 block-scaled GEMM 8192^3 (e8m0 scales 2^u, u in [-4,4]), bf16 out", "gemm_mxfp8_kernel<256,4>",
                "tensor")
    if name in ("moe", "moe_decode"):
        from triton_b200.triton_kernels.matmul import matmul as moe_matmul, swiglu_activation
        from triton_b200.triton_kernels.reduce import reduce
        from triton_b200.triton_kernels.tensor import make_ragged_tensor_metadata
        from triton_b200.triton_kernels.topk import topk
        T, D, F, E, k = (64 if name == "moe_decode" else 16384), 4096, 1536, 128, 4
        g4 = torch.Generator(device="cpu").manual_seed(4 + 1000 * rank)
        x = torch.randn(T, D, generator=g4).to(torch.bfloat16).to(dev)
        logits = torch.randn(T, E, generator=g4).to(dev)
        w1 = (0.02 * torch.randn(E, D, 2 * F, generator=g4)).to(torch.bfloat16).to(dev)
        w2 = (0.02 * torch.randn(E, F, D, generator=g4)).to(torch.bfloat16).to(dev)
        act = swiglu_activation(1.0, None)
        y = torch.empty(T * k, D, dtype=torch.bfloat16, device=dev)

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
        return (step, fl, by, f"MoE layer: {T} tokens, d_model {D}, E={E}, top-{k}, W1 [{D},{2*F}] SwiGLU W2 [{F},{D}], "
                "gate-weighted combine, seed 4", "moe_gemm_kernel", "hbm" if name == "moe_decode" else "tensor")
    if name in ("moe_mx4", "moe_mx4_decode", "moe_bf16_mx4"):
        from triton_b200.triton_kernels.matmul import PrecisionConfig, matmul as moe_matmul, swiglu_activation
        from triton_b200.triton_kernels.numerics_details.mxfp import downcast_to_mxfp
        from triton_b200.triton_kernels.reduce import reduce
        from triton_b200.triton_kernels.tensor import FP4, convert_layout, make_ragged_tensor_metadata, wrap_torch_tensor
        from triton_b200.triton_kernels.tensor_details.layout import (make_default_matmul_mxfp4_w_layout,
                                                                      make_default_matmul_mxfp4_w_scale_layout)
        from triton_b200.triton_kernels.topk import topk
        T = 64 if name == "moe_mx4_decode" else 16384
        D, F, E, k = 4096, 1536, 128, 4
        g4 = torch.Generator(device="cpu").manual_seed(4 + 1000 * rank)
        x = torch.randn(T, D, generator=g4)
        x = (x.to(torch.bfloat16) if name == "moe_bf16_mx4" else x.to(torch.float8_e4m3fn)).to(dev)
        logits = torch.randn(T, E, generator=g4).to(dev)

        def prep(w):  # quantise on the GPU, expert by expert chunks to bound memory
            v, s = downcast_to_mxfp(w.to(dev).to(torch.bfloat16), torch.uint8, axis=1)
            return (convert_layout(wrap_torch_tensor(v, dtype=FP4), make_default_matmul_mxfp4_w_layout(mx_axis=1)),
                    convert_layout(wrap_torch_tensor(s), make_default_matmul_mxfp4_w_scale_layout(mx_axis=1)))
        w1, s1 = prep(0.02 * torch.randn(E, D, 2 * F, generator=g4))
        w2, s2 = prep(0.02 * torch.randn(E, F, D, generator=g4))
        # GEMM 1 writes fp8 (the default: the activations' dtype), GEMM 2 bf16 for the combine
        pc1, pc2 = PrecisionConfig(b_mx_scale=s1), PrecisionConfig(b_mx_scale=s2, out_dtype=torch.bfloat16)
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
        if name == "moe_bf16_mx4":
            # bf16 activations: each GEMM upcasts its MXFP4 weight to bf16 first (per call, as a user of matmul gets it)
            pcb1, pcb2 = PrecisionConfig(b_mx_scale=s1), PrecisionConfig(b_mx_scale=s2)

            def step_bf16():
                sm = topk(logits, k)
                mm = sm.mask_metadata
                rg = make_ragged_tensor_metadata(mm.col_sum, T * k)
                combine = mm.col_sorted_indx
                gather = torch.div(combine, k, rounding_mode="trunc")
                gam = sm.vals.float().reshape(-1)[combine.long()]
                h = moe_matmul(x, w1, None, rg, gather_indx=gather, precision_config=pcb1, fused_activation=act)
                y = moe_matmul(h, w2, None, rg, scatter_indx=combine, gammas=gam, precision_config=pcb2)
                return reduce(y.view(T, k, D), dim=1)[0]
            return (step_bf16, fl, 0.0, f"MoE layer, bf16 activations x MXFP4 weights (upcast pass + 16-bit grouped GEMM per "
                    f"call): {T} tokens, d_model {D}, E={E}, top-{k}, seed 4", "moe_gemm_kernel", "tensor")
        active = int((topk(logits, k).mask_metadata.col_sum > 0).sum().item())
        by = active * (D * 2 * F + F * D) * (0.5 + 1.0 / 32) + R * (D + F) * 1.0 + R * (F * 1.0 + D * 2.0)
        return (step, fl, by, f"MoE layer, fp8 activations x MXFP4 weights: {T} tokens, d_model {D}, E={E}, top-{k}, "
                f"W1 [{D},{2*F}] SwiGLU W2 [{F},{D}], gate-weighted combine, seed 4", "moe_gemm_mx4_kernel",
                "hbm" if name == "moe_mx4_decode" else "tensor")
    if name == "mxfp4_upcast":
        from triton_b200.triton_kernels.matmul import upcast_mxfp4_weight
        from triton_b200.triton_kernels.tensor import FP4, convert_layout, wrap_torch_tensor
        from triton_b200.triton_kernels.tensor_details.layout import (make_default_matmul_mxfp4_w_layout,
                                                                      make_default_matmul_mxfp4_w_scale_layout)
        E, Kd, Nd = 128, 4096, 3072
        g4 = torch.Generator(device="cpu").manual_seed(4 + 1000 * rank)
        v = torch.randint(0, 256, (E, Kd // 2, Nd), generator=g4, dtype=torch.uint8).to(dev)
        s = torch.randint(118, 130, (E, Kd // 32, Nd), generator=g4, dtype=torch.uint8).to(dev)
        wv = convert_layout(wrap_torch_tensor(v, dtype=FP4), make_default_matmul_mxfp4_w_layout(mx_axis=1))
        ws = convert_layout(wrap_torch_tensor(s), make_default_matmul_mxfp4_w_scale_layout(mx_axis=1))
        del v, s
        by = E * Kd * Nd * (0.5 + 1.0 / 32 + 2.0)
        return (lambda: upcast_mxfp4_weight(wv, ws, torch.bfloat16), 0.0, by,
                f"MXFP4 -> bf16 weight upcast: E={E} matrices [{Kd},{Nd}] (W1 of the MoE layer), random codes, seed 4",
                "mxfp4_upcast_kernel", "hbm")
    if name == "moe_ep":
        import torch.distributed as dist
        from triton_b200.triton_kernels.distributed import (EpGroup, make_expt_assignment, make_expt_dict_uniform,
                                                            moe_layer_ep)
        world = dist.get_world_size() if dist.is_initialized() else 1
        T, D, F, E, k = 16384, 4096, 1536, 128, 4
        tl, per = T // world, E // world
        g4 = torch.Generator(device="cpu").manual_seed(4 + 1000 * rank)
        x = torch.randn(tl, D, generator=g4).to(torch.bfloat16).to(dev)
        logits = torch.randn(tl, E, generator=g4).to(dev)
        w1 = (0.02 * torch.randn(per, D, 2 * F, generator=g4)).to(torch.bfloat16).to(dev)
        w2 = (0.02 * torch.randn(per, F, D, generator=g4)).to(torch.bfloat16).to(dev)
        ea = make_expt_assignment(world, E, make_expt_dict_uniform(world, E), dev)
        ep = EpGroup()
        R = T * k
        fl = (2.0 * R * D * 2 * F + 2.0 * R * F * D) / world  # per rank; the line reports world * this
        return (lambda: moe_layer_ep(x, logits, w1, w2, k, ea, ep), fl, 0.0,
                f"expert-parallel MoE layer: {T} tokens total ({tl}/GPU), E={E} ({per}/GPU), top-{k}, d_model {D}, "
                "NCCL all-to-all dispatch/combine inside the timed region; strong scaling", "moe_gemm_kernel", "tensor")
    raise SystemExit(f"unknown workload {name}")


# Kernels of this library launched per step: the MoE layer runs topk, three bitmatrix-metadata kernels,
# the ragged-metadata kernel, two grouped GEMMs and the top-k reduce (the EP variant adds four row moves), and
# with 2048 or more sorted rows the row gather ahead of GEMM 1.
OWN_LAUNCHES_PER_STEP = {"moe": 9, "moe_decode": 8, "moe_ep": 12, "moe_mx4": 9, "moe_mx4_decode": 9, "moe_bf16_mx4": 11, "gemm_skinny": 2, "attn_bwd": 3, "attn_bwd_causal": 3,
                         "attn_bwd_ref_shape": 3, "attn_bwd_ref_shape_causal": 3}


def run_extra_workload(args, rank, local_rank, world):
    """Times one of the non-headline workloads on each rank (independent replicas of the sharded
    unit: (batch, head) groups for attention, N blocks for GEMMs, expert groups for MoE) and prints
    one JSON line with the same keys as the headline line."""
    import torch
    import torch.distributed as dist
    from triton_b200 import _lib
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    step, fl, by, desc, kernel, bound = build_workload(args.workload, rank, dev)
    warmup, steps = max(args.warmup, 3), max(args.steps, 1)
    for _ in range(warmup):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    sampler.sample()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    _lib.sync_check(dev)
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        peaks = read_peaks()
        tf = world * fl / (ms * 1e-3) / 1e12
        if bound == "hbm":
            ach, peak, unit = by / (ms * 1e-3) / 1e9, peaks["hbm"], "GB/s"
        else:
            ach, peak, unit = fl / (ms * 1e-3) / 1e12, peaks["bf16_burst"], "TFLOP/s"
        print(json.dumps({
            "metric": f"{args.workload} throughput", "value": tf, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong" if args.workload == "moe_ep" else "weak", "vs_baseline": None,
            "dtype": "e4m3" if args.workload in ("fp8", "fp8_blockwise", "mxfp8", "moe_mx4", "moe_mx4_decode") else "bf16", "data": "synthetic",
            "config": {"workload": desc},
            "roofline": {"bound": bound, "achieved": ach, "peak": peak, "unit": unit, "frac": ach / peak,
                         "traffic": None, "kernel": kernel,
                         "peak_kind": ("copy bandwidth" if bound == "hbm" else "burst cuBLAS bf16") + ", " + peaks["source"]},
            "gpu_launches": steps * world * OWN_LAUNCHES_PER_STEP.get(args.workload, 1), "clocks": clocks}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def make_inputs(rank: int, device):
    import torch
    g = torch.Generator(device="cpu").manual_seed(1 + 1000 * rank)
    a = (torch.randn(M, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    return a, w


def cpu_baseline(budget_s: float = 20.0):
    """Times the CPU oracle (torch fp32 matmul, all threads) on the largest cube of the workload's
    family that fits the time budget; returns the cpu_baseline object."""
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
    """Reference arm: the CPU path of the workload (oracle port) with all host threads; each step is
    a 256-row band of the 8192^3 GEMM."""
    if rank != 0:
        return
    import torch
    from oracle import gemm as o_gemm
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(1)
    rows = 256
    a = (torch.randn(rows, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    for _ in range(max(1, min(args.warmup, 2))):
        o_gemm.gemm_ref(a, w.t())
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        o_gemm.gemm_ref(a, w.t())
    dt = (time.perf_counter() - t0) / steps
    val = 2.0 * rows * N * K / dt / 1e12
    sample = f"{rows}-row band of the 8192^3 GEMM per step, torch CPU fp32 matmul, {steps} timed steps"
    print(json.dumps({
        "impl": "reference", "metric": "bf16 GEMM throughput", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "reference_path": "CPU (oracle port of the reference's torch check); "
                   "the reference's TLX kernels need its own compiler build and a GPU"},
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
    ap.add_argument("--workload", default="gemm",
                    help="gemm (headline, default) | gemm_skinny | attn | attn_causal | attn_short | attn_short_causal | attn_bwd | "
                         "attn_bwd_causal | attn_bwd_ref_shape[_causal] | fp8 | fp8_blockwise | mxfp8 | moe | moe_decode | moe_mx4 | moe_mx4_decode | moe_bf16_mx4 | mxfp4_upcast | moe_ep")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.workload != "gemm":
        run_extra_workload(args, rank, local_rank, world)
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
    a_h, w_h = make_inputs(rank, dev)
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

    if world > 1:
        t = torch.tensor([total_ms, kernel_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, kernel_ms, e2e_ms = t.tolist()

    if rank == 0:
        flops = 2.0 * M * N * K
        ms_per_step = total_ms / steps
        value = world * flops / (ms_per_step * 1e-3) / 1e12
        peaks = read_peaks()
        sustained = total_ms > 500.0
        peak = peaks["bf16_sustained"] if sustained else peaks["bf16_burst"]
        achieved = flops / (kernel_ms * 1e-3) / 1e12
        out = {
            "metric": "bf16 GEMM throughput", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sharding": "one 8192-column block of B per GPU, no collective",
                       "l2": "inputs (256 MiB) and output (128 MiB) exceed the 126 MB L2; no flush"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                         "peak_kind": ("sustained" if sustained else "burst") + " cuBLAS bf16, " + peaks["source"],
                         "frac_of_nominal_2250": achieved / 2250.0, "kernel": "gemm_kernel<256,4,PAIR,bf16> (256x512 tile per CTA pair)"},
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": 2 * M * K * 2, "d2h_bytes_per_step": M * N * 2, "steps": e2e_steps,
                    "pipeline": "3 streams (upload | product | read-back), 2 buffer sets", "matches_resident": e2e_check},
            "gpu_launches": steps * world,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline()
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
