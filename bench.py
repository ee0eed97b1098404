#!/usr/bin/env python
"""bench.py -- throughput of the GEMM hot path on B200, one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Default workload: the NVFP4 block-scaled GEMM M=8192, N=28672, K=8192 (bf16 output), the
configuration the sharded numbers are quoted on.  At N > 1 the weight matrix is split by output
columns across the ranks (strong scaling: total work fixed); A is replicated; no data-path
collective is inside the timed step (the NCCL all-gather of the bf16 output is timed beside it).

A step is one GEMM launch over inputs already resident in HBM.  L2 is flushed (a 256 MiB write)
between timed steps, each step is timed with CUDA events on the launching stream, the step times
are summed, and the maximum over ranks is reported.  `e2e` repeats the measurement through the
C ABI with HOST buffers: pinned activations copied in, the output copied back, every step.

`--impl reference` times Blaze's own host GEMM (tests/test_gemm_naive.cu:38-48, compiled into
oracle/_ref when the reference tree was present, otherwise the oracle's port of that loop) on the
box's host cores over a bounded row-slice of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, M, N, K) -- the reference's benchmark configurations
    "nvfp4_8192x28672x8192": ("nvfp4", 8192, 28672, 8192),
    "fp8_4096": ("fp8", 4096, 4096, 4096),
    "w4a16_4096x22016x4096": ("w4a16_bf16", 4096, 22016, 4096),
    "fp16_256": ("f16", 256, 256, 256),
    "nvfp4_4096x12288x4096": ("nvfp4", 4096, 12288, 4096),
    "nvfp4_4096x22016x4096": ("nvfp4", 4096, 22016, 4096),
    "bf16_8192": ("bf16", 8192, 8192, 8192),
}
DECODE_SHAPES = [(16, 12288, 4096), (16, 4096, 4096), (16, 22016, 4096), (16, 4096, 11008)]
NOMINAL_TFLOPS = {"nvfp4": 9000.0, "fp8": 4500.0, "f16": 2250.0, "bf16": 2250.0, "w4a16_bf16": 2250.0, "w4a16_f16": 2250.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch come from ncu captures kept in a tracked data
# file: per workload the bytes, the kernel instance that was captured and the commit it was captured at.
NCU_TRAFFIC_FILE = os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")
PEAK_MULT_OVER_BF16 = {"nvfp4": 4.0, "fp8": 2.0, "f16": 1.0, "bf16": 1.0, "w4a16_bf16": 1.0, "w4a16_f16": 1.0}


def ncu_traffic(key: str, kernel_info: dict | None) -> tuple:
    """(bytes per launch or None, provenance dict).  `stale` is set when the kernel that runs now is not the
    instance the capture was taken from (tile, stages, split or variant differ)."""
    try:
        with open(NCU_TRAFFIC_FILE) as f:
            rec = json.load(f).get(key)
    except Exception:
        rec = None
    if not rec:
        return None, {"source": "no ncu capture on record for this workload"}
    prov = {"source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch", "kernel": rec.get("kernel"), "commit": rec.get("commit")}
    if kernel_info is not None and rec.get("plan"):
        now = {k: kernel_info.get(k) for k in rec["plan"]}
        if now != rec["plan"]:
            prov["stale"] = True
            prov["plan_now"] = now
    return rec.get("bytes"), prov


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _loop(self):
        nv = self._nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        getter = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(getter(self._h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self) -> dict:
        s = sorted(self.samples)
        med = s[len(s) // 2] if s else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


# ------------------------------------------------------------------------- GPU workloads

class L2Flusher:
    def __init__(self, device):
        import torch
        self.buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=device)

    def flush(self):
        self.buf.fill_(1)


def make_operands(kind, M, N, K, device, seed_b=123):
    """Synthetic operands on the device: N(0,1) activations (seed 42), N(0,1) weights (seed 123; N(0,0.02)
    for W4A16), quantised by the library's own kernels.  Returns kwargs for GemmPlan and the byte count."""
    import torch
    from blaze_b200 import quantize_fp8, quantize_nvfp4
    ga = torch.Generator(device=device).manual_seed(42)
    gb = torch.Generator(device=device).manual_seed(seed_b)
    if kind == "nvfp4":
        xa = torch.randn((M, K), generator=ga, device=device)
        ad, asf, gA = quantize_nvfp4(xa, tiled=True); del xa
        xb = torch.randn((N, K), generator=gb, device=device)
        bd, bsf, gB = quantize_nvfp4(xb, tiled=True); del xb
        kw = dict(A=ad, B=bd, A_sf=asf, B_sf=bsf, a_scale=float(gA.item()), b_scale=float(gB.item()), a_sf_layout="tiled", b_sf_layout="tiled")
        nbytes = M * K // 2 + M * K // 16 + N * K // 2 + N * K // 16
    elif kind == "fp8":
        xa = torch.rand((M, K), generator=ga, device=device) * 2 - 1
        xb = torch.rand((N, K), generator=gb, device=device) * 2 - 1
        qa, sa = quantize_fp8(xa); qb, sb = quantize_fp8(xb)
        kw = dict(A=qa, B=qb, a_scale=float(sa[1].item()), b_scale=float(sb[1].item()))
        nbytes = M * K + N * K
    elif kind.startswith("w4a16"):
        dt = torch.bfloat16 if kind.endswith("bf16") else torch.float16
        A = torch.randn((M, K), generator=ga, device=device).to(dt)
        W = torch.randn((N, K), generator=gb, device=device) * 0.02
        bd, bsf, gB = quantize_nvfp4(W, tiled=True); del W
        kw = dict(A=A, B=bd, B_sf=bsf, b_scale=float(gB.item()), b_sf_layout="tiled")
        nbytes = M * K * 2 + N * K // 2 + N * K // 16
    else:
        dt = torch.bfloat16 if kind == "bf16" else torch.float16
        A = torch.randn((M, K), generator=ga, device=device).to(dt)
        B = torch.randn((N, K), generator=gb, device=device).to(dt)
        kw = dict(A=A, B=B)
        nbytes = (M * K + N * K) * 2
    torch.cuda.synchronize()
    return kw, nbytes


def time_steps(fn, steps, warmup, flusher, barrier=None):
    """W warm-ups, then K steps each bracketed by CUDA events with an L2 flush before it."""
    import torch
    for _ in range(warmup):
        flusher.flush(); fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flusher.flush()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    times = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    return sum(times) / steps, times


def run_gate_up(M, N, K, device, steps, warmup, flusher):
    """Llama-7B MLP entry, W4A16 bf16: silu(x Wg) * (x Wu) as ONE GEMM with the swiglu epilogue, beside the
    same result from two GEMMs (the gate one with SiLU) and one elementwise multiply."""
    import torch
    from blaze_b200 import GemmPlan, interleave_gate_up
    kg, _ = make_operands("w4a16_bf16", M, N, K, device, seed_b=123)
    ku, _ = make_operands("w4a16_bf16", M, N, K, device, seed_b=124)
    A = kg["A"]
    out = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    tmp = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    p_g = GemmPlan("w4a16_bf16", M, N, K, A, kg["B"], B_sf=kg["B_sf"], b_scale=kg["b_scale"], b_sf_layout="tiled", epilogue="silu")
    p_u = GemmPlan("w4a16_bf16", M, N, K, A, ku["B"], B_sf=ku["B_sf"], b_scale=ku["b_scale"], b_sf_layout="tiled")

    def separate():
        p_g.execute(tmp); p_u.execute(out); out.mul_(tmp)

    ms_sep, _ = time_steps(separate, steps, warmup, flusher)
    p_g.check(); p_u.check(); p_g.destroy(); p_u.destroy()
    # one kernel: rows interleaved in groups of 16; the tiled scale layout is per 128 rows, so the
    # row-major scales are interleaved and then tiled by the plan
    from blaze_b200 import quantize_nvfp4
    sf = []
    for seed in (123, 124):
        g = torch.Generator(device=device).manual_seed(seed)
        W = torch.randn((N, K), generator=g, device=device) * 0.02
        sf.append(quantize_nvfp4(W, tiled=False)[1]); del W
    B2 = interleave_gate_up(kg["B"], ku["B"], 16 * K // 2)
    S2 = interleave_gate_up(sf[0], sf[1], 16 * K // 16)
    p = GemmPlan("w4a16_bf16", M, 2 * N, K, A, B2, B_sf=S2, b_scale=kg["b_scale"], b_scale2=ku["b_scale"], epilogue="swiglu")
    fused = torch.empty((M, N), dtype=torch.bfloat16, device=device)
    ms_fused, _ = time_steps(lambda: p.execute(fused), steps, warmup, flusher)
    p.check()
    info = p.info()
    p.destroy()
    diff = (fused.float() - out.float()).abs().max().item()
    flops = 2.0 * M * (2 * N) * K
    return {"M": M, "N": N, "K": K, "one_kernel_ms": ms_fused, "one_kernel_tflops": flops / (ms_fused * 1e-3) / 1e12,
            "two_gemms_and_multiply_ms": ms_sep, "max_abs_diff": diff, "kernel": info, "launches": steps * info["launches"]}


def run_gemm_workload(kind, M, N, K, device, steps, warmup, flusher, out_dtype="bf16", barrier=None, variant="auto", seed_b=123, **plan_kw):
    import torch
    from blaze_b200 import GemmPlan
    kw, op_bytes = make_operands(kind, M, N, K, device, seed_b)
    A, B = kw.pop("A"), kw.pop("B")
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[out_dtype]
    C = torch.empty((M, N), dtype=dt, device=device)
    plan = GemmPlan(kind, M, N, K, A, B, out_dtype=out_dtype, variant=variant, **kw, **plan_kw)
    ms, times = time_steps(lambda: plan.execute(C), steps, warmup, flusher, barrier)
    plan.check()
    info = plan.info()
    return dict(plan=plan, C=C, A=A, B=B, kw=kw, ms=ms, times=times, info=info, op_bytes=op_bytes,
                flops=2.0 * M * N * K, out_bytes=M * N * C.element_size())


def run_sustained(plan, C, flops, seconds, device_index, peaks, mult):
    """The same plan launched back to back (no L2 flush, no gaps) for `seconds`: the rate under the power
    limit, beside the burst figure of single launches.  SM clock sampled during the region."""
    import torch
    for _ in range(3):
        plan.execute(C)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(); plan.execute(C); e.record(); torch.cuda.synchronize()
    one = max(s.elapsed_time(e), 1e-3)
    n = max(10, int(seconds * 1e3 / one))
    with ClockSampler(device_index, period_s=0.02) as clk:
        s.record()
        for _ in range(n):
            plan.execute(C)
        e.record()
        torch.cuda.synchronize()
    ms = s.elapsed_time(e) / n
    c = clk.summary()
    tf = flops / (ms * 1e-3) / 1e12
    return {"launches": n, "seconds": round(ms * n / 1e3, 3), "ms_per_step": ms, "tflops": tf,
            "frac_of_measured_sustained": tf / (peaks["bf16_tflops_sustained"] * mult),
            "peak": "%s sustained dense bf16 (%.1f TFLOP/s) x %g" % (peaks["source"], peaks["bf16_tflops_sustained"], mult),
            "sm_mhz_median": c["sm_mhz"], "ms_times_sm_mhz": (ms * c["sm_mhz"]) if c["sm_mhz"] else None, "reasons": c["reasons"]}, n


def run_comparator(kind, M, N, K, device, steps, flusher):
    """cuBLASLt's own scaled matmul (through torch) on the same operands, same events, same flush: a measured
    reference point for the block-scaled rates.  A comparator only -- nothing of the library calls it."""
    import torch
    import torch.nn.functional as F
    from blaze_b200 import GemmPlan
    try:
        kw, _ = make_operands(kind, M, N, K, device)
        A, B = kw.pop("A"), kw.pop("B")
        C = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        plan = GemmPlan(kind, M, N, K, A, B, out_dtype="bf16", **kw)
        ours_ms, _ = time_steps(lambda: plan.execute(C), steps, 3, flusher)
        plan.check()
        alpha = 1.0
        if kind == "nvfp4":
            from torch.nn.functional import ScalingType, SwizzleType
            a4, b4 = A.view(torch.float4_e2m1fn_x2), B.view(torch.float4_e2m1fn_x2).t()
            sa, sb = kw["A_sf"].view(torch.float8_e4m3fn), kw["B_sf"].view(torch.float8_e4m3fn)
            # block scales only (the fp32 tensor scales are applied to its result below): the one-kernel form
            alpha = kw["a_scale"] * kw["b_scale"]
            fn = lambda: F.scaled_mm(a4, b4, sa, ScalingType.BlockWise1x16, sb, ScalingType.BlockWise1x16,
                                     swizzle_a=SwizzleType.SWIZZLE_32_4_4, swizzle_b=SwizzleType.SWIZZLE_32_4_4, output_dtype=torch.bfloat16)
        elif kind == "fp8":
            a8, b8 = A.view(torch.float8_e4m3fn), B.view(torch.float8_e4m3fn).t()
            sa = torch.tensor([kw["a_scale"]], dtype=torch.float32, device=device)
            sb = torch.tensor([kw["b_scale"]], dtype=torch.float32, device=device)
            fn = lambda: torch._scaled_mm(a8, b8, sa, sb, out_dtype=torch.bfloat16)
        else:
            return {"unavailable": "no comparator for kind %s" % kind}
        D = fn()
        torch.cuda.synchronize()
        lib_ms, _ = time_steps(fn, steps, 3, flusher)
        rel = float(((D.float() * alpha - C.float()).abs() / C.float().abs().clamp_min(1.0)).max().item())
        plan.destroy()
        flops = 2.0 * M * N * K
        return {"ours_ms": ours_ms, "ours_tflops": flops / ours_ms / 1e9, "cublaslt_ms": lib_ms, "cublaslt_tflops": flops / lib_ms / 1e9,
                "ours_over_cublaslt": lib_ms / ours_ms, "max_rel_diff": rel}
    except Exception as ex:
        return {"unavailable": str(ex)[:200]}
    finally:
        torch.cuda.empty_cache()


def run_decode(device, steps, warmup, peaks, kind="nvfp4"):
    """M=16 decode projections of a Llama-7B layer (NVFP4 in the reference's benchmark ; the same shapes for the other kinds on
    request).  Enough distinct weight copies to exceed twice the L2 are cycled inside one CUDA graph
    so that every launch streams its weights from HBM."""
    import torch
    from blaze_b200 import GemmPlan
    out = []
    for (M, N, K) in DECODE_SHAPES:
        kw, _ = make_operands(kind, M, N, K, device)
        A, B = kw.pop("A"), kw.pop("B")
        if kind == "nvfp4":
            w_bytes = N * K // 2 + N * K // 16
            algo = w_bytes + M * K // 2 + M * K // 16 + 2 * M * N
        elif kind == "fp8":
            w_bytes = N * K
            algo = w_bytes + M * K + 2 * M * N
        else:                                                  # 16-bit activations x NVFP4 weights
            w_bytes = N * K // 2 + N * K // 16
            algo = w_bytes + M * K * 2 + 2 * M * N
        copies = max(2, -(-2 * 126 * 1024 * 1024 // w_bytes))
        Bs = [B] + [B.clone() for _ in range(copies - 1)]
        SFs = [kw["B_sf"]] + [kw["B_sf"].clone() for _ in range(copies - 1)] if "B_sf" in kw else [None] * copies
        C = torch.empty((M, N), dtype=torch.bfloat16, device=device)
        plans = []
        for b, sf in zip(Bs, SFs):
            k2 = dict(kw)
            if sf is not None:
                k2["B_sf"] = sf
            plans.append(GemmPlan(kind, M, N, K, A, b, out_dtype="bf16", **k2))
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for p in plans:
                p.execute(C)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for p in plans:
                    p.execute(C)
        for _ in range(max(3, warmup)):
            graph.replay()
        torch.cuda.synchronize()
        reps = max(3, steps)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            graph.replay()
        e.record()
        torch.cuda.synchronize()
        us = s.elapsed_time(e) * 1000.0 / (reps * copies)
        # beside it: the same number of launches of ONE plan, whose weights then stay in L2
        with torch.cuda.stream(stream):
            graph_l2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_l2, stream=stream):
                for _ in range(copies):
                    plans[0].execute(C)
        for _ in range(3):
            graph_l2.replay()
        torch.cuda.synchronize()
        s.record()
        for _ in range(reps):
            graph_l2.replay()
        e.record()
        torch.cuda.synchronize()
        us_l2 = s.elapsed_time(e) * 1000.0 / (reps * copies)
        plans[0].check()
        info = plans[0].info()
        gbs = algo / (us * 1e-6) / 1e9
        out.append({"M": M, "N": N, "K": K, "us_per_gemm": round(us, 3), "hbm_gbs": round(gbs, 1), "algorithmic_bytes": algo,
                    "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 4), "weight_copies_cycled": copies,
                    "us_per_gemm_weights_in_l2": round(us_l2, 3),
                    "split_k": info["split_k"], "grid": info["grid"], "launches": 2 * reps * copies})
        for p in plans:
            p.destroy()
        del Bs, SFs, plans, graph, graph_l2
        torch.cuda.empty_cache()
    return out


def run_e2e(res, steps, device, kind=None, shape=None, chunks=8, world=1, rank=0):
    """Same GEMM through the public call with HOST buffers: pinned activations (and their scale factors)
    copied to the device, the GEMM, the whole output copied back to pinned host memory, every step.
    The rows are cut into `chunks` blocks with one plan each (same weights), so that within a step the
    copy back of block i overlaps the copy in and the GEMM of block i+1 (three streams).  Steps do not
    overlap each other: a step's first copy in waits for the previous step's last copy back.
    With several ranks the host link is shared (the activations are replicated on every GPU), so each
    rank copies in only its 1/world share of the rows and the ranks all-gather them over NVLink first."""
    import torch
    from blaze_b200 import GemmPlan
    plan, C, A, kw = res["plan"], res["C"], res["A"], res["kw"]
    hA = torch.empty(A.shape, dtype=A.dtype, pin_memory=True); hA.copy_(A)
    sf = kw.get("A_sf")
    hS = None
    if sf is not None:
        hS = torch.empty(sf.shape, dtype=sf.dtype, pin_memory=True); hS.copy_(sf)
    hC = torch.empty(C.shape, dtype=C.dtype, pin_memory=True)
    h2d = A.numel() * A.element_size() + (sf.numel() if sf is not None else 0)
    d2h = C.numel() * C.element_size()
    M = A.shape[0]
    tiled_sf = sf is None or (kw.get("a_sf_layout") == "tiled" and sf.numel() % (M // 128 if M >= 128 else 1) == 0)
    if kind is None or M % (chunks * 256) != 0 or M // chunks < 1024 or not tiled_sf:
        chunks = 1

    if chunks == 1:
        def step():
            A.copy_(hA, non_blocking=True)
            if hS is not None:
                sf.copy_(hS, non_blocking=True)
            plan.execute(C)
            hC.copy_(C, non_blocking=True)
        plans = []
    else:
        _, N, K = shape
        Mc = M // chunks
        share = world > 1 and M % (world * 128) == 0          # the same decision on every rank
        if share:
            import torch.distributed as dist
            h2d = h2d // world
        sf_per_block = sf.numel() // (M // 128) if sf is not None else 0       # tiled scales: contiguous per 128 rows
        s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        plans, views = [], []
        for i in range(chunks):
            k2 = {k: v for k, v in kw.items() if k != "A_sf"}
            rows = slice(i * Mc, (i + 1) * Mc)
            sfv = hsv = None
            if sf is not None:
                blk = slice(i * (Mc // 128) * sf_per_block, (i + 1) * (Mc // 128) * sf_per_block)
                sfv, hsv = sf.view(-1)[blk], hS.view(-1)[blk]
                k2["A_sf"] = sfv
            plans.append(GemmPlan(kind, Mc, N, K, A[rows], res["B"], out_dtype=plan.out_dtype, **k2))
            views.append((A[rows], hA[rows], sfv, hsv, C[rows], hC[rows]))
        if share:
            # this rank's 1/world of all rows (and of the tiled scale blocks, contiguous per 128 rows)
            mine = slice(rank * (M // world), (rank + 1) * (M // world))
            a_mine, a_mine_h = A[mine], hA[mine]
            sf_mine = sf_mine_h = None
            if sf is not None:
                n_sf = sf.numel() // world
                sf_mine, sf_mine_h = sf.view(-1)[rank * n_sf:(rank + 1) * n_sf], hS.view(-1)[rank * n_sf:(rank + 1) * n_sf]
        done_prev = [torch.cuda.Event()]
        done_prev[0].record()

        def step():
            s_in.wait_event(done_prev[0])
            if share:
                with torch.cuda.stream(s_in):
                    a_mine.copy_(a_mine_h, non_blocking=True)
                    if sf_mine is not None:
                        sf_mine.copy_(sf_mine_h, non_blocking=True)
                    # in place: every rank's share already sits at its offset of the gathered tensor
                    dist.all_gather_into_tensor(A.view(-1), a_mine.view(-1))
                    if sf_mine is not None:
                        dist.all_gather_into_tensor(sf.view(-1), sf_mine)
                    ev_all = torch.cuda.Event(); ev_all.record(s_in)
                s_cmp.wait_event(ev_all)
            for i in range(chunks):
                a_d, a_h, s_d, s_h, c_d, c_h = views[i]
                if not share:
                    with torch.cuda.stream(s_in):
                        a_d.copy_(a_h, non_blocking=True)
                        if s_d is not None:
                            s_d.copy_(s_h, non_blocking=True)
                        ev_in = torch.cuda.Event(); ev_in.record(s_in)
                    s_cmp.wait_event(ev_in)
                with torch.cuda.stream(s_cmp):
                    plans[i].execute(c_d, stream=s_cmp.cuda_stream)
                    ev_c = torch.cuda.Event(); ev_c.record(s_cmp)
                s_out.wait_event(ev_c)
                with torch.cuda.stream(s_out):
                    c_h.copy_(c_d, non_blocking=True)
            ev = torch.cuda.Event(); ev.record(s_out)
            done_prev[0] = ev

    # the device copies of the activations are cleared first: what the GEMMs read must have come in through the steps
    A.zero_()
    if sf is not None:
        sf.zero_()
    torch.cuda.synchronize()
    step(); torch.cuda.synchronize()
    t0 = time.perf_counter()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if chunks == 1:
        s.record()
        for _ in range(steps):
            step()
        e.record()
    else:
        s.record(s_in)
        for _ in range(steps):
            step()
        s_out.wait_event(done_prev[0])
        e.record(s_out)
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3 / steps
    ms = s.elapsed_time(e) / steps
    for p in plans:
        p.check(); p.destroy()
    checksum = float(hC.view(-1)[:1024].float().abs().sum())       # the host copy is read
    arrived = bool(torch.equal(A.cpu(), hA)) and (sf is None or bool(torch.equal(sf.cpu(), hS)))
    if not arrived:
        raise RuntimeError("end-to-end step: the activations on the device differ from the host copy")
    return ms, h2d, d2h, checksum, chunks, wall_ms


# ------------------------------------------------------------------------- CPU reference arm

def cpu_reference_gemm(kind, M, N, K, target_seconds, threads=None):
    """Times the host reference GEMM on a row-slice of the workload.  NVFP4 / FP8 operands are
    dequantised first (exactly representable in fp16), so Blaze's own gemm_cpu_fp16 applies as is."""
    import numpy as np
    from oracle import build_oracle
    build_oracle.build_oracle()
    from oracle import oracle as O
    threads = threads or (os.cpu_count() or 1)
    use_ref = O.ref_available()
    rng = np.random.default_rng(123)
    # operands of the slice: quantise on the host with the oracle (a few rows of A, all of B is too
    # much for the reference's [K, N] fp16 layout at the large configs, so N is sliced as well)
    n_slice = min(N, 2048)
    xb = rng.standard_normal((n_slice, K)).astype(np.float32)
    xa_row = np.random.default_rng(42).standard_normal((1, K)).astype(np.float32)
    if kind == "nvfp4":
        bd, bsf, _ = O.quantize_nvfp4(xb); Bt = O.dequant_nvfp4_noglobal(bd, bsf)
        deq_a = lambda x: O.dequant_nvfp4_noglobal(*O.quantize_nvfp4(x)[:2])
    elif kind == "fp8":
        Bt = O.e4m3_to_f32(O.quantize_fp8(xb)[0]); deq_a = lambda x: O.e4m3_to_f32(O.quantize_fp8(x)[0])
    else:
        Bt = O.f16_to_f32(O.f32_to_f16(xb)); deq_a = lambda x: O.f16_to_f32(O.f32_to_f16(x))
    B16_kn = np.ascontiguousarray(O.f32_to_f16(Bt).T)                   # Blaze's [K, N] fp16 layout

    def run(rows):
        A32 = deq_a(np.repeat(xa_row, rows, axis=0) * np.linspace(0.5, 1.5, rows, dtype=np.float32)[:, None])
        A16 = O.f32_to_f16(A32)
        t0 = time.perf_counter()
        if use_ref:
            chunks = np.array_split(np.arange(rows), min(threads, rows))
            outs = [None] * len(chunks)

            def work(i):
                outs[i] = O.ref_gemm_cpu_fp16(A16[chunks[i]], B16_kn)
            ths = [threading.Thread(target=work, args=(i,)) for i in range(len(chunks))]
            [t.start() for t in ths]; [t.join() for t in ths]
        else:
            O.gemm_f32(A32, Bt, nthreads=threads)
        return time.perf_counter() - t0

    t1 = run(threads)                                                   # calibration: one row per thread
    rows = max(threads, int(threads * max(1.0, target_seconds / max(t1, 1e-3))))
    rows = min(rows, M)
    return dict(run=run, rows=rows, n_slice=n_slice, threads=threads, kind="reference" if use_ref else "port", calib_s=t1)


def reference_arm(args, kind, M, N, K, workload_name):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    total = args.steps + args.warmup
    per_step = max(0.5, min(8.0, 150.0 / max(total, 1)))
    ref = cpu_reference_gemm(kind, M, N, K, per_step)
    rows, n_slice = ref["rows"], ref["n_slice"]
    for _ in range(args.warmup):
        ref["run"](rows)
    t = [ref["run"](rows) for _ in range(args.steps)]
    sec = sum(t) / len(t)
    flops = 2.0 * rows * n_slice * K
    value = flops / sec / 1e12
    sample = "%d rows x %d columns x K=%d slice of the workload per step, %s" % (
        rows, n_slice, K, "Blaze gemm_cpu_fp16 (oracle/_ref) on row chunks, one thread each" if ref["kind"] == "reference" else "oracle port of gemm_cpu_fp16")
    line = {"impl": "reference", "metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": kind, "data": "synthetic",
            "config": {"workload": workload_name, "M": M, "N": N, "K": K, "sample": sample},
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": ref["threads"], "kind": ref["kind"], "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------- main

class GatherMismatch(Exception):
    """The fused GEMM + all-gather left a block in some rank's output that differs from GEMM + NCCL all-gather."""


def compact_decode(dec: list) -> dict:
    """The decode sweep in a few numbers per shape: [N, K, us per GEMM, GB/s, fraction of the measured HBM rate, us with the weights in L2]."""
    worst = min(dec, key=lambda d: d["frac_of_measured_hbm"])
    best = max(dec, key=lambda d: d["frac_of_measured_hbm"])
    return {"M": dec[0]["M"], "columns": ["N", "K", "us", "GB/s", "frac_of_measured_hbm", "us_weights_in_l2", "split_k", "grid"],
            "shapes": [[d["N"], d["K"], d["us_per_gemm"], d["hbm_gbs"], d["frac_of_measured_hbm"], d["us_per_gemm_weights_in_l2"], d["split_k"], d["grid"]] for d in dec],
            "worst_frac": worst["frac_of_measured_hbm"], "best_frac": best["frac_of_measured_hbm"]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="nvfp4_8192x28672x8192", choices=list(WORKLOADS) + ["decode"])
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--shape", default=None, metavar="KIND,M,N,K",
                    help="time this shape instead of a named workload (kind: nvfp4, fp8, f16, bf16, w4a16_bf16, w4a16_f16), e.g. f16,512,12288,4096")
    ap.add_argument("--decode-kind", default="nvfp4", choices=["nvfp4", "fp8", "w4a16_bf16", "w4a16_f16"],
                    help="operand kind of --workload decode (the reference's decode configuration is nvfp4)")
    ap.add_argument("--no-others", action="store_true", help="skip the secondary workloads (decode, comparator, others)")
    ap.add_argument("--comparator", action="store_true", help="with --no-others: still time cuBLASLt's scaled matmul on the main workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--sustained-seconds", type=float, default=1.5, help="length of the back-to-back region (0 = skip)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    name = args.workload
    if args.shape:
        k_, m_, n_, kk_ = args.shape.split(",")
        name = "%s_%sx%sx%s" % (k_, m_, n_, kk_)
        WORKLOADS[name] = (k_, int(m_), int(n_), int(kk_))
        args.workload = name
    if name == "decode":
        kind, M, N, K = "nvfp4", 16, 22016, 4096
    else:
        kind, M, N, K = WORKLOADS[name]
    if args.impl == "reference":
        return reference_arm(args, kind, M, N, K, name)

    import torch
    import torch.distributed as dist
    from blaze_b200 import _native
    _native.lib()                                                        # fails loudly when the CUDA library is missing
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    barrier = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() in ("VERSION", "WARN"):
            os.environ.pop("NCCL_DEBUG")               # these levels print NCCL's version banner to stdout: one JSON line only
        dist.init_process_group("nccl", device_id=device)
        barrier = lambda: dist.barrier(device_ids=[local])
    peaks = measured_peaks()
    flusher = L2Flusher(device)

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if name == "decode":
        with ClockSampler(local) as clk:
            dec = run_decode(device, args.steps, args.warmup, peaks, kind=args.decode_kind)
        best = max(dec, key=lambda d: d["hbm_gbs"])
        traffic, prov = ncu_traffic("decode_%dx%d" % (best["N"], best["K"]), None) if args.decode_kind == "nvfp4" else (None, {})
        line = {"metric": "%s_decode_hbm_gbs" % args.decode_kind, "value": best["hbm_gbs"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": best["us_per_gemm"] / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.decode_kind,
                "data": "synthetic", "config": {"workload": "%s decode M=16, Llama-7B projections" % args.decode_kind, "l2": "weight copies > 2x L2 cycled in one CUDA graph"},
                "roofline": {"bound": "hbm", "achieved": best["hbm_gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": best["hbm_gbs"] / peaks["hbm_gbs"],
                             "traffic": traffic, "traffic_source": prov, "peak_source": peaks["source"]},
                "decode": compact_decode(dec), "clocks": clk.summary(), "gpu_launches": sum(d["launches"] for d in dec)}
        print(json.dumps(line))
        return 0

    # ---- main workload; at world > 1 every rank owns N/world output columns (rows of the K-major weights)
    assert N % world == 0
    n_local = N // world
    with ClockSampler(local) as clk:
        res = run_gemm_workload(kind, M, n_local, K, device, args.steps, args.warmup, flusher, barrier=barrier, variant=args.variant,
                                seed_b=123 + 1000 * rank)
    ms_local = res["ms"]
    ms = max_over_ranks(ms_local)
    launches = args.steps * res["info"]["launches"]
    mult = PEAK_MULT_OVER_BF16[kind]

    sustained = None
    if args.sustained_seconds > 0:
        if barrier:
            barrier()
        sustained, n_s = run_sustained(res["plan"], res["C"], 2.0 * M * n_local * K, args.sustained_seconds, local, peaks, mult)
        launches += n_s
        s_ms = max_over_ranks(sustained["ms_per_step"])
        sustained["ms_per_step"] = s_ms
        sustained["tflops"] = 2.0 * M * N * K / (s_ms * 1e-3) / 1e12
        sustained["frac_of_measured_sustained"] = sustained["tflops"] / world / (peaks["bf16_tflops_sustained"] * mult)

    gather = None
    if world > 1:
        # optional exchange step, timed beside the GEMM, through the library's sharded plan (blz_sharded_plan_*):
        # its own NCCL all-gather of the bf16 output, result layout [world][M][N/world]
        from blaze_b200 import sharded
        skw = dict(res["kw"]); skw["out_dtype"] = "bf16"
        full = torch.empty((world * M, n_local), dtype=res["C"].dtype, device=device)
        sp_nccl = sharded.ShardedPlan(kind, M, N, K, res["A"], res["B"], exchange="nccl", **skw)

        def step_gather():
            sp_nccl.execute(full)
        g_ms, _ = time_steps(step_gather, max(5, args.steps // 3), 3, flusher, barrier)
        sp_nccl.check()
        g_ms = max_over_ranks(g_ms)
        gather = {"ms_per_step_gemm_plus_allgather": g_ms, "tflops": 2.0 * M * N * K / (g_ms * 1e-3) / 1e12,
                  "allgather_bytes_received_per_rank": (world - 1) * M * n_local * 2, "layout": "[world][M][N/world] bf16",
                  "through": "blz_sharded_plan, BLZ_EXCHANGE_NCCL (the library's own communicator)"}
        # the same exchange fused into the GEMM: every epilogue stores its tiles into every rank's
        # full-width output (TMA stores to peer memory over NVLink), then the ranks meet at a
        # one-element all-reduce; result layout [M][N] row-major on every rank
        try:
            sp_peer = sharded.ShardedPlan(kind, M, N, K, res["A"], res["B"], exchange="peer_stores", **skw)
            sp_peer.output.fill_(-7.0)                    # a block that never arrives stays visible
            torch.cuda.synchronize()
            barrier()
            flag = torch.zeros(1, dtype=torch.float32, device=device)

            def step_fused():
                sp_peer.execute()
                dist.all_reduce(flag)
            f_ms, _ = time_steps(step_fused, max(5, args.steps // 3), 3, flusher, barrier)
            sp_peer.check()
            f_ms = max_over_ranks(f_ms)
            # Every block of the full-width output -- the one this rank wrote and the ones its peers stored over
            # NVLink -- must equal what the local GEMMs plus the NCCL all-gather give (the ranks hold
            # different weights, so a misplaced or stale block cannot pass).
            step_gather()
            torch.cuda.synchronize()
            barrier()
            want = sharded.gathered_to_full(full.view(world, M, n_local))
            res["plan"].execute(res["C"])
            torch.cuda.synchronize()
            same_local = bool(torch.equal(sp_peer.output[:, rank * n_local:(rank + 1) * n_local], res["C"]))
            same_all = bool(torch.equal(sp_peer.output, want))
            del want
            t = torch.tensor([1.0 if same_all else 0.0], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            same_all_ranks = bool(t.item() == 1.0)
            gather["fused"] = {"ms_per_step_gemm_with_peer_stores": f_ms, "tflops": 2.0 * M * N * K / (f_ms * 1e-3) / 1e12,
                               "nvlink_bytes_sent_per_rank": (world - 1) * M * n_local * 2, "layout": "[M][N] row-major on every rank",
                               "through": "blz_sharded_plan, BLZ_EXCHANGE_PEER_STORES",
                               "local_block_matches": same_local, "all_blocks_match": same_all_ranks}
            barrier()
            sp_peer.destroy()
            if not same_all_ranks:
                raise GatherMismatch("fused GEMM + all-gather: the full-width output differs from GEMM + NCCL all-gather on some rank")
        except GatherMismatch:
            raise
        except Exception as ex:   # an unavailable exchange variant is reported beside the headline, never instead of it
            gather["fused"] = {"error": str(ex)[:300]}
        barrier()
        sp_nccl.destroy()
        del full
    flops_total = 2.0 * M * N * K
    value = flops_total / (ms * 1e-3) / 1e12

    # roofline of the dominant (only) kernel, per launch on this rank
    flops_launch = 2.0 * M * n_local * K
    achieved = flops_launch / (ms_local * 1e-3) / 1e12
    peak = peaks["bf16_tflops"] * mult
    plan_key = {k: res["info"][k] for k in ("variant", "tile_m", "tile_n", "stages", "split_k")}
    traffic, prov = ncu_traffic(name, plan_key) if world == 1 else (None, {"source": "shard sizes were not captured"})
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic, "traffic_source": prov,
                "peak_source": "%s dense bf16 burst (%.1f TFLOP/s) x %g, the nominal %s : bf16 ratio" % (peaks["source"], peaks["bf16_tflops"], mult, kind),
                "frac_of_nominal_peak": achieved / NOMINAL_TFLOPS[kind], "nominal_peak": NOMINAL_TFLOPS[kind],
                "algorithmic_flops_per_launch": flops_launch,
                "algorithmic_bytes_per_launch": res["op_bytes"] + res["out_bytes"],
                "hbm_gbs_at_this_rate": (res["op_bytes"] + res["out_bytes"]) / (ms_local * 1e-3) / 1e9}

    e2e_ms, h2d, d2h, _, e2e_chunks, e2e_wall = run_e2e(res, max(3, min(args.steps, 10)), device, kind=kind, shape=(M, n_local, K), world=world, rank=rank)
    e2e_ms = max_over_ranks(e2e_ms)
    e2e = {"value": flops_total / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": e2e_ms, "host_clock_ms_per_step": e2e_wall, "row_blocks": e2e_chunks,
           "note": "pinned host activations in, whole bf16 output back to pinned host memory, every step; weights resident; "
                   "within a step the copy back of one row block overlaps the copy in and the GEMM of the next, steps do not overlap"
                   + ("; each rank copies in 1/%d of the activations and the ranks all-gather them over NVLink (NCCL) before the first row block" % world if world > 1 else "")}

    line = {"metric": "gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": kind, "data": "synthetic",
            "config": {"workload": name, "kind": kind, "M": M, "N": N, "K": K, "out": "bf16", "accumulate": "fp32",
                       "sharding": "weights split by output columns, %d per rank; activations replicated" % n_local,
                       "l2": "256 MiB write between timed steps", "timing": "CUDA events per step on the launching stream, max over ranks",
                       "kernel": res["info"]},
            "roofline": roofline, "e2e": e2e, "clocks": clk.summary()}
    if sustained:
        line["sustained"] = sustained
    if gather:
        line["gather"] = gather

    if rank == 0 and world == 1 and args.no_others and args.comparator:
        line["comparator"] = {name: run_comparator(kind, M, N, K, device, min(args.steps, 20), flusher)}
    if rank == 0 and world == 1 and not args.no_others:
        # the second half of the metric: decode HBM GB/s on the M = 16 projections (NVFP4), compact
        try:
            dec = run_decode(device, 20, 50, peaks, kind="nvfp4")     # after the sustained leg: enough replays for the clocks to settle
            line["decode"] = compact_decode(dec)
            launches += sum(d["launches"] for d in dec)
        except Exception as ex:
            line["decode"] = {"error": str(ex)[:200]}
        # cuBLASLt's scaled matmuls on the same box: what "the peak" is worth for these dtypes in practice
        comp = {}
        for w in (name, "nvfp4_4096x12288x4096", "fp8_4096"):
            k2, m2, n2, kk2 = WORKLOADS[w]
            comp[w] = run_comparator(k2, m2, n2, kk2, device, min(args.steps, 20), flusher)
            launches += 23 if "ours_ms" in comp[w] else 0
        line["comparator"] = comp
        if "cublaslt_tflops" in comp.get(name, {}):
            roofline["cublaslt_tflops_same_box"] = comp[name]["cublaslt_tflops"]
            roofline["frac_of_cublaslt"] = achieved / comp[name]["cublaslt_tflops"]
        others = {}
        # the W4A16 prefill shape twice: weights declared static (16-bit copy made once at plan creation, the serving
        # case) and the default (packed weights expanded inside the kernel, no copy)
        for w in ("fp8_4096", "w4a16_4096x22016x4096", "w4a16_4096x22016x4096:in_kernel_expansion", "nvfp4_4096x12288x4096", "nvfp4_4096x22016x4096",
                  "bf16_8192", "fp16_256"):
            k2, m2, n2, kk2 = WORKLOADS[w.split(":")[0]]
            pkw = {"static_weights": True} if w == "w4a16_4096x22016x4096" else {}
            try:
                r2 = run_gemm_workload(k2, m2, n2, kk2, device, min(args.steps, 20), 3, flusher, out_dtype="f32" if w == "fp16_256" else "bf16", **pkw)
                tf = r2["flops"] / (r2["ms"] * 1e-3) / 1e12
                i2 = r2["info"]
                others[w] = {"ms": round(r2["ms"], 5), "tflops": round(tf, 1), "frac_of_nominal_peak": round(tf / NOMINAL_TFLOPS[k2], 4),
                             "frac_of_measured_bf16_scaled": round(tf / (peaks["bf16_tflops"] * PEAK_MULT_OVER_BF16[k2]), 4),
                             "tile": "%dx%d" % (i2["tile_m"], i2["tile_n"]), "grid": i2["grid"], "launches_per_execute": i2["launches"]}
                launches += min(args.steps, 20) * r2["info"]["launches"]
                r2["plan"].destroy()
                del r2
                torch.cuda.empty_cache()
            except Exception as ex:   # a secondary workload must not lose the headline line
                others[w] = {"error": str(ex)[:200]}
        for dk in ("fp8", "w4a16_bf16"):
            try:
                d2 = run_decode(device, 5, 3, peaks, kind=dk)
                others["%s_decode_M16" % dk] = compact_decode(d2)["shapes"]
                launches += sum(d["launches"] for d in d2)
            except Exception as ex:
                others["%s_decode_M16" % dk] = {"error": str(ex)[:200]}
        for m2 in (16, 512, 2048):
            try:
                gu = run_gate_up(m2, 11008, 4096, device, 10, 3, flusher)
                launches += gu.pop("launches")
                gu.pop("kernel", None)
                others["w4a16_bf16_gate_up_M%d" % m2] = {k: (round(v, 5) if isinstance(v, float) else v) for k, v in gu.items()}
                torch.cuda.empty_cache()
            except Exception as ex:
                others["w4a16_bf16_gate_up_M%d" % m2] = {"error": str(ex)[:200]}
        line["others"] = others
    line["gpu_launches"] = launches

    if rank == 0 and world == 1 and not args.no_cpu:
        ref = cpu_reference_gemm(kind, M, N, K, 12.0)
        sec = ref["run"](ref["rows"])
        cpu_tf = 2.0 * ref["rows"] * ref["n_slice"] * K / sec / 1e12
        line["cpu_baseline"] = {"value": cpu_tf, "unit": "TFLOP/s", "cores": ref["threads"], "kind": ref["kind"],
                                "sample": "%d rows x %d columns x K=%d slice, %.1f s" % (ref["rows"], ref["n_slice"], K, sec)}
    elif rank == 0:
        line["cpu_baseline"] = None

    res["plan"].destroy()
    if world > 1:
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
