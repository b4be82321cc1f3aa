#!/usr/bin/env python
"""Benchmark of the MXFP / minifloat fake-quantisation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (one JSON line on stdout, printed by rank 0): minifloat quantize_dequantize, E5M2,
fp32 [8192, 8192] per GPU with the value distribution of benchmark configuration 2 (seeded
synthetic data), reported as algorithmic GB/s (8 bytes per element) summed over all GPUs.
One "step" is one pass of the fused kernel over the whole tensor.  Input (256 MiB) plus output
(256 MiB) exceed the 126 MB L2, so every step streams from HBM.

Extra keys: `roofline` (achieved GB/s of the kernel against the measured HBM copy peak), `e2e`
(same metric through the host-buffer pipeline, copies inside the timed region), `cpu_baseline`
(the C oracle on the host cores), `clocks`, `gpu_launches`, and `extras` with the other
configurations (MXFP extract / compose at configurations 1 and 3).

`--impl reference` times the CPU restatement of the reference's path (the oracle) with all host
threads on the same configuration.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "minifloat_quantize_dequantize_GBps"
UNIT = "GB/s"
SHAPE = (8192, 8192)
BYTES_PER_ELT = 8                      # fp32 in + fp32 out
# DRAM bytes per element of the headline kernel from one ncu capture: 134.24 MB read + 81.93 MB written
# (mean of two launches) over 33 554 432 elements (the rest of the output is still in L2 when the kernel ends)
NCU_TRAFFIC_BYTES_PER_ELT = (134.242048e6 + 81.931264e6) / 33554432
WORKLOAD = "cfg2: minifloat quantize_dequantize E5M2 (rn, is_finite) fp32 [8192,8192] per GPU"


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_tensor_peak() -> float:
    """Measured cuBLAS bf16 burst TFLOP/s of this pool's B200 (driver-written), else the fallback 1590."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["bf16_tflops"])
        except Exception:
            pass
    return 1590.0


def library_mx_gemm_bar(M: int, N: int, K: int, dev, reps: int, flops: float) -> dict:
    """The library's own block-scaled MXFP8 GEMM (torch._scaled_mm with E8M0 scales on operands of the same
    shape) timed the same way, as a bar for the hand-written kernel.  Comparison only: no product path calls it.
    Unit scales and random codes: the time of a GEMM does not depend on the values."""
    try:
        e8 = getattr(torch, "float8_e8m0fnu")
        a = torch.randint(0, 120, (M, K), device=dev, dtype=torch.uint8).view(torch.float8_e4m3fn)
        b = torch.randint(0, 120, (N, K), device=dev, dtype=torch.uint8).view(torch.float8_e4m3fn)
        ru = lambda v, m: (v + m - 1) // m * m      # noqa: E731
        sa = torch.full((ru(M, 128) * ru(K // 32, 4),), 127, device=dev, dtype=torch.uint8).view(e8)
        sb = torch.full((ru(N, 128) * ru(K // 32, 4),), 127, device=dev, dtype=torch.uint8).view(e8)
        fn = lambda: torch._scaled_mm(a, b.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)     # noqa: E731
        fn()
        torch.cuda.synchronize()
        t = graph_time(fn, reps, rounds=9)
        return {"TFLOPs": round(flops / t / 1e9, 1), "ms": round(t, 4), "what": "torch._scaled_mm, float8_e4m3fn x float8_e4m3fn, float8_e8m0fnu block-32 scales, bf16 out"}
    except Exception as exc:      # noqa: BLE001 - a missing library kernel must not hide our own numbers
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


class ClockSampler:
    """Samples SM clock / throttle reasons of one GPU with NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples: list[tuple[float, int, int]] = []
        self.sm_max = None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=2)

    def summary(self, t0: float, t1: float) -> dict:
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-3:]
        names = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                 0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        bits = 0
        for s in inside:
            bits |= s[2]
        reasons = [n for b, n in names.items() if bits & b and n != "gpu_idle"]
        return {"sm_mhz": statistics.median(s[1] for s in inside) if inside else None, "sm_max_mhz": self.sm_max,
                "reasons": reasons, "samples": len(inside)}


def dist_setup(n_gpus: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")     # keep stdout for the one JSON line
        import datetime
        torch.cuda.set_device(local)
        # a rank that fails alone must not leave the others waiting in a collective for long
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(minutes=4))
        return dist, rank, world, local
    return None, 0, 1, 0


def cpu_baseline(sample_rows: int = 8192, reps: int = 3) -> dict:
    """The C oracle (all host threads) on the same workload; median of `reps` passes."""
    import oracle
    from mase_triton_b200 import synthetic
    from types import SimpleNamespace
    meta = SimpleNamespace(exp_bits=5, frac_bits=2, is_finite=True, round_mode="rn")
    oracle.set_num_threads(os.cpu_count() or 1)
    x = synthetic.cfg2_minifloat_fp32(rows=slice(0, sample_rows))
    oracle.quantize_dequantize_minifloat(x[:64], meta)
    ts = []
    for _ in range(reps):
        t = time.perf_counter()
        oracle.quantize_dequantize_minifloat(x, meta)
        ts.append(time.perf_counter() - t)
    t = statistics.median(ts)
    return {"value": round(x.numel() * BYTES_PER_ELT / t / 1e9, 3), "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{sample_rows}x{x.shape[1]} fp32 rows of the workload, median of {reps} passes of the C oracle ({t * 1e3:.1f} ms each)"}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from mase_triton_b200 import synthetic
    from types import SimpleNamespace
    meta = SimpleNamespace(exp_bits=5, frac_bits=2, is_finite=True, round_mode="rn")
    oracle.set_num_threads(os.cpu_count() or 1)        # torchrun exports OMP_NUM_THREADS=1
    x = synthetic.cfg2_minifloat_fp32()
    for _ in range(max(1, args.warmup)):
        oracle.quantize_dequantize_minifloat(x[:1024], meta)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.quantize_dequantize_minifloat(x, meta)
    dt = (time.perf_counter() - t0) / args.steps
    v = round(x.numel() * BYTES_PER_ELT / dt / 1e9, 3)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU restatement of the reference's PyTorch path (C oracle, OpenMP); one tensor, host cores only"},
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                             "sample": "each step is one full [8192,8192] pass"},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def time_steps(fn, steps: int, stream=None) -> list[float]:
    """Per-step device times in ms, CUDA events on the launching stream."""
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record()
    for i in range(steps):
        fn()
        ev[i + 1].record()
    torch.cuda.synchronize()
    return [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]


GRAPH_FALLBACKS: list[str] = []      # captures that failed and were timed launch by launch instead (reported in the line)


def graph_time(fn, reps: int, rounds: int = 5) -> float:
    """Median device time (ms) of one call of `fn`, measured by replaying a CUDA graph of `reps`
    back-to-back calls: no host launch overhead between kernels, so short kernels are timed honestly."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    try:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(rounds):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / reps)
        return statistics.median(ts)
    except Exception as exc:      # noqa: BLE001
        GRAPH_FALLBACKS.append(f"{type(exc).__name__}: {exc}"[:200])
        torch.cuda.synchronize()
        return statistics.median(time_steps(fn, reps))


def graph_time_interleaved(fns: dict, reps: int, rounds: int = 7) -> dict:
    """`graph_time` for several callables at once: one CUDA graph of `reps` calls each, replayed in turn for `rounds`
    rounds, median per callable.  What ran just before (clocks under the power cap, what is left in L2) then weighs on
    all of them alike instead of on whichever is measured last."""
    graphs = {}
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for fn in fns.values():
            for _ in range(3):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    try:
        for name, fn in fns.items():
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(reps):
                    fn()
            g.replay()
            graphs[name] = g
        torch.cuda.synchronize()
        ts = {name: [] for name in fns}
        for _ in range(rounds):
            for name, g in graphs.items():
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts[name].append(e0.elapsed_time(e1) / reps)
        return {name: statistics.median(v) for name, v in ts.items()}
    except Exception as exc:      # noqa: BLE001
        GRAPH_FALLBACKS.append(f"{type(exc).__name__}: {exc}"[:200])
        torch.cuda.synchronize()
        return {name: statistics.median(time_steps(fn, reps)) for name, fn in fns.items()}


def extras_single_gpu(dev, steps: int, warmup: int, peak: float) -> dict:
    """MXFP extract / compose on configurations 1 and 3, and the MX GEMM / linear on configurations
    4 and 5 (device-resident; CUDA-graph replays so that host launch gaps are not part of the time)."""
    from mase_triton_b200 import synthetic
    from mase_triton_b200.mxfp import gemm as G
    from mase_triton_b200.mxfp import kernels as mxk
    from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
    from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, OCP_MXFP4_E2M1, OCP_MXFP6_E3M2
    out = {}
    reps = max(4, min(steps, 20))
    for name, gen, meta, s_in, nsets in (("cfg1_mxfp8_fp32_4096x4096", synthetic.cfg1_mxfp8_fp32, MXFP8_E4M3_fn, 4, 4),
                                         ("cfg3_mxfp4_bf16_16384x8192", synthetic.cfg3_mxfp4_bf16, OCP_MXFP4_E2M1, 2, 1)):
        x = gen().to(dev).flatten()
        xs = [x] + [x.clone() for _ in range(nsets - 1)]      # rotate buffers so small tensors cannot sit in L2
        n = x.numel()
        i = [0]

        def ext():
            i[0] += 1
            return mxk.extract_mxfp_components(xs[i[0] % nsets], meta)
        t_ext = graph_time(ext, reps * nsets)
        se = [mxk.extract_mxfp_components(v, meta) for v in xs]

        def comp():
            i[0] += 1
            s, e = se[i[0] % nsets]
            return mxk.compose_mxfp_tensor(s, e, meta, x.dtype)
        t_cmp = graph_time(comp, reps * nsets)

        def qdq():
            i[0] += 1
            return mxk.quantize_dequantize(xs[i[0] % nsets], meta, x.dtype)
        t_qdq = graph_time(qdq, reps * nsets)
        b_ext = n * (s_in + 1 + 1 / 32)
        b_cmp = n * (1 + 1 / 32 + s_in)
        out[name] = {
            "extract_GBps": round(b_ext / t_ext / 1e6, 1), "extract_frac_of_peak": round(b_ext / t_ext / 1e6 / peak, 3),
            "compose_GBps": round(b_cmp / t_cmp / 1e6, 1), "compose_frac_of_peak": round(b_cmp / t_cmp / 1e6 / peak, 3),
            "extract_plus_compose_GBps": round((b_ext + b_cmp) / (t_ext + t_cmp) / 1e6, 1),
            "extract_plus_compose_frac_of_peak": round((b_ext + b_cmp) / (t_ext + t_cmp) / 1e6 / peak, 3),
            "fused_qdq_GBps": round(n * 2 * s_in / t_qdq / 1e6, 1),
            "ms": {"extract": round(t_ext, 4), "compose": round(t_cmp, 4), "fused_qdq": round(t_qdq, 4)},
            "buffer_sets_rotated": nsets, "timing": "CUDA graph replay",
        }
        del xs, se, x
        torch.cuda.empty_cache()

    # configuration 4: x bf16 [8192,4096], W [14336,4096], MXFP8 E4M3 both, bf16 out
    xc, wc = synthetic.cfg4_linear_operands()
    xc, wc = xc.to(dev), wc.to(dev)
    M, K = xc.shape
    N = wc.shape[0]
    flops = 2.0 * M * N * K
    a, b = G.quantize_pack(xc, MXFP8_E4M3_fn), G.quantize_pack(wc, MXFP8_E4M3_fn, G.OPERAND_B)
    o = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    gemm_clock = ClockSampler(dev.index or 0, period_s=0.002)
    gemm_clock.start()
    tg0 = time.perf_counter()
    t_gemm = graph_time(lambda: G.mx_gemm(a, b, torch.bfloat16, out=o), max(reps, 20), rounds=9)
    tg1 = time.perf_counter()
    gemm_clock.stop()
    fc = torch.nn.Linear(K, N, bias=False, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        fc.weight.copy_(wc)
    fused = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, MXFP8_E4M3_fn, None, "XqWqB", "fused")
    sep = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, MXFP8_E4M3_fn, None, "XqWqB", "separate")
    # the kernel, the fused layer and the separate layer once more in turn (graphs replayed round-robin): a time moves by
    # several per cent with what ran just before it.  The kernel keeps the better of its two medians; both are reported.
    t_gemm_first = t_gemm
    turn = graph_time_interleaved({"gemm": lambda: G.mx_gemm(a, b, torch.bfloat16, out=o), "fused": lambda: fused(xc),
                                   "separate": lambda: sep(xc)}, max(5, reps // 2))
    t_gemm_again, t_fused, t_sep = turn["gemm"], turn["fused"], turn["separate"]
    t_gemm = min(t_gemm_first, t_gemm_again)
    G.check_status(dev)
    rel = ((fused(xc).float() - sep(xc).float()).abs().mean() / sep(xc).float().abs().mean()).item()
    bf16_peak = measured_tensor_peak()
    out["cfg4_mxfp_linear_8192x14336x4096"] = {
        "gemm_kernel_TFLOPs": round(flops / t_gemm / 1e9, 1), "fused_linear_TFLOPs": round(flops / t_fused / 1e9, 1),
        "separate_linear_TFLOPs_reference_style_cublas_bf16": round(flops / t_sep / 1e9, 1),
        "gemm_frac_of_4500_nominal_mx": round(flops / t_gemm / 1e9 / 4500, 3),
        "ms": {"gemm": round(t_gemm, 4), "gemm_two_measurements": [round(t_gemm_first, 4), round(t_gemm_again, 4)],
               "fused_linear": round(t_fused, 4), "separate_linear": round(t_sep, 4)},
        "mean_rel_diff_fused_vs_separate": round(rel, 8),
        # roofline of the tensor-core kernel: 2*M*N*K flops per launch over its CUDA-graph-replay time
        "roofline": {"bound": "tensor", "achieved": round(flops / t_gemm / 1e9, 1), "unit": "TFLOP/s", "peak": 4500.0,
                     "frac": round(flops / t_gemm / 1e9 / 4500, 4), "peak_source": "nominal dense MXFP8 (no measured MX peak on file)",
                     "peak_2x_measured_bf16_burst": round(2 * bf16_peak, 1), "frac_of_2x_measured_bf16_burst": round(flops / t_gemm / 1e9 / (2 * bf16_peak), 4),
                     "kernel": "mx_gemm_kernel<bf16, MH=2>", "launch_ms": round(t_gemm, 5), "flops_per_launch": flops,
                     "clocks_during_gemm": gemm_clock.summary(tg0, tg1)},
    }
    out["cfg4_mxfp_linear_8192x14336x4096"]["library_bar_scaled_mm_mxfp8"] = library_mx_gemm_bar(M, N, K, dev, max(reps, 20), flops)
    # the other layer types on the kind::f16 GEMM (weight codes expanded in the operand loader; dense operands)
    from mase_triton_b200 import tc_linear
    wq_f = MXFPLinearPTQ.from_linear(fc, None, MXFP8_E4M3_fn, None, "XWqB", "fused")
    wq_s = MXFPLinearPTQ.from_linear(fc, None, MXFP8_E4M3_fn, None, "XWqB", "separate")
    xq_f = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, None, None, "XqWB", "fused")
    xq_s = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, None, None, "XqWB", "separate")
    t = {"XWq_fused": graph_time(lambda: wq_f(xc), reps), "XWq_separate": graph_time(lambda: wq_s(xc), max(3, reps // 2)),
         "XqW_fused": graph_time(lambda: xq_f(xc), reps), "XqW_separate": graph_time(lambda: xq_s(xc), max(3, reps // 2)),
         "XWq_codes_expanded_in_the_loader": graph_time(
             lambda: tc_linear.mxfp_weight_linear(xc, wq_f.w_scales, wq_f.w_elements, (N, K), MXFP8_E4M3_fn), reps),
         "dense_gemm": graph_time(lambda: tc_linear.dense_linear(xc, wc), reps),
         "library_dense_gemm": graph_time(lambda: torch.nn.functional.linear(xc, wc), reps)}
    x_short = xc[:512].contiguous()
    t_short = {"XWq_fused": graph_time(lambda: wq_f(x_short), reps * 4), "XWq_separate": graph_time(lambda: wq_s(x_short), reps * 4)}
    G.check_status(dev)
    rel_wq = ((wq_f(xc).float() - wq_s(xc).float()).abs().mean() / wq_s(xc).float().abs().mean()).item()
    out["cfg4_shape_mixed_layer_types_kind_f16_gemm"] = {
        "TFLOPs": {k: round(flops / v / 1e9, 1) for k, v in t.items()}, "ms": {k: round(v, 4) for k, v in t.items()},
        "mean_rel_diff_XWq_fused_vs_separate": round(rel_wq, 8),
        "short_activation_512_rows_ms": {k: round(v, 4) for k, v in t_short.items()},
        "XWq_route": "512 rows: codes expanded in the GEMM's loader; 8192 rows: expanded once by the compose kernel, same GEMM on dense operands",
        "frac_of_measured_bf16_burst": {k: round(flops / v / 1e9 / bf16_peak, 3) for k, v in t.items()},
        "note": "fused = this library's tcgen05 kind::f16 GEMM (256x256 tiles); separate = dequantise kernels + torch.nn.functional.linear"}
    # the same shape with MXFP4 activation and weight: both stay packed nibbles, tcgen05 kind::mxf4 (64 elements of K per instruction)
    a4 = G.quantize_pack(xc, OCP_MXFP4_E2M1, G.OPERAND_A, native=True)
    b4 = G.quantize_pack(wc, OCP_MXFP4_E2M1, G.OPERAND_B, native=True)
    a48, b48 = G.quantize_pack(xc, OCP_MXFP4_E2M1), G.quantize_pack(wc, OCP_MXFP4_E2M1, G.OPERAND_B)
    f4 = MXFPLinearPTQ.from_linear(fc, OCP_MXFP4_E2M1, OCP_MXFP4_E2M1, None, "XqWqB", "fused")
    s4 = MXFPLinearPTQ.from_linear(fc, OCP_MXFP4_E2M1, OCP_MXFP4_E2M1, None, "XqWqB", "separate")
    same4 = bool(torch.equal(G.mx_gemm(a4, b4, torch.bfloat16), G.mx_gemm(a48, b48, torch.bfloat16)))
    t4 = {"gemm_packed_nibbles_kind_mxf4": graph_time(lambda: G.mx_gemm(a4, b4, torch.bfloat16, out=o), max(reps, 20), rounds=9),
          "gemm_codes_widened_to_bytes_kind_mxf8f6f4": graph_time(lambda: G.mx_gemm(a48, b48, torch.bfloat16, out=o), max(reps, 20)),
          "fused_linear": graph_time(lambda: f4(xc), reps), "separate_linear": graph_time(lambda: s4(xc), max(3, reps // 2))}
    G.check_status(dev)
    out["cfg4_shape_mxfp4_x_mxfp4"] = {
        "TFLOPs": {k: round(flops / v / 1e9, 1) for k, v in t4.items()}, "ms": {k: round(v, 4) for k, v in t4.items()},
        "gemm_frac_of_9000_nominal_fp4": round(flops / t4["gemm_packed_nibbles_kind_mxf4"] / 1e9 / 9000, 3),
        "packed_nibble_gemm_equals_widened_gemm_bit_for_bit": same4,
        "note": "fused linear = one-pass quantise + nibble pack of the activation, then the kind::mxf4 GEMM"}
    del a4, b4, a48, b48, f4, s4
    del fc, fused, sep, wq_f, wq_s, xq_f, xq_s, a, b, o, xc, wc, x_short
    torch.cuda.empty_cache()

    # configuration 5: seven projections of one Llama-3-8B-shaped layer, W MXFP6 E3M2, x MXFP8 E4M3, 16x2048 tokens.
    # "independent": every projection is one public forward call (activation quantised inside every call);
    # "shared activation": q/k/v and gate/up quantise their common input once (pack_input + forward_packed).
    sweep, tot_flops, tot_ms = {}, 0.0, 0.0
    layers, inputs = {}, {}
    for pname, n_out, n_in in synthetic.CFG5_PROJECTIONS:
        w = synthetic.cfg5_weight(pname).to(dev)
        if n_in not in inputs:
            inputs[n_in] = synthetic.cfg5_input(n_in).to(dev)
        fc = torch.nn.Linear(n_in, n_out, bias=False, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            fc.weight.copy_(w)
        layers[pname] = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, OCP_MXFP6_E3M2, None, "XqWqB", "fused")
        del fc, w
    for pname, n_out, n_in in synthetic.CFG5_PROJECTIONS:
        x5, layer = inputs[n_in], layers[pname]
        t = graph_time(lambda: layer(x5), max(3, reps // 2))
        fl = 2.0 * x5.shape[0] * x5.shape[1] * n_in * n_out
        sweep[pname] = {"ms": round(t, 4), "TFLOPs": round(fl / t / 1e9, 1)}
        tot_flops += fl
        tot_ms += t
    G.check_status(dev)
    sweep["sweep_TFLOPs"] = round(tot_flops / tot_ms / 1e9, 1)
    sweep["sweep_ms"] = round(tot_ms, 4)
    shared_ms = 0.0
    groups = {}
    for gname, members in (("qkv", ("q", "k", "v")), ("o", ("o",)), ("gate_up", ("gate", "up")), ("down", ("down",))):
        x5 = inputs[layers[members[0]].in_features]
        lead = tuple(x5.shape[:-1])

        def run_group(ms=members, x5=x5, lead=lead):
            packed = layers[ms[0]].pack_input(x5)
            return [layers[m].forward_packed(packed, torch.bfloat16, lead_shape=lead) for m in ms]
        t = graph_time(run_group, max(3, reps // 2))
        for m, y in zip(members, run_group()):
            assert torch.equal(y, layers[m](x5)), f"shared-activation result of {m} differs from forward()"
        fl = sum(2.0 * x5.shape[0] * x5.shape[1] * layers[m].in_features * layers[m].out_features for m in members)
        groups[gname] = {"ms": round(t, 4), "TFLOPs": round(fl / t / 1e9, 1)}
        shared_ms += t
    G.check_status(dev)
    sweep["shared_activation"] = {"groups": groups, "sweep_TFLOPs": round(tot_flops / shared_ms / 1e9, 1), "sweep_ms": round(shared_ms, 4),
                                  "frac_of_4500_nominal_mx": round(tot_flops / shared_ms / 1e9 / 4500, 3)}
    sweep["frac_of_4500_nominal_mx"] = round(tot_flops / tot_ms / 1e9 / 4500, 3)
    out["cfg5_llama3_8b_layer_fused_linear"] = sweep
    del layers, inputs
    torch.cuda.empty_cache()

    # widening rows: blocks along a non-contiguous dimension, and the minifloat linear on the tensor cores
    from mase_triton_b200.minifloat.layers import MinifloatLinearPTQ
    from mase_triton_b200.minifloat.meta import FP8_E4M3_fn
    from mase_triton_b200.mxfp.helpers import flatten_for_quantize, permute_for_dequantize
    xs2 = synthetic.cfg1_mxfp8_fp32(shape=(8192, 8192)).to(dev)
    nb = xs2.numel() * 8
    t_str = graph_time(lambda: mxk.quantize_dequantize_strided(xs2, 0, MXFP8_E4M3_fn, xs2.dtype), reps)
    t_perm = graph_time(lambda: permute_for_dequantize(mxk.quantize_dequantize(flatten_for_quantize(xs2, 0), MXFP8_E4M3_fn, xs2.dtype),
                                                       tuple(xs2.shape), 0).contiguous(), max(3, reps // 2))
    out["mxfp8_fp32_8192x8192_blocks_along_dim0_fused_qdq"] = {
        "strided_kernel_GBps": round(nb / t_str / 1e6, 1), "strided_kernel_frac_of_peak": round(nb / t_str / 1e6 / peak, 3),
        "permuted_copy_route_GBps": round(nb / t_perm / 1e6, 1), "ms": {"strided": round(t_str, 4), "permuted": round(t_perm, 4)}}
    del xs2
    torch.cuda.empty_cache()
    xc, wc = synthetic.cfg4_linear_operands()
    xc, wc = xc.to(dev), wc.to(dev)
    flops = 2.0 * xc.shape[0] * wc.shape[0] * xc.shape[1]
    fc = torch.nn.Linear(xc.shape[1], wc.shape[0], bias=False, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        fc.weight.copy_(wc)
    mf_f = MinifloatLinearPTQ.from_linear(fc, FP8_E4M3_fn, FP8_E4M3_fn, None, "XqWqB", "fused")
    mf_s = MinifloatLinearPTQ.from_linear(fc, FP8_E4M3_fn, FP8_E4M3_fn, None, "XqWqB", "separate")
    t_mf = graph_time(lambda: mf_f(xc), reps)
    t_ms = graph_time(lambda: mf_s(xc), max(3, reps // 2))
    G.check_status(dev)
    out["graph_capture_fallbacks"] = list(GRAPH_FALLBACKS)
    out["cfg4_shape_minifloat_linear_e4m3"] = {"fused_TFLOPs": round(flops / t_mf / 1e9, 1), "separate_TFLOPs": round(flops / t_ms / 1e9, 1),
                                               "ms": {"fused": round(t_mf, 4), "separate": round(t_ms, 4)}}
    return out


def extras_multi_gpu(dev, dist, rank: int, world: int, local: int, steps: int, peak: float) -> dict:
    """The sharded configurations on `world` GPUs: configuration 3 split by rows (no collective) and the linears
    of configurations 4 and 5 column-parallel by output feature, the partial outputs gathered either by NCCL or
    by the GEMM kernel itself (peer stores).  Before anything is timed every rank checks its sharded results
    against the whole problem computed on its own GPU, bit for bit.  Times are device times, max over ranks,
    taken after a barrier: CUDA-graph replay where no collective is involved, otherwise one event pair around
    `n` back-to-back calls so that a short kernel is not a measurement of launch gaps."""
    from mase_triton_b200 import parallel, synthetic
    from mase_triton_b200.mxfp import gemm as G
    from mase_triton_b200.mxfp import kernels as mxk
    from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
    from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, OCP_MXFP4_E2M1, OCP_MXFP6_E3M2
    out = {}

    def max_over_ranks(ms: float) -> float:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sync_all():
        dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    def timed_graph(fn, reps: int) -> float:
        sync_all()
        return max_over_ranks(graph_time(fn, reps))

    def timed_many(fn, n: int) -> float:
        for _ in range(3):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) / n)

    def all_ranks_agree(flag: bool, what: str) -> None:
        t = torch.tensor([0 if flag else 1], device=dev, dtype=torch.int32)
        dist.all_reduce(t)
        if int(t.item()) != 0:
            raise RuntimeError(f"{what}: {int(t.item())} rank(s) disagree with the single-GPU result")

    # ---- configuration 3: rows split evenly, no collective ----
    rows = 16384
    lo, hi = parallel.shard_bounds(rows, rank, world)
    x_full = synthetic.cfg3_mxfp4_bf16().to(dev)
    x = x_full[lo:hi].contiguous().flatten()
    s_full, e_full = mxk.extract_mxfp_components(x_full.flatten(), OCP_MXFP4_E2M1)
    s, e = mxk.extract_mxfp_components(x, OCP_MXFP4_E2M1)
    bpr = 8192 // 32
    ok = torch.equal(s, s_full[lo * bpr:hi * bpr]) and torch.equal(e, e_full[lo * bpr:hi * bpr])
    y_full = mxk.compose_mxfp_tensor(s_full, e_full, OCP_MXFP4_E2M1, torch.bfloat16)
    ok = ok and torch.equal(mxk.compose_mxfp_tensor(s, e, OCP_MXFP4_E2M1, torch.bfloat16).view(torch.int16), y_full[lo * 8192:hi * 8192].view(torch.int16))
    ok = ok and torch.equal(mxk.quantize_dequantize(x, OCP_MXFP4_E2M1, torch.bfloat16).view(torch.int16), y_full[lo * 8192:hi * 8192].view(torch.int16))
    all_ranks_agree(ok, "configuration 3 row shard")
    del x_full, s_full, e_full, y_full
    torch.cuda.empty_cache()
    n_total = rows * 8192
    reps = 40
    t_ext = timed_graph(lambda: mxk.extract_mxfp_components(x, OCP_MXFP4_E2M1), reps)
    t_cmp = timed_graph(lambda: mxk.compose_mxfp_tensor(s, e, OCP_MXFP4_E2M1, torch.bfloat16), reps)
    t_qdq = timed_graph(lambda: mxk.quantize_dequantize(x, OCP_MXFP4_E2M1, torch.bfloat16), reps)
    b = n_total * (2 + 1 + 1 / 32)
    out["cfg3_rows_sharded"] = {"extract_GBps_total": round(b / t_ext / 1e6, 1), "compose_GBps_total": round(b / t_cmp / 1e6, 1),
                                "extract_plus_compose_GBps_total": round(2 * b / (t_ext + t_cmp) / 1e6, 1),
                                "fused_qdq_GBps_total": round(n_total * 4 / t_qdq / 1e6, 1),
                                "frac_of_peak_per_gpu": {"extract": round(b / t_ext / 1e6 / peak / world, 3), "compose": round(b / t_cmp / 1e6 / peak / world, 3),
                                                         "extract_plus_compose": round(2 * b / (t_ext + t_cmp) / 1e6 / peak / world, 3),
                                                         "fused_qdq": round(n_total * 4 / t_qdq / 1e6 / peak / world, 3)},
                                "ms": {"extract": round(t_ext, 5), "compose": round(t_cmp, 5), "fused_qdq": round(t_qdq, 5)},
                                "rows_per_gpu": hi - lo, "collective": "none", "scaling": "strong (16384 rows in total)",
                                "timing": f"CUDA graph replay of {reps} launches, max over ranks", "verified": "shard results equal the slices of the whole-tensor results on every rank"}
    del x, s, e
    torch.cuda.empty_cache()

    # ---- column-parallel linears: configuration 4 and the seven projections of configuration 5 ----
    def column_parallel(name: str, x: torch.Tensor, w: torch.Tensor, x_meta, w_meta, n_calls: int, tile_rows=None) -> dict:
        n_out, n_in = w.shape
        fc = torch.nn.Linear(n_in, n_out, bias=False, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            fc.weight.copy_(w.to(dev))
        layer = MXFPLinearPTQ.from_linear(fc, x_meta, w_meta, None, "XqWqB", "fused")
        del fc
        xg = x.to(dev)
        rows_x = xg.numel() // n_in
        want = layer(xg).reshape(rows_x, n_out)                       # the whole layer on this GPU
        via_nccl = parallel.column_parallel_mxfp_linear(layer)
        fused = parallel.GatherFusedMXFPLinear(layer, max_rows=rows_x, dtype=torch.bfloat16, tile_rows=tile_rows)
        got_nccl = via_nccl(xg).reshape(rows_x, n_out).contiguous()
        got_fused = fused(xg).reshape(rows_x, n_out)
        G.check_status(dev)
        torch.cuda.synchronize()
        ok_n = torch.equal(got_nccl.view(torch.int16), want.view(torch.int16))
        ok_f = torch.equal(got_fused.view(torch.int16), want.view(torch.int16))
        all_ranks_agree(ok_n, f"{name}: NCCL-gathered output")
        all_ranks_agree(ok_f, f"{name}: gather-fused output")
        del want, got_nccl, got_fused
        fl = 2.0 * rows_x * n_in * n_out
        n0, n1 = fused.n0, fused.n1
        a = G.pack_activation(xg.reshape(rows_x, n_in), x_meta)
        o = torch.empty((rows_x, max(1, n1 - n0)), dtype=torch.bfloat16, device=dev)
        t_gemm = timed_many(lambda: G.mx_gemm(a, fused.weight, torch.bfloat16, out=o), n_calls) if n1 > n0 else 0.0
        t_kernel = timed_many(lambda: G.mx_gemm_gather(a, fused.weight, fused.ptrs[0], rank, n_out, n0, torch.bfloat16), n_calls)
        t_local = timed_many(lambda: via_nccl(xg, gather=False), n_calls)
        t_nccl = timed_many(lambda: via_nccl(xg), n_calls)
        t_fused = timed_many(lambda: fused(xg), n_calls)
        G.check_status(dev)
        egress = rows_x * (n1 - n0) * 2 * (world - 1)
        link_ms = egress / 770e9 * 1e3
        res = {"out_features_per_gpu": n1 - n0, "tile_columns": fused.weight.tile_rows or 224,
               "TFLOPs_total": {"gemm_only": round(fl / t_gemm / 1e9, 1) if t_gemm else None, "layer_without_gather": round(fl / t_local / 1e9, 1),
                                "layer_nccl_allgather": round(fl / t_nccl / 1e9, 1), "layer_gather_fused": round(fl / t_fused / 1e9, 1)},
               "ms": {"gemm_only": round(t_gemm, 4), "gather_fused_kernel_only": round(t_kernel, 4), "layer_without_gather": round(t_local, 4),
                      "layer_nccl_allgather": round(t_nccl, 4), "layer_gather_fused": round(t_fused, 4)},
               "fused_kernel_nvlink_egress_GBps_per_gpu": round(egress / t_kernel / 1e6, 1),
               "fused_kernel_frac_of_roofline": round(max(t_gemm, link_ms) / t_kernel, 3),
               "roofline_ms": {"gemm": round(t_gemm, 4), "link_at_770_GBps": round(link_ms, 4)},
               "link_note": "770 GB/s is the measured peer-copy rate; a plain copy kernel in which every rank stores to all its peers at once reached 660-680 GB/s per GPU on four GPUs",
               "verified": "NCCL-gathered and gather-fused outputs equal the single-GPU layer bit for bit on every rank",
               "timing": f"one event pair around {n_calls} back-to-back calls, max over ranks"}
        del layer, via_nccl, fused, a, o, xg
        torch.cuda.empty_cache()
        return res, fl, {"gemm_only": t_gemm, "layer_without_gather": t_local, "layer_nccl_allgather": t_nccl, "layer_gather_fused": t_fused}

    try:
        xc, wc = synthetic.cfg4_linear_operands()
        res, _, _ = column_parallel("cfg4", xc, wc, MXFP8_E4M3_fn, MXFP8_E4M3_fn, 50)
        res["collective"] = "all-gather of bf16 [M, N/g] shards: NCCL, or peer stores issued by the GEMM kernel + a one-element all-reduce as fence"
        out["cfg4_column_parallel"] = res
        # the same with 224-column tiles (no padded work for 1792 / 3584 / 7168 features per rank, but row segments of 448 bytes)
        res224, _, _ = column_parallel("cfg4 (224-column tiles)", xc, wc, MXFP8_E4M3_fn, MXFP8_E4M3_fn, 50, tile_rows=224)
        out["cfg4_column_parallel"]["with_224_column_tiles"] = {k: res224[k] for k in ("ms", "fused_kernel_nvlink_egress_GBps_per_gpu", "fused_kernel_frac_of_roofline")}
        del xc, wc
        sweep, tot_fl, tot = {}, 0.0, {}
        inputs = {}
        for pname, n_out, n_in in synthetic.CFG5_PROJECTIONS:
            if n_in not in inputs:
                inputs = {n_in: synthetic.cfg5_input(n_in)}            # one input alive at a time (the widest is 0.9 GB)
            res, fl, ts = column_parallel(f"cfg5 {pname}", inputs[n_in], synthetic.cfg5_weight(pname), MXFP8_E4M3_fn, OCP_MXFP6_E3M2, 20)
            sweep[pname] = res
            tot_fl += fl
            for k, v in ts.items():
                tot[k] = tot.get(k, 0.0) + v
        sweep["sweep_TFLOPs_total"] = {k: round(tot_fl / v / 1e9, 1) for k, v in tot.items() if v}
        sweep["sweep_ms"] = {k: round(v, 4) for k, v in tot.items()}
        out["cfg5_column_parallel"] = sweep
    except Exception as exc:   # noqa: BLE001 - reported in the line; the headline stands
        out["column_parallel_error"] = f"{type(exc).__name__}: {exc}"[:400]
    return out


def small_cases():
    """Small single-kernel cases for profiling: name -> (builder returning (launch_fn, algorithmic bytes)).
    Inputs plus outputs are larger than L2 and well under 1 GB."""
    from mase_triton_b200 import synthetic
    from mase_triton_b200.minifloat import kernels as mfk
    from mase_triton_b200.minifloat.meta import FP8_E5M2_fn
    from mase_triton_b200.mxfp import kernels as mxk
    from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, OCP_MXFP4_E2M1
    dev = torch.device("cuda", 0)

    def minifloat_qdq_f32():
        x = synthetic.cfg2_minifloat_fp32(shape=(4096, 8192)).to(dev)
        out = torch.empty_like(x)
        return (lambda: mfk.quantize_dequantize(x, FP8_E5M2_fn, torch.float32, out=out)), x.numel() * 8

    def mx_case(gen, shape, meta, s_in, which):
        x = gen(shape=shape).to(dev).flatten()
        n = x.numel()
        if which == "extract":
            return (lambda: mxk.extract_mxfp_components(x, meta)), n * (s_in + 1 + 1 / 32)
        if which == "compose":
            s, e = mxk.extract_mxfp_components(x, meta)
            return (lambda: mxk.compose_mxfp_tensor(s, e, meta, x.dtype)), n * (s_in + 1 + 1 / 32)
        out = torch.empty_like(x)
        return (lambda: mxk.quantize_dequantize(x, meta, x.dtype, out=out)), n * 2 * s_in

    def gemm_case(M, N, K, which):
        from mase_triton_b200.mxfp import gemm as G
        from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
        g = torch.Generator().manual_seed(0)
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
        w = (0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16).to(dev)
        flops = 2.0 * M * N * K
        if which == "gemm":            # tensor-core kernel alone, operands already packed
            a, b = G.quantize_pack(x, MXFP8_E4M3_fn), G.quantize_pack(w, MXFP8_E4M3_fn, G.OPERAND_B)
            out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            return (lambda: G.mx_gemm(a, b, torch.bfloat16, out=out)), flops
        if which == "gemm4":           # MXFP4 x MXFP4, both operands packed nibbles: the kind::mxf4 form of the kernel
            a, b = G.quantize_pack(x, OCP_MXFP4_E2M1, G.OPERAND_A, native=True), G.quantize_pack(w, OCP_MXFP4_E2M1, G.OPERAND_B, native=True)
            out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            return (lambda: G.mx_gemm(a, b, torch.bfloat16, out=out)), flops
        if which == "gather_local":     # the gather-fused kernel with two destinations on this GPU (no NVLink involved)
            a, b = G.quantize_pack(x, MXFP8_E4M3_fn), G.quantize_pack(w, MXFP8_E4M3_fn, G.OPERAND_B)
            outs = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
            ptrs = [o.data_ptr() for o in outs]
            return (lambda: G.mx_gemm_gather(a, b, ptrs, 0, N, 0, torch.bfloat16)), flops
        if which == "dense":            # the kind::f16 GEMM on two dense bf16 operands
            from mase_triton_b200 import tc_linear
            return (lambda: tc_linear.dense_linear(x, w)), flops
        if which == "xwq_loader":       # weight-only quantisation, codes expanded in the GEMM's operand loader whatever M is
            from mase_triton_b200 import tc_linear
            ws, we = mxk.extract_mxfp_components(w.reshape(-1), MXFP8_E4M3_fn)
            return (lambda: tc_linear.mxfp_weight_linear(x, ws, we, (N, K), MXFP8_E4M3_fn)), flops
        fc = torch.nn.Linear(K, N, bias=False, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            fc.weight.copy_(w)
        if which == "xwq":              # weight-only quantised layer: the route the layer picks for this M
            layer = MXFPLinearPTQ.from_linear(fc, None, MXFP8_E4M3_fn, None, "XWqB", "fused")
            return (lambda: layer(x)), flops
        layer = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, MXFP8_E4M3_fn, None, "XqWqB", "fused" if which == "linear" else "separate")
        return (lambda: layer(x)), flops

    def strided_case(gen, meta, s_in, which, route):
        """blocks along dim 0 of an [8192, 8192] tensor: the strided kernels against the permuted-copy route"""
        from mase_triton_b200.mxfp.helpers import flatten_for_quantize, permute_for_dequantize
        x = gen(shape=(8192, 8192)).to(dev)
        n = x.numel()
        if which == "extract":
            if route == "strided":
                return (lambda: mxk.extract_mxfp_components_strided(x, 0, meta)), n * (s_in + 1 + 1 / 32)
            return (lambda: mxk.extract_mxfp_components(flatten_for_quantize(x, 0), meta)), n * (s_in + 1 + 1 / 32)
        if route == "strided":
            return (lambda: mxk.quantize_dequantize_strided(x, 0, meta, x.dtype)), n * 2 * s_in
        return (lambda: permute_for_dequantize(mxk.quantize_dequantize(flatten_for_quantize(x, 0), meta, x.dtype),
                                               tuple(x.shape), 0).contiguous()), n * 2 * s_in

    def minifloat_linear_case(M, N, K, backend):
        """MinifloatLinearPTQ with FP8 activation and weight: tensor-core codes (fused) against dequantise + library GEMM"""
        from mase_triton_b200.minifloat.layers import MinifloatLinearPTQ
        from mase_triton_b200.minifloat.meta import FP8_E4M3_fn
        g = torch.Generator().manual_seed(0)
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
        fc = torch.nn.Linear(K, N, bias=False, device=dev, dtype=torch.bfloat16)
        with torch.no_grad():
            fc.weight.copy_((0.02 * torch.randn(N, K, generator=g)).to(torch.bfloat16))
        layer = MinifloatLinearPTQ.from_linear(fc, FP8_E4M3_fn, FP8_E4M3_fn, None, "XqWqB", backend)
        return (lambda: layer(x)), 2.0 * M * N * K

    def quant_pack_case():
        """activation -> left operand of the block-scaled GEMM in one pass (bf16 [16384, 8192], MXFP8 E4M3)"""
        from mase_triton_b200.mxfp import gemm as G
        x = synthetic.cfg3_mxfp4_bf16(shape=(16384, 8192)).to(dev)
        return (lambda: G.quantize_pack_fused(x, MXFP8_E4M3_fn)), x.numel() * (2 + 1 + 1 / 32)

    cases = {"minifloat_qdq_f32": minifloat_qdq_f32, "mx_quant_pack_bf16": quant_pack_case}
    for backend in ("fused", "separate"):
        cases[f"mx_minifloat_linear_{backend}_cfg4"] = (lambda b=backend: minifloat_linear_case(8192, 14336, 4096, b))
    for which in ("extract", "qdq"):
        for route in ("strided", "permuted"):
            cases[f"mxfp8_{which}_dim0_{route}_f32"] = (lambda w=which, r=route: strided_case(synthetic.cfg1_mxfp8_fp32, MXFP8_E4M3_fn, 4, w, r))
            cases[f"mxfp4_{which}_dim0_{route}_bf16"] = (lambda w=which, r=route: strided_case(synthetic.cfg3_mxfp4_bf16, OCP_MXFP4_E2M1, 2, w, r))
    cases["mx_gemm_gather_local_cfg4"] = (lambda: gemm_case(8192, 14336, 4096, "gather_local"))
    for which in ("gemm", "gemm4", "linear", "separate", "xwq", "xwq_loader", "dense"):
        cases[f"mx_{which}_small"] = (lambda w=which: gemm_case(2048, 4096, 4096, w))
        cases[f"mx_{which}_cfg4"] = (lambda w=which: gemm_case(8192, 14336, 4096, w))
    for which in ("extract", "compose", "qdq"):
        cases[f"mxfp8_{which}_f32"] = (lambda w=which: mx_case(synthetic.cfg1_mxfp8_fp32, (8192, 8192), MXFP8_E4M3_fn, 4, w))
        cases[f"mxfp4_{which}_bf16"] = (lambda w=which: mx_case(synthetic.cfg3_mxfp4_bf16, (8192, 8192), OCP_MXFP4_E2M1, 2, w))
        cases[f"mxfp8_{which}_bf16"] = (lambda w=which: mx_case(synthetic.cfg3_mxfp4_bf16, (8192, 8192), MXFP8_E4M3_fn, 2, w))
    return cases


def run_case(name: str, steps: int, warmup: int) -> None:
    cases = small_cases()
    if name not in cases:
        raise SystemExit(f"unknown case {name}; choose from {sorted(cases)}")
    fn, nbytes = cases[name]()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = time_steps(fn, steps)
    t = statistics.median(ts)
    peak, kind = measured_peaks()
    if name.startswith(("mx_gemm", "mx_linear", "mx_separate", "mx_minifloat", "mx_xwq", "mx_dense")):
        print(json.dumps({"case": name, "steps": steps, "median_ms": round(t, 5), "TFLOPs": round(nbytes / t / 1e9, 1),
                          "frac_of_4500_nominal_mx": round(nbytes / t / 1e9 / 4500, 4)}), flush=True)
        return
    print(json.dumps({"case": name, "steps": steps, "median_ms": round(t, 5), "GBps": round(nbytes / t / 1e6, 1),
                      "frac_of_peak": round(nbytes / t / 1e6 / peak, 4), "peak": peak, "peak_source": kind}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the side measurements (one GPU: configurations 1, 3, 4, 5; several GPUs: the sharded "
                         "configuration 3 and the column-parallel linears of configurations 4 and 5)")
    ap.add_argument("--case", default=None, help="run one small single-kernel case (for profiling) and exit")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.case is not None:
        run_case(args.case, args.steps, args.warmup)
        return
    if args.impl == "reference":
        run_reference(args)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    dist, rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)

    from mase_triton_b200 import _lib, synthetic
    from mase_triton_b200.hostpath import HostPipeline
    from mase_triton_b200.minifloat import kernels as mfk
    from mase_triton_b200.minifloat.meta import FP8_E5M2_fn
    _lib.load()
    peak, peak_kind = measured_peaks()

    x_host = synthetic.cfg2_minifloat_fp32().pin_memory()
    n = x_host.numel()
    x = x_host.to(dev, non_blocking=True)
    out = torch.empty_like(x)
    torch.cuda.synchronize()

    def step():
        mfk.quantize_dequantize(x, FP8_E5M2_fn, torch.float32, out=out)

    def barrier():
        if dist is not None:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    barrier()
    t0 = time.perf_counter()
    per_step = time_steps(step, args.steps)
    barrier()
    total_ms = sum(per_step)
    if dist is not None:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * n * BYTES_PER_ELT / (ms_per_step * 1e-3) / 1e9
    kern_ms = statistics.mean(per_step)
    achieved = n * BYTES_PER_ELT / (kern_ms * 1e-3) / 1e9
    # K steps of 85 us are over before a clock sampler sees them: keep the same kernel running, in batches of the
    # same size, until half a second has gone by, so that the clock record covers the kernel the line reports on
    sustained = list(per_step)
    while time.perf_counter() - t0 < 0.5:
        sustained += time_steps(step, max(args.steps, 50))
    t1 = time.perf_counter()
    sustained_ms = statistics.median(sustained)

    # end to end: pinned host input -> device -> kernel -> pinned host output, every step
    out_host = torch.empty_like(x_host).pin_memory()
    pipe = HostPipeline(lambda a, b: mfk.quantize_dequantize(a, FP8_E5M2_fn, torch.float32, out=b), dev, chunk_rows=512)
    copy_only = HostPipeline(lambda a, b: None, dev, chunk_rows=512)       # the same chunked copies with no kernel: what the host link allows
    e2e_steps = max(3, min(args.steps, 10))

    def timed_pipe(p) -> float:
        p.run(x_host, out_host)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            p.run(x_host, out_host)
        e1.record()
        barrier()
        return e0.elapsed_time(e1)

    copy_ms_local = timed_pipe(copy_only)
    launches_before = pipe.launches
    e2e_ms_local = timed_pipe(pipe)
    e2e_launches = pipe.launches - launches_before
    e2e_ms, copy_ms, e2e_spread = e2e_ms_local, copy_ms_local, None
    if dist is not None:
        t = torch.tensor([e2e_ms_local, copy_ms_local, -e2e_ms_local], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms, copy_ms = float(t[0].item()), float(t[1].item())
        e2e_spread = {"fastest_rank_ms_per_step": round(-float(t[2].item()) / e2e_steps, 3), "slowest_rank_ms_per_step": round(e2e_ms / e2e_steps, 3)}
    e2e_value = world * n * BYTES_PER_ELT / (e2e_ms / e2e_steps * 1e-3) / 1e9
    copy_value = world * n * BYTES_PER_ELT / (copy_ms / e2e_steps * 1e-3) / 1e9
    sampler.stop()
    clocks = sampler.summary(t0, t1)
    # the e2e result must equal the device-resident one
    e2e_ok = bool(torch.equal(out_host.view(torch.int32), out.cpu().view(torch.int32)))

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "inputs larger than L2 (256 MiB in + 256 MiB out per step)",
                       "bytes_per_element": BYTES_PER_ELT, "elements_per_gpu": n, "parallelism": f"rows x{world} (independent shards, no collective)"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": round(n * NCU_TRAFFIC_BYTES_PER_ELT),
                         "traffic_source": "ncu dram__bytes_read+write on the 4096x8192 case scaled by elements "
                                           "(profiles/minifloat_qdq_f32_small_case_full.md); writes still in L2 at kernel end are not counted",
                         "peak_source": f"{peak_kind} HBM copy bandwidth",
                         "kernel": "ew_vec_kernel<4,4,4,4,QdqOp<f32,f32,E5M2>>", "launch_ms": round(kern_ms, 5),
                         "sustained": {"steps": len(sustained), "median_launch_ms": round(sustained_ms, 5),
                                       "achieved": round(n * BYTES_PER_ELT / (sustained_ms * 1e-3) / 1e9, 1),
                                       "frac": round(n * BYTES_PER_ELT / (sustained_ms * 1e-3) / 1e9 / peak, 4),
                                       "what": "the same launch repeated until 0.5 s had passed, so that the clock record covers it"}},
            "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": n * 4, "d2h_bytes_per_step": n * 4,
                    "steps": e2e_steps, "ms_per_step": round(e2e_ms / e2e_steps, 3), "matches_device_result": e2e_ok,
                    "path": "HostPipeline: pinned host -> 512-row chunks over 3 streams -> pinned host",
                    # the same chunked host->device and device->host copies with no kernel in between: the ceiling the
                    # host link (PCIe, shared by the ranks of one box) sets for this number
                    "copy_ceiling": round(copy_value, 2), "frac": round(e2e_value / copy_value, 4),
                    "copy_ceiling_ms_per_step": round(copy_ms / e2e_steps, 3), "rank_spread": e2e_spread},
            "gpu_launches": args.steps, "e2e_gpu_launches": e2e_launches,
            "clocks": clocks,
        }
        if world == 1:
            try:
                line["cpu_baseline"] = cpu_baseline()
            except Exception as exc:      # the baseline must never hide the GPU result
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": None, "kind": "port", "sample": f"failed: {exc}"}
        if world == 1 and not args.no_extras:
            del x, out
            torch.cuda.empty_cache()
            try:
                line["extras"] = extras_single_gpu(dev, max(5, min(args.steps, 50)), args.warmup, peak)
            except Exception as exc:
                line["extras"] = {"error": str(exc)}
    extras_multi = None
    if dist is not None and not args.no_extras:
        del x, out
        torch.cuda.empty_cache()
        try:
            extras_multi = extras_multi_gpu(dev, dist, rank, world, local, max(5, min(args.steps, 50)), peak)
        except Exception as exc:
            extras_multi = {"error": str(exc)}
    if rank == 0:
        if extras_multi is not None:
            line["extras"] = extras_multi
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier(device_ids=[local])
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
