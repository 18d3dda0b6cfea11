#!/usr/bin/env python
"""Benchmark of the quantization hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload at every N: the row-sharded configuration -- a bf16 [262144, 8192] matrix (4 GiB,
N(0,1) with 0.01% x1000 outliers, 8 seeded row chunks), rank g owning 8/N chunks.  One step =
tensor-wise dynamic e4m3 quantisation of the whole matrix (local amax -> one-scalar max
all-reduce -> cast; no exchange when N == 1) plus the MX block-32 cast of the same
rows.  Total work is fixed as N grows (strong scaling).  ``value`` is algorithmic bytes of
the whole job per second of device time (max over ranks): tensor-wise N*(2+1) compulsory
bytes + MX N*(2+1+1/32).

Rank 0 prints ONE JSON line.  Besides the contract keys it carries ``roofline`` (dominant
kernel), ``kernels`` (every kernel of the step), ``ops`` (N == 1: the single-GPU
configurations cfg1-cfg4, cold-L2, one line per op, with the reference CUDA kernel timed
beside it when oracle/_ref is built), ``cpu_baseline`` and ``e2e`` (host buffers in, host
buffers out, through driss_torch_b200.host_pipeline).

``--impl reference`` times the CPU restatement of the reference (oracle/, all host threads)
on a bounded sample of the same workload; rank 0 alone works.
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
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
TOTAL_ROWS, COLS, TOTAL_CHUNKS = 262144, 8192, 8
METRIC = "effective HBM GB/s (algorithmic bytes / device time), row-sharded tensor-wise e4m3 quant + MX block-32 cast"


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# ---- clocks ------------------------------------------------------------------------------------------

class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=5)
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---- helpers -------------------------------------------------------------------------------------------

def event_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def algorithmic_bytes(op: str, rows: int, cols: int, s_in: int = 2) -> int:
    n = rows * cols
    return {
        "saturated_cast": n * (s_in + 1) + 4,
        "amax": n * s_in + 4,
        "dynamic_scaled_quant": n * (s_in + 1),
        "cast_with_amax": n * (s_in + 1),
        "mx_fp8_quantize": n * 3 + n // 32,
        "dynamic_scaled_quant_rowwise": n * (s_in + 1) + 8 * rows,
    }[op]


def time_rotating(fn, nsets: int, iters: int, warmup: int = 3):
    """Device time of fn(i % nsets), two ways; consecutive calls touch different buffer sets, so every
    launch starts with its inputs out of L2.  A spin kernel is queued first each time so that the
    events and launches are enqueued while the GPU is busy: the intervals hold device time only.

    Returns (steady, single, single_min) in ms: `steady` = `iters` launches back to back between one
    event pair, divided by `iters` (what a pipeline of such launches sustains); `single` = median
    over `iters` isolated launches, each between its own event pair (adds the start-up and drain of
    a lone kernel, several microseconds that matter for the sub-100 us configurations)."""
    for i in range(warmup):
        fn(i % nsets)
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        a, b = event_pair()
        torch.cuda._sleep(400_000)
        a.record()
        fn(i % nsets)
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    a, b = event_pair()
    torch.cuda._sleep(4_000_000)  # about 2 ms: covers the host time of enqueueing `iters` launches
    a.record()
    for i in range(iters):
        fn(i % nsets)
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / iters, statistics.median(times), min(times)


# ---- the single-GPU per-op table (cfg1..cfg4) ----------------------------------------------------------------

def measured_tensor_peak():
    """The pool's measured dense bf16 tensor throughput (cuBLAS, burst), TFLOP/s; None if the file is absent."""
    p = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(p.read_text())["bf16_tflops"])
    except Exception:
        return None


def gemm_table(dev, iters: int, warmup: int = 3):
    """The MX block-scaled GEMM that consumes the MX casts (the reference's mx_fp8_bf16), one line per shape:
    operands from the blocked MX cast of N(0,1) data, device time per launch, TFLOP/s."""
    import driss_torch_b200 as dtq
    from driss_torch_b200 import _cabi

    rows = []
    bf16_peak = measured_tensor_peak()
    ref = None
    ref_lib = ROOT / "oracle" / "_ref" / "libdriss_torch_ref_gemm.so"  # the reference's CUTLASS GEMM, if it was built
    if ref_lib.exists():
        try:
            torch.ops.load_library(str(ref_lib))
            ref = torch.ops.DrissTorchRefGemm
        except Exception:
            ref = None
    gen = torch.Generator(device=dev)
    gen.manual_seed(1100)
    ws = _cabi.workspace(dev)
    for (m, n, k, fp4) in [(8192, 8192, 8192, False), (4096, 4096, 4096, False), (16384, 8192, 4096, False),
                           (1024, 1024, 1024, False), (8192, 8192, 8192, True)]:
        a = torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16)
        b = torch.randn(n, k, generator=gen, device=dev).to(torch.bfloat16)
        quantize = (lambda t: dtq.mx_fp4_quantize(t, blocked=True)) if fp4 else dtq.mx_fp8_quantize_blocked
        pa, sa = quantize(a)
        pb, sb = quantize(b)
        del a, b
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        # These kernels run into the board's power limit, and the clock the limiter leaves depends on what ran in
        # the last few milliseconds.  So: an idle pause before each shape, and our kernel and the reference's timed
        # in alternating blocks (ours, theirs, ours, theirs), each one's figure the mean over its blocks.
        pbt = pb.t()
        ref_fn = (ref.mx_fp4_bf16 if fp4 else ref.mx_fp8_bf16) if ref is not None else None
        time.sleep(0.5)
        mine, theirs = [], []
        for _ in range(2):
            mine.append(time_rotating(lambda i: _cabi.mx_fp8_bf16(pa, pb, sa, sb, out=out, ws=ws, fp4=fp4), 1, iters, warmup))
            if ref_fn is not None:
                theirs.append(time_rotating(lambda i: ref_fn(pa, pbt, sa, sb), 1, iters, warmup))
        ms = statistics.mean(t[0] for t in mine)
        single = statistics.mean(t[1] for t in mine)
        flops = 2.0 * m * n * k
        set_bytes = pa.numel() + pb.numel() + 2 * m * n
        d = {"config": "gemm", "op": "mx_fp4_bf16" if fp4 else "mx_fp8_bf16", "shape": [m, n, k], "us": round(ms * 1e3, 2),
             "us_single_launch": round(single * 1e3, 2), "TFLOPs": round(flops / (ms * 1e-3) / 1e12, 1),
             "note": "%s with E8M0 block scales, fp32 accumulation in tensor memory, bf16 out; back-to-back launches "
                     "on one buffer set of %d MB (operands + output): %s; power-limited kernels: half a second idle "
                     "before the shape, then blocks of launches alternating with the reference kernel's, mean over blocks" % (
                         "e2m1 x e2m1 (packed two per byte)" if fp4 else "e4m3 x e4m3", set_bytes >> 20,
                         "larger than L2, no flush" if set_bytes > 126e6 else "NOT larger than L2: an "
                         "L2-warm figure, as behind the casts that produce the operands")}
        if bf16_peak:
            d["x_measured_bf16_peak"] = round(flops / (ms * 1e-3) / 1e12 / bf16_peak, 3)
            d["peak_note"] = (f"against the pool's measured cuBLAS bf16 throughput ({bf16_peak} TFLOP/s, MEASURED_PEAKS.json); "
                              "no fp8 / fp4 peak is measured on this pool: nominal dense fp8 is 2x, fp4 4x nominal bf16 "
                              "(4.5 / 9 vs 2.25 PFLOP/s)")
        d["device_status"] = _cabi.workspace_status(ws)
        if ref_fn is not None:
            want = ref_fn(pa, pbt, sa, sb)
            d["equals_reference_kernel_bitwise"] = bool(torch.equal(want.view(torch.int16), out.view(torch.int16)))
            rms = statistics.mean(t[0] for t in theirs)
            d["reference_kernel_us"] = round(rms * 1e3, 2)
            d["reference_kernel_TFLOPs"] = round(flops / (rms * 1e-3) / 1e12, 1)
            d["speedup_vs_reference_kernel"] = round(rms / ms, 2)
            del want
        rows.append(d)
        del pa, pb, sa, sb, out
    torch.cuda.empty_cache()

    # sweep_mm: the row-wise scaled fp8 GEMM behind the row-wise quantisation.  The reference's kernels for it are
    # Hopper-only, so the comparison is the library's row-wise scaled matmul (torch._scaled_mm -> cuBLASLt), same
    # operands and scales, where this torch build has one for the device.
    for (m, n, k) in [(8192, 8192, 8192), (16384, 8192, 4096)]:
        x = torch.randn(m, k, generator=gen, device=dev).to(torch.bfloat16)
        w = torch.randn(n, k, generator=gen, device=dev).to(torch.bfloat16)
        xq, _, xs = dtq.dynamic_scaled_quant_rowwise(x, E4M3)
        wq, _, ws_ = dtq.dynamic_scaled_quant_rowwise(w, E4M3)
        x_deq, w_deq = (1.0 / xs).reshape(m).contiguous(), (1.0 / ws_).reshape(n).contiguous()
        del x, w
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        time.sleep(0.5)
        lib = None
        try:
            got = torch._scaled_mm(xq, wq.t(), x_deq.reshape(m, 1), w_deq.reshape(1, n), out_dtype=torch.bfloat16)
            lib = lambda i: torch._scaled_mm(xq, wq.t(), x_deq.reshape(m, 1), w_deq.reshape(1, n), out_dtype=torch.bfloat16)
            del got
        except Exception:
            lib = None
        mine, theirs = [], []
        for _ in range(2):
            mine.append(time_rotating(lambda i: _cabi.rowwise_fp8_bf16(xq, wq, x_deq, w_deq, out=out, ws=ws), 1, iters, warmup))
            if lib is not None:
                theirs.append(time_rotating(lib, 1, iters, warmup))
        ms = statistics.mean(t[0] for t in mine)
        flops = 2.0 * m * n * k
        d = {"config": "gemm", "op": "sweep_mm (row-wise scaled fp8 GEMM)", "shape": [m, n, k], "us": round(ms * 1e3, 2),
             "us_single_launch": round(statistics.mean(t[1] for t in mine) * 1e3, 2),
             "TFLOPs": round(flops / (ms * 1e-3) / 1e12, 1),
             "note": "e4m3 x e4m3, fp32 accumulation, per-row scales of both operands applied to the accumulator, bf16 out; "
                     "operands from dynamic_scaled_quant_rowwise; timed like the MX GEMM lines",
             "device_status": _cabi.workspace_status(ws)}
        if bf16_peak:
            d["x_measured_bf16_peak"] = round(flops / (ms * 1e-3) / 1e12 / bf16_peak, 3)
        if theirs:
            lms = statistics.mean(t[0] for t in theirs)
            d["library_scaled_mm_us"] = round(lms * 1e3, 2)
            d["speedup_vs_library_scaled_mm"] = round(lms / ms, 2)
        rows.append(d)
        del xq, wq, xs, ws_, x_deq, w_deq, out
    torch.cuda.empty_cache()
    return rows


def per_op_table(dev, peak, iters: int, warmup: int = 3):
    import driss_torch_b200  # noqa: F401  (registers the ops; loads the CUDA libraries)
    from driss_torch_b200 import _cabi, workloads

    ref = None
    ref_lib = ROOT / "oracle" / "_ref" / "libdriss_torch_ref.so"
    if ref_lib.exists():
        try:
            torch.ops.load_library(str(ref_lib))
            ref = torch.ops.DrissTorchRef
        except Exception:
            ref = None

    rows = []

    def timed(fn, nsets, iters):
        return time_rotating(fn, nsets, iters, warmup)

    def line(cfg, op, shape, t, nbytes, ref_t=None, note=None):
        ms, single, single_min = t
        ref_ms = ref_t[0] if ref_t else None
        gbs = nbytes / (ms * 1e-3) / 1e9
        d = {"config": cfg, "op": op, "shape": list(shape), "us": round(ms * 1e3, 2),
             "us_single_launch": round(single * 1e3, 2), "us_single_launch_min": round(single_min * 1e3, 2),
             "algorithmic_bytes": nbytes, "GBps": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 4),
             "frac_of_nominal_8TBps": round(gbs / NOMINAL_HBM_GBS, 4),
             "GBps_single_launch": round(nbytes / (single * 1e-3) / 1e9, 1)}
        if ref_ms is not None:
            d["reference_kernel_us"] = round(ref_ms * 1e3, 2)
            d["speedup_vs_reference_kernel"] = round(ref_ms / ms, 2)
        if note:
            d["note"] = note
        rows.append(d)

    def sets_for(bytes_per_set):
        return max(2, int(-(-300e6 // bytes_per_set)) + 1)  # consecutive sets cover > 2x the 126 MB L2

    # cfg1: saturated_cast bf16 [4096,4096] -> e4m3
    w = workloads.WORKLOADS["cfg1"]
    x = workloads.make_cfg1(device=dev)
    scale = workloads.tensor_scale(x, E4M3)
    ns = sets_for(x.numel() * 3)
    xs = [x.clone() for _ in range(ns)]
    outs = [torch.empty(x.shape, dtype=E4M3, device=dev) for _ in range(ns)]
    t = timed(lambda i: _cabi.saturated_cast(xs[i], scale, E4M3, out=outs[i]), ns, iters)
    rt = timed(lambda i: ref.saturated_cast(xs[i], scale, E4M3, False), ns, iters) if ref else None
    line("cfg1", "saturated_cast", x.shape, t, algorithmic_bytes("saturated_cast", w.rows, w.cols), rt)
    outs_t = [torch.empty(w.cols, w.rows, dtype=E4M3, device=dev) for _ in range(ns)]
    t = timed(lambda i: _cabi.saturated_cast_transposed(xs[i], scale, E4M3, out_t=outs_t[i]), ns, iters)
    line("cfg1", "saturated_cast_transposed", x.shape, t, algorithmic_bytes("saturated_cast", w.rows, w.cols), None,
         note="output [cols, rows]; the reference declares the flag but does not implement it")
    t = timed(lambda i: _cabi.saturated_cast_transposed(xs[i], scale, E4M3, out_t=outs_t[i], out=outs[i]), ns, iters)

    def cast_twice(i):
        _cabi.saturated_cast(xs[i], scale, E4M3, out=outs[i])
        _cabi.saturated_cast(xs[i].t().contiguous(), scale, E4M3, out=outs_t[i])

    t2 = timed(cast_twice, ns, iters)
    line("cfg1", "saturated_cast_dual (x and x^T from one read)", x.shape, t, x.numel() * 4 + 4, None,
         note=f"same two outputs by cast + torch transpose + cast: {t2[0] * 1e3:.1f} us")
    del xs, outs, outs_t

    # the shapes of the reference author's own benchmark (benchmarks/benchmark_saturated_casting.py:52-64),
    # bf16 -> e4m3 and e5m2, N(0,1) values as there, the reference kernel timed beside each
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000)
    for (r, c) in [(512, 512), (1024, 1024), (2048, 2048), (1024, 8192), (8192, 1280), (8192, 7168), (3584, 8192),
                   (2048, 109760), (1, 3232), (2048, 1), (14144, 2048)]:
        xa = torch.randn(r, c, generator=gen, device=dev).to(torch.bfloat16)
        ns = min(sets_for(xa.numel() * 3), 64)
        xs = [xa.clone() for _ in range(ns)]
        for dt_, name in ((E4M3, "e4m3"), (E5M2, "e5m2")):
            sc = workloads.tensor_scale(xa, dt_)
            outs = [torch.empty(xa.shape, dtype=dt_, device=dev) for _ in range(ns)]
            t = timed(lambda i: _cabi.saturated_cast(xs[i], sc, dt_, out=outs[i]), ns, iters)
            rt = timed(lambda i: ref.saturated_cast(xs[i], sc, dt_, False), ns, iters) if ref else None
            line("author", f"saturated_cast->{name}", xa.shape, t, algorithmic_bytes("saturated_cast", r, c), rt)
            del outs
        del xs, xa

    # cfg2: amax + fused dynamic_scaled_quant bf16 [8192,8192], e4m3 and e5m2
    w = workloads.WORKLOADS["cfg2"]
    x = workloads.make_cfg2(device=dev)
    ns = 3
    xs = [x.clone() for _ in range(ns)]
    outs = [torch.empty(x.shape, dtype=E4M3, device=dev) for _ in range(ns)]
    one = torch.empty(1, dtype=torch.float32, device=dev)
    t = timed(lambda i: _cabi.amax(xs[i], out=one), ns, iters)
    rt = timed(lambda i: ref.amax(xs[i]), ns, iters) if ref else None
    line("cfg2", "amax", x.shape, t, algorithmic_bytes("amax", w.rows, w.cols), rt)
    t = timed(lambda i: _cabi.cast_with_amax(xs[i], one, E4M3, out=outs[i]), ns, iters)
    line("cfg2", "cast_with_amax->e4m3", x.shape, t, algorithmic_bytes("cast_with_amax", w.rows, w.cols), None,
         note="phase 2 of the sharded tensor-wise path (amax already on the device); no reference op")
    xf = None
    for dt_, name in ((E4M3, "e4m3"), (E5M2, "e5m2")):
        o = [t.view(dt_) for t in outs]
        t = timed(lambda i: _cabi.dynamic_scaled_quant(xs[i], dt_, out=o[i]), ns, iters)
        rt = None
        if ref:  # the reference instantiates fp32 input only: time it on float(x) (twice the input bytes)
            if xf is None:
                xf = [t_.float() for t_ in xs]
            rt = timed(lambda i: ref.dynamic_scaled_quant(xf[i], dt_), ns, iters)
        line("cfg2", f"dynamic_scaled_quant->{name}", x.shape, t,
             algorithmic_bytes("dynamic_scaled_quant", w.rows, w.cols), rt,
             note="compulsory bytes N*(2+1); a two-pass kernel moves N*(2*2+1) unless the re-read hits L2; "
                  "reference kernel timed on fp32 input")
    outs_t = [torch.empty(w.cols, w.rows, dtype=E4M3, device=dev) for _ in range(ns)]
    ws_ = _cabi.workspace(dev)

    def dual(i):
        _cabi.dynamic_scaled_quant_dual(xs[i], E4M3, out=outs[i], out_t=outs_t[i], amax_out=one, ws=ws_)

    def twice(i):
        _cabi.dynamic_scaled_quant(xs[i], E4M3, out=outs[i], ws=ws_)
        _cabi.dynamic_scaled_quant(xs[i].t().contiguous(), E4M3, out=outs_t[i], ws=ws_)

    t = timed(dual, ns, iters)
    t2 = timed(twice, ns, iters)
    line("cfg2", "dynamic_scaled_quant_dual (amax, then x and x^T cast from one read)", x.shape, t,
         x.numel() * 4, None,
         note=f"compulsory bytes N*(2+1+1); two launches (the second started under the tail of the first) move "
              f"N*(2+2+1+1); the same two outputs by fused op + torch transpose + fused op: {t2[0] * 1e3:.1f} us")
    del xs, outs, xf, outs_t

    # cfg3: mx_fp8_quantize bf16 [16384,8192]
    w = workloads.WORKLOADS["cfg3"]
    x = workloads.make_cfg3(device=dev)
    ns = 2
    xs = [x.clone() for _ in range(ns)]
    ps = [torch.empty(x.shape, dtype=E4M3, device=dev) for _ in range(ns)]
    ss = [torch.empty(x.numel() // 32, dtype=torch.float8_e8m0fnu, device=dev) for _ in range(ns)]
    t = timed(lambda i: _cabi.mx_fp8_quantize(xs[i], payload=ps[i], scales=ss[i]), ns, iters)
    rt = timed(lambda i: ref.mx_fp8_quantize(xs[i], 32, 1, False, E4M3), ns, iters) if ref else None
    line("cfg3", "mx_fp8_quantize", x.shape, t, algorithmic_bytes("mx_fp8_quantize", w.rows, w.cols), rt)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    t = timed(lambda i: _cabi.mx_fp8_quantize_tma(xs[i], payload=ps[i], scales=ss[i], status=status), ns, iters)
    line("cfg3", "mx_fp8_quantize (TMA-staged variant)", x.shape, t, algorithmic_bytes("mx_fp8_quantize", w.rows, w.cols),
         None, note=f"same outputs through a cp.async.bulk + mbarrier shared-memory ring; status {int(status.item())}")
    sb = [torch.empty(_cabi.load().dtq_mx_blocked_scale_bytes(w.rows, w.cols), dtype=torch.uint8, device=dev)
          .view(torch.float8_e8m0fnu) for _ in range(ns)]
    t = timed(lambda i: _cabi.mx_fp8_quantize_blocked(xs[i], payload=ps[i], scales=sb[i]), ns, iters)
    line("cfg3", "mx_fp8_quantize_blocked", x.shape, t, algorithmic_bytes("mx_fp8_quantize", w.rows, w.cols), None,
         note="scales written in the MX GEMM's blocked layout (the reference needs a separate to_blocked pass)")
    t = timed(lambda i: _cabi.mx_quantize(xs[i], E5M2, payload=ps[i].view(E5M2), scales=ss[i]), ns, iters)
    line("cfg3", "mx_fp8_quantize -> e5m2 payload", x.shape, t, algorithmic_bytes("mx_fp8_quantize", w.rows, w.cols), None,
         note="the reference accepts fp8_type=e5m2 but writes e4m3; same scale rule with e5m2's largest exponent")
    p4 = [torch.empty(w.rows, w.cols // 2, dtype=torch.uint8, device=dev) for _ in range(ns)]
    t = timed(lambda i: _cabi.mx_quantize(xs[i], "e2m1", payload=p4[i], scales=ss[i]), ns, iters)
    line("cfg3", "mx_fp4_quantize (e2m1, two per byte)", x.shape, t, x.numel() * 2 + x.numel() // 2 + x.numel() // 32, None,
         note="producer for the operands of the reference's mx_fp4_bf16, which has none")
    del p4
    pt = [torch.empty(w.cols, w.rows, dtype=E4M3, device=dev) for _ in range(ns)]
    st = [torch.empty(x.numel() // 32, dtype=torch.float8_e8m0fnu, device=dev) for _ in range(ns)]
    dual_bytes = x.numel() * 2 + 2 * (x.numel() + x.numel() // 32)
    t = timed(lambda i: _cabi.mx_fp8_quantize_dual(xs[i], ps[i], ss[i], pt[i], st[i]), ns, iters)

    def two_casts(i):
        _cabi.mx_fp8_quantize(xs[i], payload=ps[i], scales=ss[i])
        _cabi.mx_fp8_quantize(xs[i].t().contiguous(), payload=pt[i], scales=st[i])

    t2 = timed(two_casts, ns, iters)
    line("cfg3", "mx_fp8_quantize_dual (x and x^T from one read)", x.shape, t, dual_bytes, None,
         note=f"same four outputs by cast + torch transpose + cast: {t2[0] * 1e3:.1f} us")
    del xs, ps, ss, sb, pt, st

    # cfg4: row-wise dynamic quant bf16 [32768,4096] (no reference op)
    w = workloads.WORKLOADS["cfg4"]
    x = workloads.make_cfg4(device=dev)
    ns = 2
    xs = [x.clone() for _ in range(ns)]
    ps = [torch.empty(x.shape, dtype=E4M3, device=dev) for _ in range(ns)]
    am = torch.empty(w.rows, 1, dtype=torch.float32, device=dev)
    sc = torch.empty(w.rows, 1, dtype=torch.float32, device=dev)
    t = timed(
        lambda i: _cabi.dynamic_scaled_quant_rowwise(xs[i], E4M3, out=ps[i], amax_out=am, scale_out=sc), ns, iters)
    line("cfg4", "dynamic_scaled_quant_rowwise", x.shape, t,
         algorithmic_bytes("dynamic_scaled_quant_rowwise", w.rows, w.cols), None, note="no reference op")
    del xs, ps
    torch.cuda.empty_cache()
    return rows


# ---- CPU baselines and the oracle check of the timed buffers -------------------------------------------

def load_workloads():
    """The input generators (driss_torch_b200/workloads.py) loaded as a stand-alone module: importing the
    package would load the CUDA libraries, which the CPU-only reference arm must not map."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("dtq_workloads", ROOT / "driss_torch_b200" / "workloads.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def make_chunks_cpu(workloads, chunk_ids, chunk_rows: int):
    """Row chunks of the workload from the CPU generator (the one source of the values for both arms, so their
    output checksums are comparable); a few chunks at a time, since one chunk's generation is mostly serial."""
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=min(4, max(1, len(chunk_ids)))) as pool:
        return list(pool.map(lambda c: workloads.make_cfg5_chunk(c, rows=chunk_rows, cols=COLS), chunk_ids))


class CpuStep:
    """One step of the workload on the CPU restatement of the reference kernels (oracle/quant_oracle.c): the
    tensor-wise e4m3 quantisation (amax over every chunk, then the cast) and the MX cast of a list of row chunks,
    into preallocated output buffers."""

    def __init__(self, chunks):
        from oracle import quant_oracle as qo

        self.qo, self.chunks = qo, chunks
        self.payload = [torch.empty(c.shape, dtype=torch.uint8) for c in chunks]
        self.mx_payload = [torch.empty(c.shape, dtype=torch.uint8) for c in chunks]
        self.mx_scales = [torch.empty(c.numel() // 32, dtype=torch.uint8) for c in chunks]
        self.amax, self.scale = 0.0, None

    def run(self):
        qo = self.qo
        self.amax = max([0.0] + [qo.amax(c).item() for c in self.chunks])
        for c, p, mp, ms in zip(self.chunks, self.payload, self.mx_payload, self.mx_scales):
            _, self.scale = qo.cast_with_amax(c, self.amax, E4M3, out=p)
            qo.mx_fp8_quantize(c, payload=mp, scales=ms)

    def time(self, repeats: int) -> float:
        best = float("inf")
        for _ in range(repeats):
            t0 = time.perf_counter()
            self.run()
            best = min(best, time.perf_counter() - t0)
        return best

    def checksums(self):
        return [sum(int(t.sum(dtype=torch.int64)) for t in ts) for ts in (self.payload, self.mx_payload, self.mx_scales)]


def time_cpu_eager(x, repeats: int):
    """The reference tests' PyTorch-eager expressions for the same step, on CPU tensors."""
    from oracle import eager

    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        eager.dynamic_scaled_quant_eager(x, E4M3)
        eager.mx_fp8_quantize_eager(x)
        best = min(best, time.perf_counter() - t0)
    return best


def step_bytes(rows: int) -> int:
    return algorithmic_bytes("dynamic_scaled_quant", rows, COLS) + algorithmic_bytes("mx_fp8_quantize", rows, COLS)


def oracle_check_and_cpu_baseline(x, payload, mx_payload, mx_scales, amax, scale, check_rows: int, chunk_rows: int,
                                  whole_matrix: bool, time_it: bool):
    """After the timed region: the first `check_rows` rows of the buffers the benchmark just timed (the input as it
    sits on the device, and the three outputs) against the C oracle, byte for byte; `whole_matrix` says that
    these rows are the entire matrix, in which case the oracle derives the amax itself and its byte sums are the
    reference for `output_checksums`.  The same oracle run is the CPU baseline (`time_it`: best of 2 more runs)."""
    from oracle import quant_oracle as qo

    qo.set_num_threads(os.cpu_count() or 1)  # torchrun pins OMP_NUM_THREADS=1 for its children
    bpr = COLS // 32
    spans = [(r0, min(check_rows, r0 + chunk_rows)) for r0 in range(0, check_rows, chunk_rows)]
    step = CpuStep([x[r0:r1].cpu() for r0, r1 in spans])
    gpu_amax, gpu_scale = float(amax.item()), float(scale.item())
    step.run()
    if not whole_matrix:  # a part of the matrix cannot know the global amax: take the device's, check it is no smaller
        assert step.amax <= gpu_amax
        step.amax = gpu_amax
        for c, p in zip(step.chunks, step.payload):
            _, step.scale = qo.cast_with_amax(c, gpu_amax, E4M3, out=p)
    equal = step.amax == gpu_amax and float(step.scale.item()) == gpu_scale
    differing = 0
    for (r0, r1), p, mp, ms in zip(spans, step.payload, step.mx_payload, step.mx_scales):
        differing += int((payload[r0:r1].view(torch.uint8).cpu() != p).sum())
        differing += int((mx_payload[r0:r1].view(torch.uint8).cpu() != mp).sum())
        differing += int((mx_scales[r0 * bpr:r1 * bpr].view(torch.uint8).cpu() != ms).sum())
    parity = {"rows": check_rows, "whole_matrix": whole_matrix, "bytes_equal": bool(equal and differing == 0),
              "bytes_differing": differing, "amax_equal": step.amax == gpu_amax,
              "checker": "oracle/quant_oracle.c on the timed input as downloaded from the device"}
    if whole_matrix:
        parity["oracle_checksums"] = step.checksums()
    cpu = None
    if time_it:
        t = step.time(repeats=2)
        sample_rows = min(check_rows, 32768)
        te = time_cpu_eager(step.chunks[0][:sample_rows], repeats=2)
        cpu = {"value": round(step_bytes(check_rows) / t / 1e9, 3), "unit": "GB/s", "cores": qo.num_threads(),
               "kind": "port",
               "sample": f"{check_rows}x{COLS} bf16 rows (" + ("the whole matrix" if whole_matrix else "rank 0's first rows")
                         + "), best of 2; oracle/quant_oracle.c with OpenMP",
               "eager_value": round(step_bytes(sample_rows) / te / 1e9, 3), "eager_cores": torch.get_num_threads(),
               "eager_note": f"the reference tests' PyTorch-eager formulas (oracle/eager.py) on the first {sample_rows} rows, best of 2"}
    return parity, cpu


def run_reference_arm(args, rank: int):
    """CPU restatement of the reference kernels on the whole matrix, every step (rank 0 only; no CUDA library
    is loaded in this process)."""
    if rank != 0:
        return
    from oracle import quant_oracle as qo

    workloads = load_workloads()
    # torchrun pins OMP_NUM_THREADS=1 for its children; this arm is meant to use every host core
    qo.set_num_threads(os.cpu_count() or 1)
    chunk_rows = args.rows // TOTAL_CHUNKS
    step = CpuStep(make_chunks_cpu(workloads, list(range(TOTAL_CHUNKS)), chunk_rows))
    for _ in range(args.warmup):
        step.run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step.run()
    dt_ = (time.perf_counter() - t0) / args.steps
    value = step_bytes(args.rows) / dt_ / 1e9
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt_ * 1e3, 3), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16->fp8 (f64 scale arithmetic)", "data": "synthetic",
        "config": {"workload": f"cfg5: bf16 [{args.rows},{COLS}] row-sharded over {args.gpus} GPU(s); tensor-wise e4m3 "
                               "quant (amax -> max all-reduce -> cast) + MX block-32 cast",
                   "what_runs": "CPU restatement of the reference kernels (oracle/quant_oracle.c, OpenMP, every host "
                                "core) on the whole matrix every step; the reference itself is CUDA-only and has no "
                                "CPU implementation"},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": qo.num_threads(), "kind": "port",
                         "sample": f"the whole {args.rows}x{COLS} bf16 matrix every step"},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "output_checksums": step.checksums(), "gpu_launches": 0,
    }), flush=True)


# ---- main ---------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-ops-table", action="store_true", help="skip the cfg1-cfg4 per-op table")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--rows", type=int, default=TOTAL_ROWS, help="total rows (smaller for profiling captures)")
    ap.add_argument("--exchange", choices=["auto", "p2p", "nccl"], default="auto",
                    help="N > 1: how the per-GPU maxima meet: inside the one fused launch over NVLink peer memory (p2p), "
                         "or an NCCL all-reduce between an amax launch and a cast launch (nccl); auto = p2p for shards up to 1.5 GiB "
                         "(measured: the single persistent launch wins there, two stream launches win above)")
    ap.add_argument("--compose", choices=["shared-read", "separate"], default="shared-read",
                    help="shared-read: the MX cast also delivers the amax (and exchanges it), then the cast: two reads "
                         "of the input; separate: amax, cast and MX cast as independent ops: three reads")
    ap.add_argument("--ops-table-only", action="store_true", help="only the cfg1-cfg4 per-op table (profiling captures)")
    ap.add_argument("--gemm-only", action="store_true", help="only the MX GEMM lines (profiling captures)")
    ap.add_argument("--op-iters", type=int, default=0, help="timed launches per op in the per-op table (default max(20, steps))")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if TOTAL_CHUNKS % world or args.rows % (TOTAL_CHUNKS * 128):
        raise SystemExit("the workload shards as 8 row chunks: use 1, 2, 4 or 8 GPUs and rows % 1024 == 0")

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import driss_torch_b200 as dtq
    from driss_torch_b200 import _cabi, workloads
    from driss_torch_b200.host_pipeline import HostQuantizer

    peak, peak_kind = measured_peak()
    if args.gemm_only:
        iters = args.op_iters or max(20, args.steps)
        print(json.dumps({"ops": gemm_table(dev, iters=iters, warmup=min(3, iters))}), flush=True)
        return
    if args.ops_table_only:
        iters = args.op_iters or max(20, args.steps)
        print(json.dumps({"ops": per_op_table(dev, peak, iters=iters, warmup=min(3, iters))}), flush=True)
        return
    chunk_rows = args.rows // TOTAL_CHUNKS
    # generated by the CPU generator and uploaded: the reference arm generates the same values
    per_rank = TOTAL_CHUNKS // world
    x = torch.empty(per_rank * chunk_rows, COLS, dtype=torch.bfloat16, device=dev)
    for i, part in enumerate(make_chunks_cpu(workloads, list(range(rank * per_rank, (rank + 1) * per_rank)), chunk_rows)):
        x[i * chunk_rows:(i + 1) * chunk_rows].copy_(part)
    del part
    rows_local = x.shape[0]
    payload = torch.empty(x.shape, dtype=E4M3, device=dev)
    mx_payload = torch.empty(x.shape, dtype=E4M3, device=dev)
    mx_scales = torch.empty(x.numel() // 32, dtype=torch.float8_e8m0fnu, device=dev)
    amax = torch.zeros(1, dtype=torch.float32, device=dev)
    scale = torch.zeros(1, dtype=torch.float32, device=dev)
    ws = _cabi.workspace(dev)

    # At N == 1 the exchange disappears; amax + cast are then exactly the two launches that
    # dtq_dynamic_scaled_quant itself issues for an input this large (above 320 MiB it does not use
    # its single fused launch, see csrc/dynamic_scaled_quant.cu), timed separately here.
    exchange, peer_ptrs, exchange_note = "none", None, None
    if world > 1:
        exchange = args.exchange
        if exchange == "auto":
            # the single cooperative launch of the separate composition pays off only while part of the shard
            # stays on chip; the shared-read composition has no such limit
            exchange = "p2p" if args.compose == "shared-read" or rows_local * COLS * 2 <= 1.5 * 2**30 else "nccl"
        if exchange == "p2p":
            try:
                from driss_torch_b200.sharded import ShardedQuantizer

                sq = ShardedQuantizer(fused_exchange=True, device=dev)
                peer_ptrs = sq._exchange["ptrs"]
            except Exception as exc:  # symmetric memory unavailable on this box: fall back, and say so
                exchange, exchange_note = "nccl", f"p2p exchange unavailable ({type(exc).__name__}: {exc}); used NCCL"
            ok = torch.tensor([1 if exchange == "p2p" else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if ok.item() == 0:
                exchange = "nccl"
    shared = args.compose == "shared-read"
    if shared:
        first = {"p2p": "mx_fp8_quantize_amax_p2p (MX cast + amax; its one-warp finishing launch exchanges over NVLink)"}.get(
            exchange, "mx_fp8_quantize_amax (MX cast + amax, with its one-warp finishing launch)")
        names = [first] + (["all_reduce(max) [NCCL]"] if exchange == "nccl" else []) + ["cast_with_amax"]
        my_launches_per_step = 3
    elif exchange == "p2p":
        names = ["dynamic_scaled_quant_p2p (amax + NVLink exchange + cast, one launch)", "mx_fp8_quantize"]
        my_launches_per_step = 2
    elif exchange == "nccl":
        names = ["amax", "all_reduce(max) [NCCL]", "cast_with_amax", "mx_fp8_quantize"]
        my_launches_per_step = 3
    else:
        names = ["amax", "cast_with_amax", "mx_fp8_quantize"]
        my_launches_per_step = 3
    epoch = [0]

    def step(events=None):
        marks = []

        def mark():
            if events is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append(e)

        mark()
        if shared:
            epoch[0] += 1
            _cabi.mx_fp8_quantize_amax(x, payload=mx_payload, scales=mx_scales, amax_out=amax, ws=ws,
                                       peer_ptrs=peer_ptrs if exchange == "p2p" else None, rank=rank, epoch=epoch[0])
            mark()
            if exchange == "nccl":
                dist.all_reduce(amax, op=dist.ReduceOp.MAX)
                mark()
            _cabi.cast_with_amax(x, amax, E4M3, out=payload, scale_out=scale)
            mark()
            if events is not None:
                events.append(marks)
            return
        if exchange == "p2p":
            epoch[0] += 1
            _cabi.dynamic_scaled_quant_p2p(x, E4M3, peer_ptrs, rank, epoch[0], out=payload, amax_out=amax,
                                           scale_out=scale, ws=ws)
            mark()
        else:
            _cabi.amax(x, out=amax, ws=ws)
            mark()
            if world > 1:
                dist.all_reduce(amax, op=dist.ReduceOp.MAX)
                mark()
            _cabi.cast_with_amax(x, amax, E4M3, out=payload, scale_out=scale)
            mark()
        _cabi.mx_fp8_quantize(x, payload=mx_payload, scales=mx_scales)
        mark()
        if events is not None:
            events.append(marks)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    # The timed region has no event between the kernels of a step: an event there would make each launch wait
    # for the previous kernel to drain, and the step relies on programmatic dependent launch (the finishing warp
    # and the cast become resident under the tail of the kernel before them).
    t_start, t_end = event_pair()
    t_start.record()
    for _ in range(args.steps):
        step()
    t_end.record()
    barrier()
    elapsed_ms = t_start.elapsed_time(t_end)
    clocks = sampler.stop() if rank == 0 else None
    # per-kernel durations: the same K steps once more, now with an event after every kernel
    barrier()  # rank 0 has just spent time stopping the clock sampler: start together again
    events = []
    m_start, m_end = event_pair()
    m_start.record()
    for _ in range(args.steps):
        step(events)
    m_end.record()
    barrier()
    marked_ms_per_step = m_start.elapsed_time(m_end) / args.steps
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = t.item()
    ms_per_step = elapsed_ms / args.steps

    # per-kernel durations inside the timed region (this rank)
    per_kernel_ms = [statistics.mean(m[i].elapsed_time(m[i + 1]) for m in events) for i in range(len(names))]
    kt = torch.tensor(per_kernel_ms, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(kt, op=dist.ReduceOp.MAX)
    per_kernel_ms = kt.tolist()

    # correctness guard on the timed outputs: a checksum of checksums that every rank contributes to
    # (plain byte sums, so the three numbers are the same for every N: the sharded result is the
    # single-GPU result)
    check = torch.stack([payload.view(torch.uint8).sum(dtype=torch.int64),
                         mx_payload.view(torch.uint8).sum(dtype=torch.int64),
                         mx_scales.view(torch.uint8).sum(dtype=torch.int64)])
    if world > 1:
        dist.all_reduce(check)
    status = _cabi.workspace_status(ws)

    # the timed buffers against the oracle, outside the timed region: the whole matrix at N == 1, rank 0's first
    # chunk otherwise (the other ranks' outputs are covered by the checksums, which the reference arm also prints)
    parity, cpu = None, None
    if rank == 0 and not args.no_cpu:
        parity, cpu = oracle_check_and_cpu_baseline(
            x, payload, mx_payload, mx_scales, amax, scale, check_rows=rows_local if world == 1 else chunk_rows,
            chunk_rows=chunk_rows, whole_matrix=world == 1, time_it=world == 1)
    barrier()

    total_rows = args.rows
    tw_bytes = algorithmic_bytes("dynamic_scaled_quant", total_rows, COLS)
    mx_bytes = algorithmic_bytes("mx_fp8_quantize", total_rows, COLS)
    value = (tw_bytes + mx_bytes) / (ms_per_step * 1e-3) / 1e9

    kernels = []
    for name, ms in zip(names, per_kernel_ms):
        if "NCCL" in name:
            kernels.append({"kernel": name, "ms": round(ms, 4), "bytes": 4})
            continue
        op = ("dynamic_scaled_quant" if name.startswith("dynamic_scaled_quant_p2p")
              else "mx_fp8_quantize" if name.startswith("mx_fp8_quantize") else name)
        nbytes = algorithmic_bytes(op, rows_local, COLS)
        gbs = nbytes / (ms * 1e-3) / 1e9
        k = {"kernel": name, "ms": round(ms, 4), "algorithmic_bytes_per_launch": nbytes, "GBps": round(gbs, 1),
             "frac_of_measured_peak": round(gbs / peak, 4), "frac_of_nominal_8TBps": round(gbs / NOMINAL_HBM_GBS, 4)}
        kernels.append(k)
    mine = [k for k in kernels if "NCCL" not in k["kernel"]]
    dominant = max(mine, key=lambda k: k["ms"])
    roofline = {"bound": "hbm", "kernel": dominant["kernel"], "achieved": dominant["GBps"], "peak": peak,
                "unit": "GB/s", "frac": round(dominant["GBps"] / peak, 4), "peak_kind": f"of {peak_kind}",
                "traffic": None, "frac_of_nominal_8TBps": dominant["frac_of_nominal_8TBps"]}
    tw_ms = sum(k["ms"] for k in mine if not k["kernel"].startswith("mx"))
    if shared:
        step_ms = sum(k["ms"] for k in mine)
        roofline["note"] = ("shared-read composition: the MX cast delivers the amax, so the step reads the input twice, "
                            "N*(2+1+1/32) + N*(2+1) = %d bytes moved per GPU in %.4f ms (%.1f GB/s); the ops' own "
                            "algorithmic bytes (what `value` counts) add up to the same figure, since the amax costs no traffic" % (
                                algorithmic_bytes("mx_fp8_quantize", rows_local, COLS)
                                + algorithmic_bytes("cast_with_amax", rows_local, COLS), step_ms,
                                (algorithmic_bytes("mx_fp8_quantize", rows_local, COLS)
                                 + algorithmic_bytes("cast_with_amax", rows_local, COLS)) / (step_ms * 1e-3) / 1e9))
    else:
        roofline["note"] = ("tensor-wise quant (amax and cast, as one or two launches): together %.4f ms for %d compulsory bytes N*(2+1) "
                        "(%.1f GB/s) and N*(2*2+1) moved (%.1f GB/s); the global-max dependency forces the second read "
                        "of an input this much larger than L2" % (
                            tw_ms, algorithmic_bytes("dynamic_scaled_quant", rows_local, COLS),
                            algorithmic_bytes("dynamic_scaled_quant", rows_local, COLS) / (tw_ms * 1e-3) / 1e9,
                            rows_local * COLS * 5 / (tw_ms * 1e-3) / 1e9))
    # DRAM read+write per launch from the ncu capture summarised in
    # profiles/step_kernels_dram_traffic_512MiB.md, scaled to this launch: what the chip keeps out of
    # DRAM (registers, shared memory, L2) is a constant, not a fraction.
    n_local = rows_local * COLS
    if dominant["kernel"].startswith("dynamic_scaled_quant_p2p"):
        roofline["traffic"] = int(max(3 * n_local, 5 * n_local - 138e6))
    elif dominant["kernel"].startswith("mx_fp8_quantize"):
        roofline["traffic"] = int(3.03125 * n_local - min(54e6, 0.25 * n_local))
    elif dominant["kernel"] == "cast_with_amax":
        roofline["traffic"] = int(3 * n_local - min(34e6, 0.25 * n_local))
    elif dominant["kernel"] == "amax":
        roofline["traffic"] = int(2 * n_local)
    roofline["traffic_source"] = "ncu dram__bytes_read+write on a 512 MiB case, scaled (profiles/step_kernels_dram_traffic_512MiB.md)"

    # ---- end to end: host buffers in, host buffers out ------------------------------------------------
    e2e = None
    if not args.no_e2e:
        del payload, mx_payload, mx_scales
        torch.cuda.empty_cache()
        # Two matrices in flight: matrix k+1's host->device copy runs while matrix k's tensor-wise payload
        # goes back (it cannot leave before the whole input has arrived: the global amax).  Every step still
        # copies its own input in and all its outputs out; each in-flight step has its own host output buffers.
        hq = HostQuantizer(rows_local, COLS, dev, chunk_rows=4096, depth=2)
        xh = torch.empty(x.shape, dtype=torch.bfloat16, pin_memory=True)
        xh.copy_(x)
        host_outs = [(torch.empty(x.shape, dtype=E4M3, pin_memory=True), torch.empty(x.shape, dtype=E4M3, pin_memory=True),
                      torch.empty(x.numel() // 32, dtype=torch.float8_e8m0fnu, pin_memory=True)) for _ in range(2)]
        e2e_steps = max(2, min(args.steps, 6))
        hq.run(xh, *host_outs[0])
        barrier()
        t0 = time.perf_counter()
        prev = None
        for i in range(e2e_steps):
            ticket = hq.submit(xh, *host_outs[i % 2])
            if prev is not None:
                hq.wait(prev)
            prev = ticket
        hq.wait(prev)
        barrier()
        ph, mph, msh = host_outs[(e2e_steps - 1) % 2]
        wall = (time.perf_counter() - t0) / e2e_steps
        tt = torch.tensor([wall], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        wall = tt.item()
        e2e_sums = [t_.view(torch.uint8).sum(dtype=torch.int64) for t_ in (ph, mph, msh)]
        # the PCIe bound of the same pipeline: the same pinned buffers, chunks, streams and dependencies, no kernels
        copy_outs = host_outs[e2e_steps % 2]
        hq.wait(hq.submit(xh, *copy_outs, copies_only=True))
        barrier()
        t0 = time.perf_counter()
        prev = None
        for i in range(e2e_steps):
            ticket = hq.submit(xh, *copy_outs, copies_only=True)
            if prev is not None:
                hq.wait(prev)
            prev = ticket
        hq.wait(prev)
        barrier()
        copy_wall = (time.perf_counter() - t0) / e2e_steps
        tt = torch.tensor([copy_wall], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        copy_wall = tt.item()
        h2d = x.numel() * 2
        d2h = x.numel() * 2 + x.numel() // 32
        e2e = {"value": round((tw_bytes + mx_bytes) / wall / 1e9, 2), "unit": "GB/s", "ms_per_step": round(wall * 1e3, 3),
               "steps": e2e_steps, "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
               "launches_per_step": hq.launches,
               "copy_bound_ms": round(copy_wall * 1e3, 3), "frac_of_copy_bound": round(copy_wall / wall, 4),
               "copy_bound_note": "the same pinned buffers, chunks, three streams and dependencies with the kernels left "
                                  "out: what the host<->device copies alone take per step",
               "api": "driss_torch_b200.host_pipeline.HostQuantizer.submit/wait, two matrices in flight (pinned host tensors in and out)"}
        e2e_check = torch.stack(e2e_sums).to(dev)
        if world > 1:
            dist.all_reduce(e2e_check)
        e2e["matches_device_run"] = bool(torch.equal(e2e_check, check))
        del hq, xh, ph, mph, msh, host_outs

    ops = None
    if world == 1 and not args.no_ops_table:
        del x
        torch.cuda.empty_cache()
        ops = per_op_table(dev, peak, iters=args.op_iters or max(20, args.steps))
        ops += gemm_table(dev, iters=args.op_iters or max(20, args.steps))

    if rank == 0:
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16->fp8 (f64 scale arithmetic)",
            "data": "synthetic",
            "config": {"workload": f"cfg5: bf16 [{total_rows},{COLS}] row-sharded over {world} GPU(s); tensor-wise e4m3 "
                                   "quant (amax -> max all-reduce -> cast) + MX block-32 cast",
                       "composition": args.compose,
                       "rows_per_gpu": rows_local, "exchange": exchange, "l2": "inputs larger than L2 (no flush needed)",
                       "timing": "CUDA events on the launch stream, max over ranks"},
            "bytes_per_step": tw_bytes + mx_bytes,
            "frac_of_measured_peak": round(value / (peak * world), 4),
            "frac_of_nominal_8TBps": round(value / (NOMINAL_HBM_GBS * world), 4),
            "roofline": roofline, "kernels": kernels,
            "kernels_note": "per-kernel ms: a second pass of the same steps with an event after every kernel, which "
                            f"serialises the launches ({marked_ms_per_step:.4f} ms per step that way); the timed region "
                            "has no events inside a step",
            "clocks": clocks,
            "gpu_launches": my_launches_per_step * args.steps,
            "device_status": status, "output_checksums": check.tolist(),
        }
        if exchange_note:
            out["config"]["exchange_note"] = exchange_note
        if e2e is not None:
            out["e2e"] = e2e
        if ops is not None:
            out["ops"] = ops
        if parity is not None:
            out["parity_checked"] = parity
        if cpu is not None:
            out["cpu_baseline"] = cpu
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
