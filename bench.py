#!/usr/bin/env python
"""Benchmark of the MXFP8 linear hot path: MX quantisation + block-scaled GEMM.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: the four Llama-3-8B linear shapes at M = 16384 tokens (QKV 4096->6144, O 4096->4096,
fused gate+up 4096->28672, down 14336->4096), bf16 activations N(0,1), weights N(0,0.02),
synthetic and seeded.  One step = for each of the four layers: quantise X row-wise, quantise the
weight (shard) row-wise, run the block-scaled GEMM.  The layers are independent problems: each GEMM is
issued before the next layer's quantisers, which may start while it runs (DW_QUANT_OVERLAP_PREVIOUS;
--serial: every launch after the previous one has finished).
With N GPUs every weight is sharded along its output dimension across the ranks and X is replicated, so
the total work is fixed: strong scaling.  The ranks share the quantisation of X (each quantises 1/N of
the rows and copies its slice into every peer's operand buffer over NVLink with the copy engines, under the
GEMMs: deepwell_b200/exchange.py; --no-exchange: every rank quantises all of X itself, no data-path
collective); a rank's slices and weight shards are quantised by one launch (dw_mxfp8_quantize_rows_batch).

Prints ONE JSON line (rank 0).  Keys beyond the basic contract:
  value              whole-job TFLOP/s with inputs resident in HBM (CUDA events, max over ranks)
  e2e                the same through the public API (cutlass_kernels.BlackwellGemmKernel.gemm) with pinned host
                     buffers: the host->device copy of every X and the device->host copy of every Y inside the timed
                     region, on their own streams
  roofline           the GEMM, measured live with CUDA events around every GEMM launch of the timed region
                     (`achieved_alone`: the same launches with nothing else on the GPU); both fractions, of 2 x the
                     measured bf16 burst rate and of 2 x the measured sustained rate; `frac` is the one that fits the run
  sustained          the same step repeated for >= 2.5 s with the SM clock sampled throughout: the steady state under
                     the power cap, which the short timed region does not reach
  roofline_quantize  the row quantiser on the largest activation, against the measured copy bandwidth
  vendor_gemm        the vendor's block-scaled GEMM (torch._scaled_mm) alternated with ours on the same operands
  gpt2_mlp, swiglu_mlp, decoder_step   secondary workloads (GPT-2-small MLP forward+backward; the Llama-3-8B gated MLP
                     with and without the SwiGLU epilogue; the end-to-end optimize() training step of a 12-layer
                     decoder), each beside the same layers in bf16 (N = 1 only)
  exchange           N > 1: how the quantisation of X was shared (rows per layer, bytes pushed per step, the budgets
                     tried) and `parity`: the assembled operands against the rank's own quantisation of all of X
  with_gather, sharded     N > 1: the step with every layer's output all-gathered over NVLink (by NCCL, and by the copy
                     engines: `copy_engines`, checked against the NCCL result), and a parity check of
                     ColumnParallelDWLinear / RowParallelDWLinear under NCCL against the unsharded layer
  cpu_baseline       the CPU restatement of the same path on the host cores (rank 0, N = 1)

--impl reference times only that CPU path (the reference ships no GPU implementation of an MXFP8 GEMM; its CPU path
for the GEMM stage is a Python module calling torch.matmul, which is loaded from an install of the reference under
baseline/_ref when that is present).

Other modes (each prints its own JSON): --workload decoder_step, --sweep-quantize (quantise-only bandwidth sweep),
--compare-vendor, --probe-corun (what runs beside the GEMM), --profile-case (a few launches of one kernel on a small
case, for an ncu capture),
--traffic-from-csv (turns an ncu CSV of the GEMM launches into bench_gemm_dram_traffic.json),
--emulate-world W (tuning aid: rank 0's shard sizes of a W-GPU job on one GPU).
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS = [("qkv", 4096, 6144), ("o", 4096, 4096), ("gate_up", 4096, 28672), ("down", 14336, 4096)]   # (name, K, N)
M_TOKENS = 16384
METRIC = "mxfp8_quant_gemm_tflops"
WORKLOAD = "llama3_8b_linears_M16384"
CPU_SAMPLE_ROWS = 4096
NOMINAL_MXFP8_TFLOPS = 4500.0
TRAFFIC_JSON = os.path.join(ROOT, "bench_gemm_dram_traffic.json")
REFERENCE_GEMM_MODULE = os.path.join(ROOT, "baseline", "_ref", "deepwell", "cutlass_kernels.py")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def gemm_dram_traffic():
    """Mean DRAM bytes (read + write) per GEMM launch of one step at N = 1, from the ncu capture recorded in
    bench_gemm_dram_traffic.json (written by --traffic-from-csv); None when that file is absent."""
    if not os.path.exists(TRAFFIC_JSON):
        return None, None
    with open(TRAFFIC_JSON) as f:
        t = json.load(f)
    per_layer = {k: v["dram_read_bytes"] + v["dram_write_bytes"] for k, v in t["layers"].items()}
    return sum(per_layer.values()) / max(1, len(per_layer)), t


def total_flops(m=M_TOKENS):
    return sum(2.0 * m * k * n for _, k, n in LAYERS)


# ----------------------------------------------------------------------------------------------
# clocks during the timed region
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML every 5 ms."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self._stop, self.ok = [], set(), None, threading.Event(), False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.ok:
            self.thread.start()

    def stop(self):
        self._stop.set()
        if self.ok:
            self.thread.join(timeout=1.0)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------
# CPU path (oracle): the reference arm and the cpu_baseline leg
# ----------------------------------------------------------------------------------------------
_ref_gemm_kernel = None


def reference_gemm_kernel():
    """BlackwellGemmKernel of the reference's own CPU module (src/deepwell/cutlass_kernels.py:9-55 of the reference,
    whose gemm is alpha * torch.matmul(a, b) + beta * c), loaded by path from an install of the reference under
    baseline/_ref; None when no such install travelled with the repository."""
    global _ref_gemm_kernel
    if _ref_gemm_kernel is None and os.path.exists(REFERENCE_GEMM_MODULE):
        import importlib.util
        spec = importlib.util.spec_from_file_location("_reference_cutlass_kernels", REFERENCE_GEMM_MODULE)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ref_gemm_kernel = mod.BlackwellGemmKernel()
    return _ref_gemm_kernel


def cpu_step(inputs):
    """One pass of the CPU path over the sample: quantise X and W (the C restatement with OpenMP: the reference has no
    CPU quantiser), dequantise, then the GEMM stage in fp32 on all host threads through the reference's own CPU module
    when it is installed (torch.matmul either way), bf16 output."""
    from oracle import mx_ref as c
    kern = reference_gemm_kernel()
    out = []
    for xb, wb in inputs:
        xc, xs = c.quantize_rowwise(xb, 0)
        wc, ws = c.quantize_rowwise(wb, 0)
        a = torch.from_numpy(c.dequantize(xc, xs))
        b = torch.from_numpy(c.dequantize(wc, ws))
        y = kern.gemm(a, b.t()) if kern is not None else torch.matmul(a, b.t())
        out.append(y.bfloat16())
    return out


def cpu_inputs(rows):
    from oracle import mx_oracle as o
    g = torch.Generator("cpu").manual_seed(3456)
    items = []
    for _, k, n in LAYERS:
        x = torch.randn(rows, k, generator=g).bfloat16()
        w = (torch.randn(n, k, generator=g) * 0.02).bfloat16()
        items.append((o.torch_bf16_bits(x), o.torch_bf16_bits(w)))
    return items


def time_cpu(steps, warmup, rows=CPU_SAMPLE_ROWS):
    from oracle import mx_ref as c
    c.build()
    inputs = cpu_inputs(rows)
    for _ in range(warmup):
        cpu_step(inputs)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(inputs)
    dt = (time.perf_counter() - t0) / max(1, steps)
    cores = max(torch.get_num_threads(), c.num_threads())
    ref_gemm = reference_gemm_kernel() is not None
    return {"value": total_flops(rows) / dt / 1e12, "unit": "TFLOP/s", "cores": cores,
            "kind": "reference" if ref_gemm else "port",
            "sample": f"first {rows} of {M_TOKENS} token rows of all four layers (full N and K), {dt:.2f} s per pass: "
                      "C/OpenMP restatement of the quantiser (the reference has no CPU quantiser) + GEMM stage in fp32 "
                      "on the dequantised operands through "
                      + ("the reference's own CPU module deepwell/cutlass_kernels.py (BlackwellGemmKernel.gemm = "
                         "torch.matmul)" if ref_gemm else "torch.matmul (what the reference's CPU module calls)")}, dt


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core it may run on."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(n)          # read by the C restatement's OpenMP runtime when it loads
    torch.set_num_threads(n)
    return n


def run_reference_arm(args, rank):
    if rank != 0:
        return
    use_all_host_threads()
    cb, dt = time_cpu(args.steps, args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "mxfp8(e4m3+e8m0), fp32 accumulate", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample_rows": CPU_SAMPLE_ROWS, "layers": [l[0] for l in LAYERS]},
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# small single-kernel cases for profiler captures (inputs larger than L2, well under 1 GB)
# ----------------------------------------------------------------------------------------------
def run_profile_case(args):
    from deepwell_b200 import _native as nv
    L = nv.load()
    nv.set_gemm_variant(args.variant)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    g = torch.Generator(device=dev).manual_seed(1)
    u8 = lambda *s: torch.empty(*s, dtype=torch.uint8, device=dev)
    if args.profile_case == "gemm":
        M, N, K = 8192, 8192, 4096
        x = torch.randn(M, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
        xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
        wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        sw = nv.status_word(dev)
        run = lambda: L.dw_mxfp8_gemm(xc.data_ptr(), xs.data_ptr(), wc.data_ptr(), ws.data_ptr(), y.data_ptr(), None,
                                      M, N, K, 1.0, 0.0, None, 0, sw.data_ptr(), st)
        units = f"gemm M={M} N={N} K={K}: {2.0 * M * N * K / 1e9:.1f} GFLOP per launch"
    elif args.profile_case == "quant_batch":
        # what one rank of a 4-GPU job quantises per step in one launch: its quarter of the rows of the four activations
        # and its quarter of the four weights (dw_mxfp8_quantize_rows_batch)
        import ctypes
        shapes = [(M_TOKENS // 4, k) for _, k, _ in LAYERS] + [(n // 4, k) for _, k, n in LAYERS]
        xs_ = [torch.randn(r, c, device=dev, generator=g).bfloat16() for r, c in shapes]
        cs_ = [u8(r, c) for r, c in shapes]
        ss_ = [u8(nv.scale_bytes(r, c, 1)) for r, c in shapes]
        n = len(shapes)
        P, I = ctypes.c_void_p * n, ctypes.c_int64 * n
        a = (P(*[t.data_ptr() for t in xs_]), P(*[t.data_ptr() for t in cs_]), P(*[t.data_ptr() for t in ss_]),
             I(*[r for r, _ in shapes]), I(*[c for _, c in shapes]))
        run = lambda: L.dw_mxfp8_quantize_rows_batch(n, a[0], a[1], a[2], a[3], a[4], 0, 1, 0, st)
        units = f"quant_batch {n} matrices: {sum(r * c for r, c in shapes) * 3.03125 / 1e6:.1f} MB algorithmic per launch"
    else:
        # quant_col_long: 2^21 rows, the transposed payload's rows 2 MiB apart (staged write-out)
        R, C = ((1 << 21), 128) if args.profile_case == "quant_col_long" else (16384, 8192)
        x = torch.randn(R, C, device=dev, generator=g).bfloat16()
        cr, ct = u8(R, C), u8(C, R)
        sr, sc = u8(nv.scale_bytes(R, C, 1)), u8(nv.scale_bytes(C, R, 1))
        if args.profile_case == "quant_row":
            run = lambda: L.dw_mxfp8_quantize(x.data_ptr(), cr.data_ptr(), sr.data_ptr(), R, C, 0, 0, 1, st)
            bpe = 3.03125
        elif args.profile_case in ("quant_col", "quant_col_long"):
            run = lambda: L.dw_mxfp8_quantize(x.data_ptr(), ct.data_ptr(), sc.data_ptr(), R, C, 1, 0, 1, st)
            bpe = 3.03125
        else:
            run = lambda: L.dw_mxfp8_quantize_both(x.data_ptr(), cr.data_ptr(), sr.data_ptr(), ct.data_ptr(),
                                                   sc.data_ptr(), R, C, 0, 1, st)
            bpe = 4.0625
        units = f"{args.profile_case} {R}x{C}: {R * C * bpe / 1e6:.1f} MB algorithmic per launch"
    for _ in range(3):
        assert run() == 0
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        assert run() == 0
    e1.record()
    torch.cuda.synchronize(dev)
    print(json.dumps({"profile_case": args.profile_case, "units": units, "ms_per_launch": e0.elapsed_time(e1) / 3}))


def traffic_from_csv(path):
    """Reads an ncu --csv launch log holding dram__bytes_read.sum, dram__bytes_write.sum and gpu__time_duration.sum of
    the four GEMM launches of one step (in layer order) and writes bench_gemm_dram_traffic.json, the one place the
    bench line's `roofline.traffic` comes from."""
    rows = []
    with open(path, newline="") as f:
        lines = [l for l in f if l.startswith('"')]
    for rec in csv.DictReader(lines):
        rows.append(rec)
    per_launch = {}
    for rec in rows:
        lid = int(rec["ID"])
        d = per_launch.setdefault(lid, {"kernel": rec["Kernel Name"], "block": rec.get("Block Size", ""), "grid": rec.get("Grid Size", "")})
        val = float(rec["Metric Value"].replace(",", ""))
        unit = rec["Metric Unit"]
        name = rec["Metric Name"]
        if name.startswith("dram__bytes"):
            val *= {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(unit, 1.0)
            d["dram_read_bytes" if "read" in name else "dram_write_bytes"] = val
        elif name.startswith("gpu__time_duration"):
            val *= {"ns": 1e-3, "us": 1.0, "usecond": 1.0, "ms": 1e3, "msecond": 1e3, "nsecond": 1e-3}.get(unit, 1.0)
            d["duration_us"] = val
    launches = [per_launch[k] for k in sorted(per_launch)]
    if len(launches) != len(LAYERS):
        raise SystemExit(f"expected {len(LAYERS)} GEMM launches in {path}, found {len(launches)}")
    out = {"source": "ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum --clock-control none "
                     "-k regex:mx_gemm on `python bench.py --steps 1 --warmup 3 --serial --e2e-steps 0 --sustained-seconds 0 "
                     "--no-cpu-baseline --no-extra-legs`, the four GEMM launches of the last step",
           "M": M_TOKENS, "layers": {}}
    for (name, k, n), l in zip(LAYERS, launches):
        alg = M_TOKENS * k + n * k + 2 * M_TOKENS * n
        out["layers"][name] = {"K": k, "N": n, "kernel": l["kernel"], "block": l["block"], "grid": l["grid"],
                               "duration_us": l.get("duration_us"), "dram_read_bytes": l["dram_read_bytes"],
                               "dram_write_bytes": l["dram_write_bytes"], "algorithmic_bytes": alg,
                               "ratio": (l["dram_read_bytes"] + l["dram_write_bytes"]) / alg}
    with open(TRAFFIC_JSON, "w") as f:
        json.dump(out, f, indent=1)
    print(json.dumps(out))


# ----------------------------------------------------------------------------------------------
# quantise-only sweep: Student-t(3) x 0.5 inputs, K in {128, 1024, 4096, 16384}, 2^20 .. 2^32 elements
# ----------------------------------------------------------------------------------------------
def run_quantize_sweep(args):
    from deepwell_b200 import _native as nv
    L = nv.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    peak = measured_peaks()["hbm_gbs"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)           # larger than L2
    g = torch.Generator(device=dev).manual_seed(4567)
    rows_out = []
    lo, hi = args.sweep_log2_min, args.sweep_log2_max
    for log2n in range(lo, hi + 1, 2):
        n = 1 << log2n
        # one buffer per size, re-viewed for every K (values are i.i.d., the shape does not matter to them)
        x_flat = torch.empty(n, dtype=torch.bfloat16, device=dev)
        step_elems = min(n, 1 << 26)
        for off in range(0, n, step_elems):
            z = torch.randn(step_elems, device=dev, generator=g)
            v = torch.distributions.Chi2(torch.tensor(3.0, device=dev)).sample((step_elems,))
            x_flat[off:off + step_elems] = (0.5 * z / torch.sqrt(v / 3)).bfloat16()
            del z, v
        codes = torch.empty(n, dtype=torch.uint8, device=dev)
        for k in (128, 1024, 4096, 16384):
            r = n // k
            if r < 32:
                continue
            for name, direction in (("row", nv.DIR_ROW), ("col", nv.DIR_COL_T)):
                scales = torch.empty(nv.scale_bytes(r if direction == nv.DIR_ROW else k, k if direction == nv.DIR_ROW else r,
                                                    nv.SF_TILED), dtype=torch.uint8, device=dev)
                run = lambda: nv.check(L.dw_mxfp8_quantize(x_flat.data_ptr(), codes.data_ptr(), scales.data_ptr(), r, k,
                                                           direction, 0, nv.SF_TILED, st), "quantize")
                small = n * 3 < (256 << 20)                  # working set could sit in L2: flush between launches
                reps = 5 if log2n >= 28 else 20
                for _ in range(3):
                    run()
                times = []
                for _ in range(reps):
                    if small:
                        flush.zero_()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    run()
                    e1.record()
                    torch.cuda.synchronize(dev)
                    times.append(e0.elapsed_time(e1))
                ms = float(np.median(times))
                gbs = n * 3.03125 / (ms * 1e-3) / 1e9
                # the same launch back to back (no flush, no host round trip between launches): what a training step sees
                b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                b0.record()
                for _ in range(reps):
                    run()
                b1.record()
                torch.cuda.synchronize(dev)
                ms_b2b = b0.elapsed_time(b1) / reps
                gbs_b2b = n * 3.03125 / (ms_b2b * 1e-3) / 1e9
                rows_out.append({"log2_elements": log2n, "K": k, "direction": name, "us": ms * 1e3, "GBps": gbs,
                                 "frac_of_measured_copy": gbs / peak, "l2_flushed": small, "us_back_to_back": ms_b2b * 1e3,
                                 "GBps_back_to_back": gbs_b2b, "frac_back_to_back": gbs_b2b / peak})
                print(json.dumps(rows_out[-1]), flush=True)
        del x_flat, codes
    print(json.dumps({"sweep": "quantize", "peak_hbm_gbs": peak, "points": len(rows_out)}))


# ----------------------------------------------------------------------------------------------
# vendor comparison: cuBLASLt's block-scaled GEMM (through torch._scaled_mm) alternated with ours
# ----------------------------------------------------------------------------------------------
def compare_vendor(dev, shapes, rounds=3, reps=10):
    """Per shape: `rounds` alternations of (vendor x reps, ours x reps) on the same quantised operands, CUDA events.
    The vendor kernel reads the same codes and the same tiled E8M0 scale buffers (its scale layout is this one)."""
    from deepwell_b200 import _native as nv
    out = {}
    for name, (M, N, K) in shapes.items():
        g = torch.Generator(device=dev).manual_seed(M + N + K)
        x = torch.randn(M, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
        xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
        wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
        del x, w
        sa, sb = xs.view(torch.float8_e8m0fnu), ws.view(torch.float8_e8m0fnu)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        f_vendor = lambda: torch._scaled_mm(xc, wc.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
        f_ours = lambda: nv.gemm(xc, xs, wc, ws, out=y)
        try:
            yv = f_vendor()
        except Exception as e:        # a torch build without the block-scaled path
            out[name] = {"error": f"vendor kernel unavailable: {type(e).__name__}: {str(e)[:120]}"}
            continue
        f_ours()
        identical = bool(torch.equal(yv, y))
        del yv

        def timed(fn):
            for _ in range(2):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fn()
            e1.record()
            torch.cuda.synchronize(dev)
            return e0.elapsed_time(e1) / reps

        flops = 2.0 * M * N * K
        v, u = [], []
        for _ in range(rounds):
            v.append(flops / (timed(f_vendor) * 1e-3) / 1e12)
            u.append(flops / (timed(f_ours) * 1e-3) / 1e12)
        out[name] = {"shape": [M, N, K], "vendor_tflops": [round(t, 1) for t in v], "ours_tflops": [round(t, 1) for t in u],
                     "ours_over_vendor": float(np.median(u) / np.median(v)), "outputs_identical": identical}
        del xc, xs, wc, ws, y
    return out


def run_compare_vendor(args):
    from deepwell_b200 import _native as nv
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    nv.load()
    nv.set_gemm_variant(args.variant)
    shapes = {name: (M_TOKENS, n, k) for name, k, n in LAYERS}
    shapes.update({"gpt2_fc": (8192, 3072, 768), "gpt2_proj": (8192, 768, 3072), "square_8192x4096": (8192, 8192, 4096)})
    sampler = ClockSampler(0)
    sampler.start()
    res = compare_vendor(dev, shapes, rounds=5, reps=20)
    print(json.dumps({"compare": "vendor block-scaled GEMM (torch._scaled_mm) vs dw_mxfp8_gemm, alternated, TFLOP/s",
                      "shapes": res, "clocks": sampler.stop()}))


# ----------------------------------------------------------------------------------------------
# what runs beside the GEMM?  (evidence for the step's launch order)
# ----------------------------------------------------------------------------------------------
def run_probe_corun(args):
    """Stream A: one long GEMM.  Stream B, released when A reaches the GEMM: a one-block kernel, a 256 MB device copy, the
    row quantiser of a 16384 x 14336 activation.  Reported: when B's work was done, counted from the start of the GEMM,
    beside the durations of both alone; for the quantiser also the single-stream order GEMM -> quantiser with and
    without DW_QUANT_OVERLAP_PREVIOUS.  The first GEMM shape occupies 64 of the 74 CTA pairs (20 SMs free), the others all."""
    from deepwell_b200 import _native as nv
    L = nv.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lo, hi = torch.cuda.Stream.priority_range()
    sw = nv.status_word(dev)
    QM, QK = 16384, 14336
    qx = torch.randn(QM, QK, device=dev).bfloat16()
    qc = torch.empty(QM, QK, dtype=torch.uint8, device=dev)
    qs = torch.empty(nv.scale_bytes(QM, QK, nv.SF_TILED), dtype=torch.uint8, device=dev)
    small = torch.zeros(32, device=dev)
    big_src = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    big_dst = torch.empty_like(big_src)

    def alone(fn, st, n=5):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(n):
            fn()
        e1.record(st)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n * 1e3

    def median(v):
        return sorted(v)[len(v) // 2]

    rows = []
    for (M, N, K) in [(32768, 768, 14336), (16384, 28672, 4096), (16384, 4096, 14336)]:
        g = torch.Generator(device=dev).manual_seed(M + N)
        x = torch.randn(M, K, device=dev, generator=g).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=g) * 0.02).bfloat16()
        xc, xs = nv.quantize(x, nv.DIR_ROW, 0, nv.SF_TILED)
        wc, ws = nv.quantize(w, nv.DIR_ROW, 0, nv.SF_TILED)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        del x, w
        sa, sb = torch.cuda.Stream(dev, priority=hi), torch.cuda.Stream(dev, priority=lo)
        gemm = lambda s: nv.check(L.dw_mxfp8_gemm(xc.data_ptr(), xs.data_ptr(), wc.data_ptr(), ws.data_ptr(), y.data_ptr(), None,
                                                  M, N, K, 1.0, 0.0, None, 0, sw.data_ptr(), s.cuda_stream), "gemm")

        def work(kind, s, flags=0):
            with torch.cuda.stream(s):
                if kind == "one_block_kernel":
                    small.add_(1.0)
                elif kind == "copy_256MB":
                    big_dst.copy_(big_src)
                else:
                    nv.check(L.dw_mxfp8_quantize_ex(qx.data_ptr(), qc.data_ptr(), qs.data_ptr(), QM, QK, nv.DIR_ROW, 0, nv.SF_TILED,
                                                    flags, s.cuda_stream), "quantize")

        gemm_alone = alone(lambda: gemm(sa), sa)
        for kind in ("one_block_kernel", "copy_256MB", "quantize_rowwise"):
            b_alone = alone(lambda: work(kind, sb), sb)
            tg, tb = [], []
            for _ in range(5):
                torch.cuda.synchronize()
                a0, a1, b1 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                a0.record(sa)
                gemm(sa)
                a1.record(sa)
                sb.wait_event(a0)
                work(kind, sb)
                b1.record(sb)
                torch.cuda.synchronize()
                tg.append(a0.elapsed_time(a1) * 1e3)
                tb.append(a0.elapsed_time(b1) * 1e3)
            row = {"gemm": [M, N, K], "gemm_alone_us": round(gemm_alone, 1), "other_work": kind, "other_alone_us": round(b_alone, 1),
                   "second_stream": {"gemm_us": round(median(tg), 1), "other_done_at_us": round(median(tb), 1)}}
            if kind == "quantize_rowwise":
                for name, flags in (("same_stream_overlap_previous", nv.QUANT_OVERLAP_PREVIOUS), ("same_stream_plain", 0)):
                    t = []
                    for _ in range(5):
                        torch.cuda.synchronize()
                        a0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        a0.record(sa)
                        gemm(sa)
                        work(kind, sa, flags)
                        b1.record(sa)
                        torch.cuda.synchronize()
                        t.append(a0.elapsed_time(b1) * 1e3)
                    row[name] = {"both_done_at_us": round(median(t), 1)}
            rows.append(row)
            print(json.dumps(row), flush=True)
        del xc, xs, wc, ws, y
    nv.check_status(dev)
    print(json.dumps({"probe": "corun", "cases": len(rows)}))


# ----------------------------------------------------------------------------------------------
# Secondary workloads
# ----------------------------------------------------------------------------------------------
def build_decoder(vocab, hidden, heads, ffn, layers):
    import torch.nn as nn
    import torch.nn.functional as F

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln1, self.ln2 = nn.LayerNorm(hidden), nn.LayerNorm(hidden)
            self.qkv, self.proj = nn.Linear(hidden, 3 * hidden), nn.Linear(hidden, hidden)
            self.up, self.down = nn.Linear(hidden, ffn), nn.Linear(ffn, hidden)

        def forward(self, x):
            b, s, h = x.shape
            q, k, v = self.qkv(self.ln1(x)).view(b, s, 3, heads, h // heads).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
            x = x + self.proj(a.transpose(1, 2).reshape(b, s, h))
            return x + self.down(F.gelu(self.up(self.ln2(x))))

    class Decoder(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(vocab, hidden)
            self.blocks = nn.ModuleList([Block() for _ in range(layers)])
            self.ln_f = nn.LayerNorm(hidden)
            self.head = nn.Linear(hidden, vocab, bias=False)

        def forward(self, ids):
            x = self.embed(ids)
            for blk in self.blocks:
                x = blk(x)
            return self.head(self.ln_f(x))

    return Decoder()


def decoder_step_numbers(steps, warmup):
    """End-to-end optimize() training step: random-init 12-layer pre-LN decoder (hidden 1024, 16 heads, FFN 4096, vocab
    32000), batch 8 x sequence 2048 uniform token ids; every nn.Linear replaced by deepwell.optimize(precision='mxfp8').
    One step = ids host->device, forward, cross-entropy, backward, fused AdamW step, loss device->host.  The same
    model with its bf16 nn.Linear layers is timed beside it.  Attention (torch SDPA), LayerNorm, GELU, the loss and the
    optimizer are PyTorch's own in both arms: only the linear layers differ."""
    import copy
    import torch.nn.functional as F
    import deepwell_b200 as dw

    vocab, hidden, heads, ffn, layers, batch, seq = 32000, 1024, 16, 4096, 12, 8, 2048
    torch.manual_seed(1234)
    base = build_decoder(vocab, hidden, heads, ffn, layers).cuda().bfloat16()
    arms = {"bf16_nn_linear": copy.deepcopy(base), "mxfp8_dwlinear": dw.optimize(copy.deepcopy(base), precision="mxfp8", verbose=False)}
    del base
    n_dw = sum(isinstance(m, dw.DWLinear) for m in arms["mxfp8_dwlinear"].modules())
    lin_params = sum(m.weight.numel() for m in arms["mxfp8_dwlinear"].modules() if isinstance(m, dw.DWLinear))
    ids_host = torch.randint(0, vocab, (steps + warmup, batch, seq), generator=torch.Generator().manual_seed(7)).pin_memory()
    out, losses = {}, {}
    for name, net in arms.items():
        opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = []
        for i in range(steps + warmup):
            if i == warmup:
                torch.cuda.synchronize()
                ev0.record()
            ids = ids_host[i].cuda(non_blocking=True)
            opt.zero_grad(set_to_none=True)
            logits = net(ids)
            loss = F.cross_entropy(logits[:, :-1].reshape(-1, vocab).float(), ids[:, 1:].reshape(-1))
            loss.backward()
            opt.step()
            cur.append(loss.item())
        ev1.record()
        torch.cuda.synchronize()
        out[name] = ev0.elapsed_time(ev1) / steps
        losses[name] = cur
        del opt, logits, loss
        arms[name] = None
        torch.cuda.empty_cache()
    tokens = batch * seq
    ms = out["mxfp8_dwlinear"]
    return {"workload": "preln_decoder_12x1024_ffn4096_vocab32000_b8_s2048_train_step", "steps": steps, "warmup": warmup,
            "tokens_per_s": tokens / ms * 1e3, "ms_per_step": ms, "dwlinear_modules": n_dw,
            "linear_tflop_per_step": 6.0 * lin_params * tokens / 1e12, "optimizer": "AdamW(fused)",
            "bf16_nn_linear": {"ms_per_step": out["bf16_nn_linear"], "tokens_per_s": tokens / out["bf16_nn_linear"] * 1e3},
            "speedup_vs_bf16_nn_linear": out["bf16_nn_linear"] / ms,
            "loss_first_last": {k: [v[0], v[-1]] for k, v in losses.items()},
            "h2d_bytes_per_step": tokens * 8, "d2h_bytes_per_step": 4}


def run_decoder_step(args):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for the product path")
    torch.cuda.set_device(0)
    sampler = ClockSampler(0)
    sampler.start()
    r = decoder_step_numbers(args.steps, args.warmup)
    clocks = sampler.stop()
    print(json.dumps({
        "metric": "decoder_train_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "mxfp8 linears (e4m3+e8m0, fp32 accumulate), bf16 elsewhere", "data": "synthetic",
        "config": {"workload": r["workload"], "dwlinear_modules": r["dwlinear_modules"],
                   "linear_tflop_per_step": r["linear_tflop_per_step"], "optimizer": r["optimizer"],
                   "l2": "activations and weights far larger than L2"},
        "bf16_nn_linear": r["bf16_nn_linear"], "speedup_vs_bf16_nn_linear": r["speedup_vs_bf16_nn_linear"],
        "loss_first_last": r["loss_first_last"],
        "e2e": {"value": r["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                "d2h_bytes_per_step": r["d2h_bytes_per_step"],
                "api": "deepwell_b200.optimize(model, precision='mxfp8'); ids host->device and loss.item() every step"},
        "clocks": clocks}))


def gpt2_mlp_numbers(reps=30):
    """GPT-2-small MLP linears, forward + backward, 8 x 1024 = 8192 tokens: 768 -> 3072 and 3072 -> 768, bf16 weights
    N(0,0.02), activations and output gradients N(0,1).  DWLinear (three MXFP8 GEMMs + the quantisers per layer)
    beside bf16 nn.Linear, microseconds per forward+backward, CUDA events over `reps` iterations after warm-up."""
    import torch.nn as nn
    import deepwell_b200 as dw
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(2345)
    res = {}
    for name, k, n in (("fc_768_3072", 768, 3072), ("proj_3072_768", 3072, 768)):
        lin = nn.Linear(k, n, bias=True).to(dev).bfloat16()
        with torch.no_grad():
            lin.weight.copy_((torch.randn(n, k, device=dev, generator=g) * 0.02).bfloat16())
        mx = dw.DWLinear.from_linear(lin)
        x = torch.randn(8192, k, device=dev, generator=g).bfloat16().requires_grad_(True)
        gy = torch.randn(8192, n, device=dev, generator=g).bfloat16()

        def fb(layer):
            x.grad = None
            layer.weight.grad = None
            layer.bias.grad = None
            layer(x).backward(gy)

        times = {}
        for arm, layer in (("bf16_nn_linear_us", lin), ("mxfp8_dwlinear_us", mx)):
            for _ in range(5):
                fb(layer)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                fb(layer)
            e1.record()
            torch.cuda.synchronize(dev)
            times[arm] = e0.elapsed_time(e1) / reps * 1e3
        times["speedup_vs_bf16"] = times["bf16_nn_linear_us"] / times["mxfp8_dwlinear_us"]
        times["gflop_fwd_bwd"] = 6.0 * 8192 * k * n / 1e9
        res[name] = times
    res["tokens"] = 8192
    res["note"] = "forward + backward of one layer, eager (one Python->C++ call per direction), inputs resident in HBM"
    return res


def swiglu_mlp_numbers(reps=10):
    """The Llama-3-8B MLP at 16384 tokens (hidden 4096, intermediate 14336), forward without autograd: gate+up projection,
    silu(gate) * up, down projection.  Fused: one quantiser launch and two GEMMs, the gated product formed in the first
    GEMM's epilogue and written as the second GEMM's quantised operand (FusedSwiGLUMLP).  Unfused: the same module with
    three MXFP8 layers and torch's silu and product in bf16 between them.  Beside both, three bf16 nn.Linear layers."""
    import torch.nn as nn
    import torch.nn.functional as F
    from deepwell_b200.kernels.blackwell_production import FusedSwiGLUMLP
    dev = torch.device("cuda", torch.cuda.current_device())
    h, f, m = 4096, 14336, M_TOKENS
    torch.manual_seed(99)
    mlp = FusedSwiGLUMLP(h, f).to(dev)
    with torch.no_grad():
        for lin in (mlp.gate_proj, mlp.up_proj, mlp.down_proj):
            lin.weight.normal_(0.0, 0.02)
    x = torch.randn(m, h, device=dev).bfloat16()
    gate, up, down = (nn.Linear(a, b, bias=False).to(dev).bfloat16() for a, b in ((h, f), (h, f), (f, h)))

    def timed(fn):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / reps * 1e3

    res = {"tokens": m, "hidden": h, "intermediate": f, "gflop": 6.0 * m * h * f / 1e9}
    with torch.no_grad():
        mlp.fuse = True
        y_fused = mlp(x)
        res["fused_us"] = timed(lambda: mlp(x))
        mlp.fuse = False
        y_three = mlp(x)
        res["unfused_mxfp8_us"] = timed(lambda: mlp(x))
        mlp.fuse = True
        res["bf16_nn_linear_us"] = timed(lambda: down(F.silu(gate(x)) * up(x)))
    res["fused_vs_unfused_rel_frobenius"] = float((y_fused.float() - y_three.float()).norm() / y_three.float().norm())
    res["speedup_fused_vs_unfused"] = res["unfused_mxfp8_us"] / res["fused_us"]
    res["speedup_fused_vs_bf16"] = res["bf16_nn_linear_us"] / res["fused_us"]
    res["fused_tflops"] = res["gflop"] / res["fused_us"] * 1e3
    return res


# ----------------------------------------------------------------------------------------------
# N > 1: the sharded modules under NCCL, checked against the unsharded layer
# ----------------------------------------------------------------------------------------------
def sharded_leg(dev, rank, world):
    """ColumnParallelDWLinear (QKV 4096 -> 6144, gather_output) and RowParallelDWLinear (down 14336 -> 4096, all-reduce and
    reduce-scatter) forward + backward on `world` GPUs under NCCL against the unsharded DWLinear computed on every rank
    from the same seeded tensors.  Y of the column-parallel layer must be bit-equal (same kernel, same order over K);
    gradients and the row-parallel output are sums of `world` bf16 partials that the collective adds in bf16, so their
    tolerance grows with the number of roundings: |got - ref| <= 1e-2 * sqrt(world / 2) * max(|ref|, mean|ref|) on 99.9 % of
    the elements and 4e-2 * sqrt(world / 2) everywhere (a model of exactly those roundings on normal data puts the 99.9 %
    quantile at 0.008 / 0.011 / 0.015 and the worst of 4 M elements at 0.017 / 0.029 / 0.034 for 2 / 4 / 8 ranks).  Also times the
    column-parallel forward with and without the gather, and the row-parallel forward with its reduction."""
    import torch.distributed as dist
    import deepwell_b200 as dw
    from deepwell_b200.sharded import ColumnParallelDWLinear, RowParallelDWLinear

    m = 8192
    res = {"tokens": m, "world": world}

    def close(got, ref, what):
        got, ref = got.float(), ref.float()
        floor = ref.abs().mean()
        err = (got - ref).abs() / torch.maximum(ref.abs(), floor)
        widen = max(1.0, world / 2.0) ** 0.5
        frac_ok = float((err <= 1e-2 * widen).float().mean())
        worst = float(err.max())
        res[what + "_max_rel_err"] = worst
        return frac_ok >= 0.999 and worst <= 4e-2 * widen and not bool(torch.isnan(got).any())

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / reps * 1e3], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    g = torch.Generator(device=dev).manual_seed(777)          # same seed on every rank: replicated tensors
    ok = True
    # ---- column-parallel: QKV ----
    k, n = 4096, 6144
    x = torch.randn(m, k, device=dev, generator=g).bfloat16()
    w = (torch.randn(n, k, device=dev, generator=g) * 0.02).bfloat16()
    b = torch.randn(n, device=dev, generator=g).bfloat16()
    gy = torch.randn(m, n, device=dev, generator=g).bfloat16()
    full = dw.DWLinear(k, n, bias=True, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        full.weight.copy_(w)
        full.bias.copy_(b)
    xr = x.clone().requires_grad_(True)
    y_ref = full(xr)
    y_ref.backward(gy)
    col = ColumnParallelDWLinear(k, n, bias=True, gather_output=True, device=dev, dtype=torch.bfloat16)
    col.load_full_weight(w, b)
    xs = x.clone().requires_grad_(True)
    y = col(xs)
    y.backward(gy)
    torch.cuda.synchronize(dev)
    bit_equal = bool(torch.equal(y.view(torch.int16), y_ref.view(torch.int16)))
    res["column_parallel_y_bit_equal"] = bit_equal
    ok &= bit_equal
    ok &= close(xs.grad, xr.grad, "column_parallel_dx")
    dw_equal = bool(torch.equal(col.local.weight.grad.view(torch.int16), full.weight.grad[col.n0:col.n1].view(torch.int16)))
    res["column_parallel_dw_bit_equal"] = dw_equal
    ok &= dw_equal
    ok &= close(col.local.bias.grad, full.bias.grad[col.n0:col.n1], "column_parallel_db")
    nogather = ColumnParallelDWLinear(k, n, bias=True, gather_output=False, device=dev, dtype=torch.bfloat16)
    nogather.load_full_weight(w, b)
    blocked = ColumnParallelDWLinear(k, n, bias=True, gather_output=True, blocked_output=True, device=dev, dtype=torch.bfloat16)
    blocked.load_full_weight(w, b)
    with torch.no_grad():
        res["qkv_fwd_us_unsharded"] = timed(lambda: full(x))
        res["qkv_fwd_us_no_gather"] = timed(lambda: nogather(x))
        res["qkv_fwd_us_with_gather"] = timed(lambda: col(x))
        res["qkv_fwd_us_with_gather_blocked_layout"] = timed(lambda: blocked(x))
    res["gather_bytes_per_rank"] = m * (n // world) * 2 * (world - 1)
    del full, col, nogather, blocked, x, w, b, gy, xr, xs, y, y_ref
    # ---- row-parallel: down projection, fed by this rank's slice of the features ----
    k, n = 14336, 4096
    x = torch.randn(m, k, device=dev, generator=g).bfloat16()
    w = (torch.randn(n, k, device=dev, generator=g) * 0.02).bfloat16()
    gy = torch.randn(m, n, device=dev, generator=g).bfloat16()
    full = dw.DWLinear(k, n, bias=False, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        full.weight.copy_(w)
    xr = x.clone().requires_grad_(True)
    y_ref = full(xr)
    y_ref.backward(gy)
    row = RowParallelDWLinear(k, n, bias=False, input_is_parallel=True, device=dev, dtype=torch.bfloat16)
    row.load_full_weight(w)
    xl = x[:, row.k0:row.k1].clone().requires_grad_(True)
    y = row(xl)
    y.backward(gy)
    torch.cuda.synchronize(dev)
    ok &= close(y, y_ref, "row_parallel_y")
    ok &= close(xl.grad, xr.grad[:, row.k0:row.k1], "row_parallel_dx")
    ok &= close(row.local.weight.grad, full.weight.grad[:, row.k0:row.k1], "row_parallel_dw")
    rs = RowParallelDWLinear(k, n, bias=False, input_is_parallel=True, scatter_output=True, device=dev, dtype=torch.bfloat16)
    rs.load_full_weight(w)
    with torch.no_grad():
        y_rs = rs(xl.detach())
        ok &= close(y_rs, y_ref[rank * (m // world):(rank + 1) * (m // world)], "row_parallel_reduce_scatter_y")
        xd = xl.detach()
        res["down_fwd_us_unsharded"] = timed(lambda: full(x))
        res["down_fwd_us_all_reduce"] = timed(lambda: row(xd))
        res["down_fwd_us_reduce_scatter"] = timed(lambda: rs(xd))
    flag = torch.tensor([1 if ok else 0], device=dev, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    res["parity"] = "ok" if int(flag.item()) == 1 else "MISMATCH"
    return res


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="deepwell_b200", choices=["deepwell_b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--sustained-seconds", type=float, default=2.5,
                    help="length of the sustained leg (the same step repeated; 0 switches it off)")
    ap.add_argument("--variant", type=int, default=0, help="GEMM kernel variant (0 = automatic)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra-legs", action="store_true",
                    help="skip the secondary legs (vendor comparison, GPT-2 MLP, decoder step, sharded parity, gather)")
    ap.add_argument("--sweep-quantize", action="store_true",
                    help="quantise-only bandwidth sweep (K in {128,1024,4096,16384}, 2^20..2^32 elements, both directions)")
    ap.add_argument("--sweep-log2-min", type=int, default=20)
    ap.add_argument("--sweep-log2-max", type=int, default=32)
    ap.add_argument("--compare-vendor", action="store_true",
                    help="alternate the vendor block-scaled GEMM (torch._scaled_mm) with dw_mxfp8_gemm on the workload's shapes")
    ap.add_argument("--probe-corun", action="store_true",
                    help="measure what runs beside the GEMM (a second stream's kernel, copy, quantiser) and exit")
    ap.add_argument("--traffic-from-csv", default=None, help="ncu CSV of the GEMM launches -> bench_gemm_dram_traffic.json")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="tuning aid: on one GPU, run the shard sizes rank 0 would get in a job of this many GPUs")
    ap.add_argument("--serial", action="store_true", help="quantise and GEMM on one stream, every launch after the previous one has finished")
    ap.add_argument("--two-streams", action="store_true", help="the next layer's quantisers on a second, lower-priority stream")
    ap.add_argument("--exchange-push", choices=["graph", "stream"], default="graph",
                    help="N > 1: the peer copies of the shared quantisation as one replayed CUDA graph per step (default) or issued one by one")
    ap.add_argument("--exchange-budget", default="0,0.2,0.4,0.6,0.8,1.1,all",
                    help="N > 1: share as many rows of X as a rank can receive (at 700 GB/s) in this multiple of the step's GEMM "
                         "time ('all' = every row, 0 = none: every rank quantises all of X itself, in one launch); several "
                         "values, comma-separated: each is tried for a few steps before the timed region and the fastest kept")
    ap.add_argument("--quant-batch-pairs", action="store_true",
                    help="the activation and the weight shard of a layer quantised by one launch (dw_mxfp8_quantize_rows_batch)")
    ap.add_argument("--exchange-own-work", choices=["auto", "start", "spread"], default="auto",
                    help="N > 1 with shared quantisation: the rank's own quantisations in one launch at the start of the step, or spread "
                         "behind the GEMMs; auto = measured before the timed region")
    ap.add_argument("--no-quant-batch", action="store_true",
                    help="N > 1: one quantiser launch per slice and weight shard instead of dw_mxfp8_quantize_rows_batch")
    ap.add_argument("--no-exchange", action="store_true",
                    help="N > 1: every rank quantises the whole of every X itself (no sharing of the quantisation over NVLink)")
    ap.add_argument("--profile-case", default=None, choices=["gemm", "quant_row", "quant_both", "quant_col", "quant_col_long", "quant_batch"],
                    help="run a few launches of one kernel on a small case (for an ncu capture) and exit")
    ap.add_argument("--workload", default="linears", choices=["linears", "decoder_step"],
                    help="linears: the headline Llama-3-8B linear shapes; decoder_step: end-to-end optimize() training step (1 GPU)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.traffic_from_csv:
        traffic_from_csv(args.traffic_from_csv)
        return
    if args.profile_case:
        run_profile_case(args)
        return
    if args.sweep_quantize:
        run_quantize_sweep(args)
        return
    if args.compare_vendor:
        if rank == 0:
            run_compare_vendor(args)
        return
    if args.probe_corun:
        if rank == 0:
            run_probe_corun(args)
        return
    if args.workload == "decoder_step":
        if rank == 0:
            run_decoder_step(args)
        return

    import torch.distributed as dist
    from deepwell_b200 import _native as nv
    from deepwell_b200 import cutlass_kernels as ck
    from deepwell_b200.sharded import shard_bounds

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    L = nv.load()
    if L.dw_mxfp8_device_supported(local_rank) != 1:
        raise SystemExit("device is not sm_100 (B200)")
    nv.set_gemm_variant(args.variant)
    warmup = max(3, args.warmup)

    # ---- synthetic inputs, resident in HBM ----
    g = torch.Generator(device=dev).manual_seed(3456)
    layers = []
    for name, k, n in LAYERS:
        n0, n1 = shard_bounds(n, max(world, args.emulate_world), rank)
        x = torch.randn(M_TOKENS, k, device=dev, generator=g).bfloat16()
        w_full = (torch.randn(n, k, device=dev, generator=g) * 0.02).bfloat16()
        w = w_full[n0:n1].contiguous()
        del w_full
        nl = n1 - n0
        u8 = lambda *s: torch.empty(*s, dtype=torch.uint8, device=dev)
        layers.append({"name": name, "k": k, "n": nl, "x": x, "w": w, "xc": u8(M_TOKENS, k),
                       "xs": u8(nv.scale_bytes(M_TOKENS, k, nv.SF_TILED)), "wc": u8(nl, k),
                       "ws": u8(nv.scale_bytes(nl, k, nv.SF_TILED)),
                       "y": torch.empty(M_TOKENS, nl, dtype=torch.bfloat16, device=dev)})
    status = nv.status_word(dev)
    # Everything runs on `stream`.  The four layers are independent problems, so the (HBM-bound) quantisers of layer i+1
    # can run while the (tensor-bound) GEMM of layer i does.  No kernel is scheduled beside a GEMM thread block on its own
    # SM (measured), so the overlap that exists is on the SMs the GEMM leaves free: those it does not need for its number
    # of rounds of tiles, and those whose last tile is done.  Default: one stream, GEMM(i) issued BEFORE the quantisers of
    # layer i+1, which are launched with DW_QUANT_OVERLAP_PREVIOUS (they start once the GEMM's blocks are resident).
    # --two-streams: the quantisers on a second, lower-priority stream with events.  --serial: one stream, no overlap.
    overlap = not (args.serial or args.two_streams)
    lo_pri, hi_pri = torch.cuda.Stream.priority_range()
    stream = torch.cuda.Stream(dev, priority=hi_pri)
    torch.cuda.set_stream(stream)
    st = stream.cuda_stream
    qstream = torch.cuda.Stream(dev, priority=lo_pri) if args.two_streams else stream
    sq = qstream.cuda_stream
    for l in layers:
        l["quantised"] = torch.cuda.Event()            # operands of this layer are ready
        l["consumed"] = torch.cuda.Event()             # the GEMM that read them has finished
    gemm_events, pair_events = [], []

    import ctypes
    for l in layers:                                   # argument arrays of the one-launch form (X and W of a layer together)
        P2, I2 = ctypes.c_void_p * 2, ctypes.c_int64 * 2
        l["batch_args"] = (P2(l["x"].data_ptr(), l["w"].data_ptr()), P2(l["xc"].data_ptr(), l["wc"].data_ptr()),
                           P2(l["xs"].data_ptr(), l["ws"].data_ptr()), I2(M_TOKENS, l["n"]), I2(l["k"], l["k"]))
    pair_batch = args.quant_batch_pairs and all(l["n"] % 128 == 0 and l["k"] % 128 == 0 for l in layers) and M_TOKENS % 128 == 0

    def quantise_operands(l, flags):
        if pair_batch:
            xa, ca, sa, ra, ka = l["batch_args"]
            nv.check(L.dw_mxfp8_quantize_rows_batch(2, xa, ca, sa, ra, ka, nv.RULE_OCP_FLOOR, nv.SF_TILED, flags, st), "quantize X, W")
            return
        nv.check(L.dw_mxfp8_quantize_ex(l["x"].data_ptr(), l["xc"].data_ptr(), l["xs"].data_ptr(), M_TOKENS, l["k"],
                                        nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, flags, st), "quantize X")
        nv.check(L.dw_mxfp8_quantize_ex(l["w"].data_ptr(), l["wc"].data_ptr(), l["ws"].data_ptr(), l["n"], l["k"],
                                        nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, flags, st), "quantize W")

    def overlapped_step(record: bool, after_gemm=None):
        """GEMM of layer i, then (behind it on the same stream, allowed to start while it runs) the quantisers of layer
        i + 1; the last layer's GEMM is followed by the first layer's quantisers for the next step.  Per step: 4 GEMMs,
        4 activation and 4 weight quantisations, 12 launches."""
        for i, l in enumerate(layers):
            nxt = layers[(i + 1) % len(layers)]
            if after_gemm is not None and "gather_done" in l:
                stream.wait_event(l["gather_done"])    # the previous step's all-gather has read this layer's Y
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            nv.check(L.dw_mxfp8_gemm(l["xc"].data_ptr(), l["xs"].data_ptr(), l["wc"].data_ptr(), l["ws"].data_ptr(),
                                     l["y"].data_ptr(), None, M_TOKENS, l["n"], l["k"], 1.0, 0.0, None, 0,
                                     status.data_ptr(), st), "gemm")
            quantise_operands(nxt, nv.QUANT_OVERLAP_PREVIOUS)
            if record:
                e1.record(stream)                      # GEMM + the quantisers that overlapped it
                pair_events.append((e0, e1))
            if after_gemm is not None:
                after_gemm(l)
        return (2 if pair_batch else 3) * len(layers)

    # ---- N > 1: the ranks share the quantisation of the replicated activations (deepwell_b200/exchange.py) ----
    # How much is shared is a budget: the rows a rank can receive per step (at ~700 GB/s) within a multiple of the step's
    # GEMM time, largest activation first, the last one partly; the remaining rows every rank quantises itself.  With the
    # copies longer than the step the fence would wait for them, with too few rows shared the ranks repeat HBM-bound work:
    # the multiple is measured (a few steps per candidate before the timed region) unless --exchange-budget fixes it.
    exchange, ex_index, exchange_info, ex_plans = None, {}, None, []
    if world > 1 and overlap and not args.no_exchange and not args.emulate_world and M_TOKENS % (128 * world) == 0:
        order = sorted(range(len(layers)), key=lambda j: -layers[j]["k"])
        ex_index = {i: n for n, i in enumerate(order)}
        gemm_s = total_flops() / world / 2.6e15

        def plan_for(factor):
            left, rows = factor * gemm_s, []
            for i in order:
                per_row = layers[i]["k"] * (1 + 1 / 32) * (world - 1) / world / 700e9
                r = min(M_TOKENS, int(left / per_row)) // (128 * world) * (128 * world)
                rows.append(r)
                left -= r * per_row
            return rows

        factors = [1e9 if f.strip() == "all" else float(f) for f in str(args.exchange_budget).split(",") if f.strip()]
        for f in factors:
            plan = plan_for(f)
            if plan not in [q for _, q in ex_plans]:
                ex_plans.append((f, plan))
        try:
            from deepwell_b200.exchange import QuantizedRowExchange
            exchange = QuantizedRowExchange([(M_TOKENS, layers[i]["k"]) for i in order], device=dev, push=args.exchange_push)
            exchange.set_shared_rows(ex_plans[0][1])
            exchange_info = {"layers": [layers[i]["name"] for i in order], "how": exchange.how, "push": exchange.push_mode}
        except Exception as e:          # no peer mapping on this box: every rank quantises everything itself
            exchange, ex_index = None, {}
            exchange_info = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
    step_no = [0]

    def exchange_step(record: bool, after_gemm=None):
        """The step with shared quantisation: this rank's row slices of the exchanged activations for the NEXT step are
        quantised first and travel to the peers while this step's GEMMs run; the other activations and the weight shards
        are quantised here; a 4-byte all-reduce at the end makes the next step's operands complete on every rank."""
        now, nxt = step_no[0] % 2, (step_no[0] + 1) % 2
        order = sorted(ex_index, key=lambda j: ex_index[j])
        # the rank's row slices and its weight shards are small: all of them leave in one or two launches
        batch_w = not args.no_quant_batch
        n_launch = exchange.quantise_and_push([layers[i]["x"] for i in order], nxt,
                                              extra=[(l["w"], l["wc"].view(torch.uint8), l["ws"]) for l in layers] if batch_w else ())
        for i, l in enumerate(layers):
            if i in ex_index:
                a_codes, a_sf = exchange.operand(now, ex_index[i])
                a_ptr, s_ptr = a_codes.data_ptr(), a_sf.data_ptr()
            else:
                nv.check(L.dw_mxfp8_quantize(l["x"].data_ptr(), l["xc"].data_ptr(), l["xs"].data_ptr(), M_TOKENS, l["k"],
                                             nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, st), "quantize X")
                a_ptr, s_ptr = l["xc"].data_ptr(), l["xs"].data_ptr()
                n_launch += 1
            if not batch_w:
                nv.check(L.dw_mxfp8_quantize(l["w"].data_ptr(), l["wc"].data_ptr(), l["ws"].data_ptr(), l["n"], l["k"],
                                             nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, st), "quantize W")
                n_launch += 1
            if after_gemm is not None and "gather_done" in l:
                stream.wait_event(l["gather_done"])
            nv.check(L.dw_mxfp8_gemm(a_ptr, s_ptr, l["wc"].data_ptr(), l["ws"].data_ptr(), l["y"].data_ptr(), None,
                                     M_TOKENS, l["n"], l["k"], 1.0, 0.0, None, 0, status.data_ptr(), st), "gemm")
            n_launch += 1
            if after_gemm is not None:
                after_gemm(l)
        exchange.fence(nxt)
        step_no[0] += 1
        return n_launch

    exchange_spread = [args.exchange_own_work == "spread"]   # True: exchange_step_spread instead of exchange_step

    def exchange_step_spread(record: bool, after_gemm=None):
        """The same exchange with the rank's own work spread over the step: only its slices of the shared rows are quantised
        at the start (they have to travel); the rows every rank quantises itself and the weight shards follow the GEMMs one by
        one with DW_QUANT_OVERLAP_PREVIOUS, as in the step without exchange.  Layer i's GEMM is followed by the local rows of
        activation i for the NEXT step (the other slot) and by the weight shard of layer i + 1."""
        now, nxt = step_no[0] % 2, (step_no[0] + 1) % 2
        order = sorted(ex_index, key=lambda j: ex_index[j])
        shared, local = exchange.pieces([layers[i]["x"] for i in order], nxt)
        n_launch = exchange.quantise(shared)
        exchange.push(nxt)
        for i, l in enumerate(layers):
            a_codes, a_sf = exchange.operand(now, ex_index[i])
            if after_gemm is not None and "gather_done" in l:
                stream.wait_event(l["gather_done"])
            nv.check(L.dw_mxfp8_gemm(a_codes.data_ptr(), a_sf.data_ptr(), l["wc"].data_ptr(), l["ws"].data_ptr(), l["y"].data_ptr(),
                                     None, M_TOKENS, l["n"], l["k"], 1.0, 0.0, None, 0, status.data_ptr(), st), "gemm")
            n_launch += 1
            for x_rows, codes, scales in local[ex_index[i]]:
                nv.check(L.dw_mxfp8_quantize_ex(x_rows.data_ptr(), codes.data_ptr(), scales.data_ptr(), x_rows.shape[0], x_rows.shape[1],
                                                nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, nv.QUANT_OVERLAP_PREVIOUS, st), "quantize X")
                n_launch += 1
            w = layers[(i + 1) % len(layers)]
            nv.check(L.dw_mxfp8_quantize_ex(w["w"].data_ptr(), w["wc"].data_ptr(), w["ws"].data_ptr(), w["n"], w["k"],
                                            nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, nv.QUANT_OVERLAP_PREVIOUS, st), "quantize W")
            n_launch += 1
            if after_gemm is not None:
                after_gemm(l)
        exchange.fence(nxt)
        step_no[0] += 1
        return n_launch

    exchange_on = [True]       # the legs that gather every output keep NVLink for Y: there every rank quantises all of X itself
    exchange_used = [True]     # False: the candidates were measured and the plain step (nothing shared, separate launches) won

    def step(record: bool, after_gemm=None, force_separate=False):
        if exchange is not None and exchange_on[0] and not force_separate:
            return exchange_step_spread(record, after_gemm) if exchange_spread[0] else exchange_step(record, after_gemm)
        if overlap and not force_separate:
            return overlapped_step(record, after_gemm)
        launches = 0
        for l in layers:
            if qstream is not stream:
                qstream.wait_event(l["consumed"])      # do not overwrite operands a GEMM may still read
            nv.check(L.dw_mxfp8_quantize(l["x"].data_ptr(), l["xc"].data_ptr(), l["xs"].data_ptr(), M_TOKENS, l["k"],
                                         nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, sq), "quantize X")
            nv.check(L.dw_mxfp8_quantize(l["w"].data_ptr(), l["wc"].data_ptr(), l["ws"].data_ptr(), l["n"], l["k"],
                                         nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, sq), "quantize W")
            if qstream is not stream:
                l["quantised"].record(qstream)
                stream.wait_event(l["quantised"])
            if after_gemm is not None and "gather_done" in l:
                stream.wait_event(l["gather_done"])    # the previous step's all-gather has read this layer's Y
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            nv.check(L.dw_mxfp8_gemm(l["xc"].data_ptr(), l["xs"].data_ptr(), l["wc"].data_ptr(), l["ws"].data_ptr(),
                                     l["y"].data_ptr(), None, M_TOKENS, l["n"], l["k"], 1.0, 0.0, None, 0,
                                     status.data_ptr(), st), "gemm")
            if record:
                e1.record(stream)
                gemm_events.append((e0, e1))
            if qstream is not stream:
                l["consumed"].record(stream)
            if after_gemm is not None:
                after_gemm(l)
            launches += 3
        return launches

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(v):
        if world > 1:
            t = torch.tensor([v], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return v

    def timed_steps(n_steps, record, after_gemm=None, finish=None):
        """n_steps steps bracketed by barrier + synchronize, CUDA events on the GEMM stream, max over ranks (ms)."""
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        qstream.wait_event(t0)                        # nothing of the timed steps starts before the timer
        n_launch = 0
        for _ in range(n_steps):
            n_launch += step(record, after_gemm)
        if finish is not None:
            finish()
        t1.record(stream)                             # the last GEMM depends on every quantisation before it
        barrier()
        return max_over_ranks(t0.elapsed_time(t1)), n_launch

    if overlap:
        quantise_operands(layers[0], 0)               # the pipeline's first operands; later ones follow a GEMM
    def prime_exchange():                             # the first step's operands: slot 0
        step_no[0] = 0
        exchange.quantise_and_push([layers[i]["x"] for i in sorted(ex_index, key=lambda j: ex_index[j])], 0)
        exchange.fence(0)
        quantise_operands(layers[0], 0)               # W of the first layer, which the spread form expects to be there

    if exchange is not None:
        if len(ex_plans) > 1:                         # measure the candidates, keep the fastest (the same on every rank)
            tried = []
            for f, plan in ex_plans:
                exchange.set_shared_rows(plan)
                prime_exchange()
                for _ in range(2):
                    step(False)
                t_ms, _ = timed_steps(6, False)
                tried.append((t_ms / 6, f, plan))
            best = min(tried, key=lambda t: t[0])
            exchange.set_shared_rows(best[2])
            exchange_info["tried_ms_per_step"] = {("all" if f > 1e6 else f"{f:g} x GEMM time"): round(t, 4) for t, f, _ in tried}
            # the best plan again with the rank's own quantisations spread over the step instead of one launch at its start
            if args.exchange_own_work == "auto":
                prime_exchange()
                exchange_spread[0] = True
                for _ in range(2):
                    step(False)
                t_ms, _ = timed_steps(6, False)
                exchange_info["tried_ms_per_step"]["best plan, own work behind the GEMMs"] = round(t_ms / 6, 4)
                if t_ms / 6 < best[0]:
                    best = (t_ms / 6, best[1], best[2])
                else:
                    exchange_spread[0] = False
            # and the step without the exchange object: every rank quantises all of X itself, one launch per operand,
            # each behind the previous layer's GEMM
            exchange_on[0] = False
            quantise_operands(layers[0], 0)
            for _ in range(2):
                step(False)
            t_ms, _ = timed_steps(6, False)
            exchange_info["tried_ms_per_step"]["no exchange, separate launches"] = round(t_ms / 6, 4)
            exchange_used[0] = best[0] <= t_ms / 6
            exchange_on[0] = exchange_used[0]
        exchange_info["used"] = exchange_used[0]
        exchange_info["own_work"] = "behind the GEMMs" if exchange_spread[0] else "one launch at the start of the step"
        if exchange_used[0]:
            exchange_info["shared_rows"] = list(exchange.shared_rows)
            exchange_info["bytes_pushed_per_rank_per_step"] = int(exchange.bytes_pushed_per_call)
            prime_exchange()
        else:
            exchange_info["shared_rows"] = [0] * len(layers)
            exchange_info["bytes_pushed_per_rank_per_step"] = 0
            quantise_operands(layers[0], 0)
    for _ in range(warmup):
        step(False)
    nv.check_status(dev)

    sampler = ClockSampler(local_rank)
    sampler.start()
    elapsed_ms, launches = timed_steps(args.steps, True)
    clocks = sampler.stop()
    nv.check_status(dev)
    ms_per_step = elapsed_ms / args.steps
    value = total_flops() / (ms_per_step * 1e-3) / 1e12
    if exchange is not None and exchange_used[0]:
        # the operands the exchange assembled (this rank's slice + the peers') against this rank's own quantisation of the whole X
        same = True
        for i, j in ex_index.items():
            l = layers[i]
            nv.check(L.dw_mxfp8_quantize(l["x"].data_ptr(), l["xc"].data_ptr(), l["xs"].data_ptr(), M_TOKENS, l["k"],
                                         nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, st), "quantize X")
            codes, scales = exchange.operand(step_no[0] % 2, j)
            same = same and bool(torch.equal(codes, l["xc"])) and bool(torch.equal(scales, l["xs"]))
        flag = torch.tensor([1 if same else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        exchange_info["parity"] = "ok" if int(flag.item()) == 1 else "MISMATCH"

    # ---- roofline of the dominant kernel (GEMM), live CUDA-event durations of this rank ----
    if overlap:
        # Inside the timed region a GEMM's end cannot be told apart from the quantisers that overlap it (an event between
        # them would hold the quantisers back).  The GEMM's own launch durations come from a second pass of the same
        # steps, straight after the timed region, in which every launch waits for the previous one.
        for _ in range(args.steps):
            step(True, force_separate=True)
        torch.cuda.synchronize(dev)
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_events)
    gemm_flops_step = sum(2.0 * M_TOKENS * l["n"] * l["k"] for l in layers)
    achieved = args.steps * gemm_flops_step / (gemm_ms * 1e-3) / 1e12
    peaks = measured_peaks()
    peak_burst, peak_sustained = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
    # The denominator that fits the run: a timed region shorter than a second with the SM clock at its maximum is a
    # burst measurement (the power cap has not bitten yet), anything else is held to the sustained figure.
    at_max_clock = clocks["sm_mhz"] is None or clocks["sm_max_mhz"] is None or clocks["sm_mhz"] >= 0.95 * clocks["sm_max_mhz"]
    burst_run = elapsed_ms < 1000.0 and at_max_clock
    peak = peak_burst if burst_run else peak_sustained
    traffic, traffic_info = gemm_dram_traffic()
    roofline = {"bound": "tensor", "kernel": "mx_gemm_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "frac_of_burst": achieved / peak_burst, "frac_of_sustained": achieved / peak_sustained,
                "peak_burst": peak_burst, "peak_sustained": peak_sustained,
                "peak_choice": ("burst" if burst_run else "sustained") + f": timed region {elapsed_ms:.0f} ms, median SM clock "
                               f"{clocks['sm_mhz']} of {clocks['sm_max_mhz']} MHz",
                "peak_basis": f"2 x the bf16 dense rate of {peaks['source']} MEASURED_PEAKS (MXFP8 issues at twice the bf16 "
                              "tensor rate): burst for a sub-second region at full clock, else sustained; nominal dense "
                              "MXFP8 is 4500",
                "frac_of_nominal_4500": achieved / NOMINAL_MXFP8_TFLOPS,
                "traffic": traffic if world == 1 else None,
                "traffic_note": "mean DRAM bytes per GEMM launch (ncu, N = 1, bench_gemm_dram_traffic.json); algorithmic mean "
                                "A + B + D = 5.16e8",
                "gemm_ms_per_step": gemm_ms / args.steps, "launches_timed": len(gemm_events),
                **({"gemm_plus_overlapped_quantisers_ms_per_step": sum(a.elapsed_time(b) for a, b in pair_events) / args.steps,
                    "timing": "GEMM launch durations from a pass of the same steps right after the timed region in which "
                              "every launch waits for the previous one; in the timed region itself each GEMM overlaps the "
                              "next layer's quantisers"} if overlap else {})}

    def gemm_only(reps):
        ev = []
        for _ in range(reps):
            for l in layers:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                nv.check(L.dw_mxfp8_gemm(l["xc"].data_ptr(), l["xs"].data_ptr(), l["wc"].data_ptr(), l["ws"].data_ptr(),
                                         l["y"].data_ptr(), None, M_TOKENS, l["n"], l["k"], 1.0, 0.0, None, 0,
                                         status.data_ptr(), st), "gemm")
                e1.record(stream)
                ev.append((e0, e1))
        torch.cuda.synchronize(dev)
        return sum(a.elapsed_time(b) for a, b in ev) / reps

    # the same GEMM launches with nothing else on the GPU (in the timed region the next layer's
    # quantisation runs underneath them and takes its share of power and issue slots)
    if not args.serial:
        torch.cuda.synchronize(dev)
        if overlap:
            for l in layers:
                quantise_operands(l, 0)
        alone_ms = gemm_only(3)
        alone_tf = gemm_flops_step / (alone_ms * 1e-3) / 1e12
        roofline["achieved_alone"] = alone_tf
        roofline["frac_alone_of_burst"] = alone_tf / peak_burst
        roofline["note"] = "achieved_alone: the four GEMM launches back to back with nothing else running, after everything else"

    # ---- sustained leg: the same step for >= args.sustained_seconds, clocks sampled throughout ----
    sustained = None
    if args.sustained_seconds > 0:
        n_sus = max(args.steps, int(math.ceil(args.sustained_seconds * 1e3 / ms_per_step)))
        sus_sampler = ClockSampler(local_rank)
        sus_sampler.start()
        sus_ms, _ = timed_steps(n_sus, False)
        sus_clocks = sus_sampler.stop()
        sus_step = sus_ms / n_sus
        sus_value = total_flops() / (sus_step * 1e-3) / 1e12
        sustained = {"value": sus_value, "unit": "TFLOP/s", "ms_per_step": sus_step, "steps": n_sus, "seconds": sus_ms / 1e3,
                     "sm_mhz_median": sus_clocks["sm_mhz"], "sm_max_mhz": sus_clocks["sm_max_mhz"],
                     "reasons": sus_clocks["reasons"], "clock_samples": sus_clocks["samples"],
                     "frac_of_sustained_peak": sus_value / world / peak_sustained,
                     "frac_of_burst_peak": sus_value / world / peak_burst,
                     "note": "whole step (quantisers + GEMMs), per GPU, over 2 x measured sustained / burst bf16 rate"}
        nv.check_status(dev)

    # ---- quantiser bandwidth (second kernel of the path), timed alone on the largest activation ----
    big = max(layers, key=lambda l: l["k"])
    qe0, qe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    qe0.record(stream)
    for _ in range(reps):
        L.dw_mxfp8_quantize(big["x"].data_ptr(), big["xc"].data_ptr(), big["xs"].data_ptr(), M_TOKENS, big["k"],
                            nv.DIR_ROW, nv.RULE_OCP_FLOOR, nv.SF_TILED, st)
    qe1.record(stream)
    torch.cuda.synchronize(dev)
    q_ms = qe0.elapsed_time(qe1) / reps
    q_gbs = M_TOKENS * big["k"] * 3.03125 / (q_ms * 1e-3) / 1e9
    roofline_q = {"bound": "hbm", "kernel": "mx_quant_row_bg_kernel", "achieved": q_gbs, "peak": peaks["hbm_gbs"],
                  "unit": "GB/s", "frac": q_gbs / peaks["hbm_gbs"], "frac_of_nominal_8000": q_gbs / 8000.0,
                  "shape": [M_TOKENS, big["k"]], "bytes_per_element": 3.03125}

    # ---- N > 1: the same step with every layer's output all-gathered along N over NVLink (NCCL, its own stream) ----
    with_gather = None
    if world > 1 and not args.no_extra_legs:
        try:
            cstream = torch.cuda.Stream(dev)
            for l in layers:
                l["gathered"] = torch.empty(world, M_TOKENS, l["n"], dtype=torch.bfloat16, device=dev)   # rank-major blocks
                l["gemm_done"] = torch.cuda.Event()

            def gather_after(l):
                l["gemm_done"].record(stream)
                cstream.wait_event(l["gemm_done"])
                with torch.cuda.stream(cstream):
                    dist.all_gather_into_tensor(l["gathered"].view(world * M_TOKENS, l["n"]), l["y"])
                    l["gather_done"] = torch.cuda.Event()
                    l["gather_done"].record(cstream)

            even = all(n % (32 * world) == 0 for _, _, n in LAYERS)
            exchange_on[0] = False
            if overlap:
                quantise_operands(layers[0], 0)       # the pipeline's first operands (the exchange step does not leave them)
            if even:
                for _ in range(2):
                    step(False, gather_after)
                stream.wait_stream(cstream)
                g_ms, _ = timed_steps(args.steps, False, gather_after, finish=lambda: stream.wait_stream(cstream))
                g_step = g_ms / args.steps
                with_gather = {"value": total_flops() / (g_step * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": g_step,
                               "gather_bytes_per_rank_per_step": int(sum(M_TOKENS * l["n"] * 2 * (world - 1) for l in layers)),
                               "note": "each GEMM's output shard all-gathered (NCCL all_gather_into_tensor on its own stream, "
                                       "overlapping the next layer's GEMM); every rank quantises all of X itself in this leg "
                                       "(NVLink carries Y only); without the gather: `value`"}
            nv.check_status(dev)
        except Exception as e:
            with_gather = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
        # ---- the same gather by the copy engines (deepwell_b200.exchange.ColumnGather): every rank copies its shard into its
        #      block of the rank-major [world, M, n_local] result on every rank (plain copies, which run while the next GEMM
        #      holds the SMs), or into columns [n0, n1) of the row-major [M, N] result (pitched copies)
        if with_gather is not None and "error" not in with_gather:
            from deepwell_b200.exchange import ColumnGather
            own_y = [l["y"] for l in layers]
            for key, layout in (("copy_engines", "blocked"), ("copy_engines_row_major", "row_major")):
                try:
                    # two slots: a layer's GEMM of step s + 1 fills one while the copies of step s still read the other
                    cg = ColumnGather([(M_TOKENS, l["n"] * world) for l in layers], device=dev, layout=layout, slots=2)
                    cg_done = {}
                    for i, l in enumerate(layers):
                        l["cg_index"], l["cg_slot"] = i, 0
                        l["y"] = cg.shard(i, 0)            # the GEMMs write straight into the buffers the copies read
                        l.pop("gather_done", None)

                    def push_after(l):
                        i, slot = l["cg_index"], l["cg_slot"]
                        cg_done[(i, slot)] = cg.push(i, slot)
                        l["cg_slot"] = slot ^ 1
                        l["y"] = cg.shard(i, slot ^ 1)      # the next step's GEMM of this layer writes the other slot ...
                        if (i, slot ^ 1) in cg_done:
                            l["gather_done"] = cg_done[(i, slot ^ 1)]       # ... once that slot's copies have been made

                    for _ in range(2):
                        step(False, push_after)
                    cg.fence()
                    c_ms, _ = timed_steps(args.steps, False, push_after, finish=cg.fence)
                    c_step = c_ms / args.steps
                    # parity: what arrived against the NCCL all-gather of the same shards
                    same = True
                    for i, l in enumerate(layers):
                        dist.all_gather_into_tensor(l["gathered"].view(world * M_TOKENS, l["n"]), cg.shard(i, l["cg_slot"] ^ 1))
                        full = cg.full(i, l["cg_slot"] ^ 1)     # the slot the last step filled
                        for r in range(world):
                            got = full[r] if layout == "blocked" else full[:, r * l["n"]:(r + 1) * l["n"]]
                            same = same and bool(torch.equal(got, l["gathered"][r]))
                    flag = torch.tensor([1 if same else 0], device=dev, dtype=torch.int32)
                    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                    with_gather[key] = {
                        "value": total_flops() / (c_step * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": c_step,
                        "layout": "[world, M, n_local]" if layout == "blocked" else "[M, N]", "how": cg.how,
                        "parity_vs_nccl_all_gather": "ok" if int(flag.item()) == 1 else "MISMATCH"}
                    del cg
                except Exception as e:
                    with_gather[key] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}
                for l, y in zip(layers, own_y):
                    l["y"] = y
                    l.pop("gather_done", None)
            with_gather["copy_engines_note"] = (
                "each rank copies its shard into every rank's result with device-to-device copies on the copy engines over NVLink "
                "(plain copies for the rank-major layout, replayed as one CUDA graph per layer; pitched copies for the row-major "
                "one) behind each GEMM; one 4-byte all-reduce at the end of the timed region as fence")
        for l in layers:
            l.pop("gathered", None)
            l.pop("gather_done", None)
        exchange_on[0] = exchange_used[0]
        if exchange is not None and exchange_used[0]:
            prime_exchange()
        elif overlap:
            quantise_operands(layers[0], 0)

    # ---- end to end through the public API with host buffers ----
    e2e = None
    if args.e2e_steps > 0:
        host_x = [torch.empty(M_TOKENS, l["k"], dtype=torch.bfloat16).pin_memory() for l in layers]
        host_y = [torch.empty(M_TOKENS, l["n"], dtype=torch.bfloat16).pin_memory() for l in layers]
        for hx, l in zip(host_x, layers):
            hx.copy_(l["x"])
        kernels = []
        for l in layers:
            kern = ck.BlackwellGemmKernel()
            kern.initialize(M_TOKENS, l["n"], l["k"], "mxfp8", True, 32)
            kernels.append(kern)

        # three streams: host->device copies, compute (the public API call), device->host copies.
        # PCIe carries both directions at once, and the copies of other layers hide the compute.
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        dev_x = [torch.empty(M_TOKENS, l["k"], dtype=torch.bfloat16, device=dev) for l in layers]
        # N > 1: X is replicated on every rank (column-parallel layers).  Each rank uploads 1/N of its rows over its
        # own PCIe link and the ranks exchange the slices over NVLink (one all-gather per layer), instead of every
        # rank pulling the whole X out of the same host memory.
        r0, r1 = shard_bounds(M_TOKENS, world, rank)
        even_rows = world > 1 and M_TOKENS % world == 0
        x_slice = [torch.empty(r1 - r0, l["k"], dtype=torch.bfloat16, device=dev) for l in layers] if even_rows else None
        arrived = [torch.cuda.Event() for _ in layers]
        computed = [torch.cuda.Event() for _ in layers]
        freed = [torch.cuda.Event() for _ in layers]

        def e2e_step():
            outs = []
            for i, (hx, hy, l, kern) in enumerate(zip(host_x, host_y, layers, kernels)):
                s_in.wait_event(freed[i])                       # previous step's GEMM has read dev_x[i]
                with torch.cuda.stream(s_in):
                    if even_rows:
                        x_slice[i].copy_(hx[r0:r1], non_blocking=True)
                        dist.all_gather_into_tensor(dev_x[i], x_slice[i])
                    else:
                        dev_x[i].copy_(hx, non_blocking=True)
                    arrived[i].record(s_in)
                stream.wait_event(arrived[i])
                y = kern.gemm(dev_x[i], l["w"].t())             # quantise X, quantise W, GEMM
                computed[i].record(stream)
                freed[i].record(stream)
                s_out.wait_event(computed[i])
                with torch.cuda.stream(s_out):
                    hy.copy_(y, non_blocking=True)
                    y.record_stream(s_out)
                outs.append(y)

        # Steps follow one another without a host synchronisation in between (the device-side events above order every
        # buffer's reuse), so the download of step s overlaps the upload of step s + 1: PCIe carries both directions
        # all the time.  Every step's copies are inside the timed region, which ends when the last download has landed.
        for _ in range(2):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        barrier()
        dt = max_over_ranks((time.perf_counter() - t0) / args.e2e_steps)
        e2e = {"value": total_flops() / dt / 1e12, "unit": "TFLOP/s",
               # whole-job bytes per step: every row of every X crosses PCIe once (N > 1: each rank uploads its
               # slice, NVLink replicates it), every rank downloads its shard of every Y
               "h2d_bytes_per_step": int(sum(hx.numel() * 2 for hx in host_x)) * (1 if even_rows or world == 1 else world),
               "d2h_bytes_per_step": int(sum(hy.numel() * 2 for hy in host_y)) * world, "ms_per_step": dt * 1e3,
               "steps": args.e2e_steps, "warmup": 2,
               "api": "deepwell_b200.cutlass_kernels.BlackwellGemmKernel.gemm, pinned host X in, pinned host Y out, "
                      "copies on their own streams, steps back to back" + ("; X uploaded as 1/N row slices and all-gathered over NVLink"
                                                       if even_rows else "")}
        nv.check_status(dev)
        del host_x, host_y, dev_x, kernels

    # ---- secondary legs ----
    extra = {}
    if not args.no_extra_legs and not args.emulate_world:
        if world > 1:
            try:
                extra["sharded"] = sharded_leg(dev, rank, world)
            except Exception as e:
                extra["sharded"] = {"parity": "not run", "error": f"{type(e).__name__}: {str(e)[:300]}"}
            extra["sharded_parity"] = extra["sharded"].get("parity")
        elif rank == 0:
            for key, fn in (("vendor_gemm", lambda: compare_vendor(dev, {n: (M_TOKENS, nn, k) for n, k, nn in LAYERS})),
                            ("gpt2_mlp", gpt2_mlp_numbers), ("swiglu_mlp", swiglu_mlp_numbers),
                            ("decoder_step", lambda: decoder_step_numbers(steps=5, warmup=3))):
                try:
                    for l in layers:                      # the headline tensors are no longer needed
                        l.pop("y", None)
                    extra[key] = fn()
                    nv.check_status(dev)
                except Exception as e:
                    extra[key] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
                torch.cuda.empty_cache()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        use_all_host_threads()
        cpu_baseline, _ = time_cpu(steps=2, warmup=1)

    if rank == 0:
        bytes_step = sum(l["x"].numel() * 2 + l["w"].numel() * 2 + M_TOKENS * l["n"] * 2 for l in layers)
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "mxfp8(e4m3+e8m0), fp32 accumulate, bf16 out", "data": "synthetic",
                "config": {"workload": WORKLOAD, "M": M_TOKENS, "layers": {n: [k, nn] for n, k, nn in LAYERS},
                           "parallelism": f"N-sharded x{world}, X replicated, no data-path collective" if (exchange is None or not exchange_used[0]) else
                                          f"N-sharded x{world}, X replicated; the quantisation of X is shared (rows {exchange_info['shared_rows']} of "
                                          f"{exchange_info['layers']}): each rank quantises 1/N of those rows and copies its slice into every peer's "
                                          "operand buffer over NVLink (copy engines, under the GEMMs), the other rows every rank quantises itself; "
                                          "one 4-byte all-reduce per step as fence",
                           "step": "per layer: quantise X, quantise W shard, block-scaled GEMM"
                                   + ("; each GEMM is issued before the next layer's quantisers, which may start while it "
                                      "runs (DW_QUANT_OVERLAP_PREVIOUS)" if overlap else
                                      ("; quantisers of the next layer on a second, lower-priority stream" if args.two_streams else "")),
                           "l2": f"inputs larger than L2: {bytes_step / 1e9:.2f} GB touched per step per GPU",
                           "gemm_variant": args.variant,
                           **({"emulated_world": args.emulate_world,
                               "note": "TUNING RUN: one rank's shard on one GPU; value is not a job throughput"}
                              if args.emulate_world else {})},
                "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline, "sustained": sustained,
                "roofline_quantize": roofline_q, "with_gather": with_gather, "exchange": exchange_info, **extra,
                "cpu_baseline": cpu_baseline}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
