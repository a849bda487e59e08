#!/usr/bin/env python
"""Benchmark of the MXFP8 linear hot path: MX quantisation + block-scaled GEMM.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload: the four Llama-3-8B linear shapes at M = 16384 tokens (QKV 4096->6144, O 4096->4096,
fused gate+up 4096->28672, down 14336->4096), bf16 activations N(0,1), weights N(0,0.02),
synthetic and seeded.  One step = for each of the four layers: quantise X row-wise, quantise the
weight (shard) row-wise, run the block-scaled GEMM.  The layers are independent problems, so the
quantisation of layer i+1 runs on a second stream under the GEMM of layer i (--serial: one stream).
With N GPUs every weight is sharded along its output dimension across the ranks (X is replicated;
no collective on the data path), so the total work is fixed: strong scaling.

Prints ONE JSON line (rank 0).  `value` is whole-job TFLOP/s with inputs resident in HBM;
`e2e` is the same through the public API with pinned host buffers, the host->device copy of
every X and the device->host copy of every Y inside the timed region, on their own streams;
`roofline` is measured live with CUDA events around every GEMM launch (`achieved_alone`: the same
launches with nothing else on the GPU); `roofline_quantize` times the row quantiser on the largest
activation; `cpu_baseline` times the CPU restatement of the same path on the host cores (rank 0, N = 1).

--impl reference times only that CPU path (the reference ships no GPU implementation of an
MXFP8 GEMM and its CPU path is a Python module calling torch.matmul).

Other modes (each prints its own JSON): --workload decoder_step (end-to-end optimize() training step of
a 12-layer decoder beside the same model with bf16 nn.Linear), --sweep-quantize (quantise-only bandwidth
sweep), --profile-case (a few launches of one kernel on a small case, for an ncu capture),
--emulate-world W (tuning aid: rank 0's shard sizes of a W-GPU job on one GPU).
"""
from __future__ import annotations

import argparse
import json
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
# dram__bytes_read.sum + dram__bytes_write.sum of the four GEMM launches of one step at N = 1 (ncu capture of
# this file's own launches, summarised in profiles/mx_gemm_kernel_bench_shapes_dram_traffic.md), bytes
GEMM_DRAM_TRAFFIC = {"qkv": 278289152, "o": 178107648, "gate_up": 1457078272, "down": 1161285120}
GEMM_DRAM_TRAFFIC_BYTES = sum(GEMM_DRAM_TRAFFIC.values()) / len(GEMM_DRAM_TRAFFIC)      # mean per launch


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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
def cpu_step(inputs):
    """One pass of the CPU restatement over the sample: quantise X and W (C, OpenMP), dequantise,
    fp32 matmul (torch, all host threads; the reference's CPU GEMM is torch.matmul), bf16 output."""
    from oracle import mx_oracle as o
    from oracle import mx_ref as c
    out = []
    for xb, wb in inputs:
        xc, xs = c.quantize_rowwise(xb, 0)
        wc, ws = c.quantize_rowwise(wb, 0)
        a = torch.from_numpy(c.dequantize(xc, xs))
        b = torch.from_numpy(c.dequantize(wc, ws))
        y = torch.matmul(a, b.t())
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
    return {"value": total_flops(rows) / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"first {rows} of {M_TOKENS} token rows of all four layers (full N and K), "
                      f"{dt:.2f} s per pass: C/OpenMP quantiser + torch.matmul fp32 on dequantised operands"}, dt


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
    else:
        R, C = 16384, 8192
        x = torch.randn(R, C, device=dev, generator=g).bfloat16()
        cr, ct = u8(R, C), u8(C, R)
        sr, sc = u8(nv.scale_bytes(R, C, 1)), u8(nv.scale_bytes(C, R, 1))
        if args.profile_case == "quant_row":
            run = lambda: L.dw_mxfp8_quantize(x.data_ptr(), cr.data_ptr(), sr.data_ptr(), R, C, 0, 0, 1, st)
            bpe = 3.03125
        elif args.profile_case == "quant_col":
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
    for log2n in range(20, 33, 2):
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
                rows_out.append({"log2_elements": log2n, "K": k, "direction": name, "us": ms * 1e3, "GBps": gbs,
                                 "frac_of_measured_copy": gbs / peak, "l2_flushed": small})
                print(json.dumps(rows_out[-1]), flush=True)
        del x_flat, codes
    print(json.dumps({"sweep": "quantize", "peak_hbm_gbs": peak, "points": len(rows_out)}))


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
# ----------------------------------------------------------------------------------------------
# Secondary workload: the end-to-end deepwell.optimize() training step of a pre-LN decoder
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


def run_decoder_step(args):
    """BASELINE config 5: random-init 12-layer pre-LN decoder (hidden 1024, 16 heads, FFN 4096, vocab 32000), batch 8 x
    sequence 2048 uniform token ids; every nn.Linear replaced by deepwell.optimize(precision='mxfp8').  One step = ids
    host->device, forward, cross-entropy, backward, fused AdamW step, loss device->host.  The same model with its
    bf16 nn.Linear layers is timed beside it.  Prints one JSON line; attention (torch SDPA), LayerNorm, GELU, the loss
    and the optimizer are PyTorch's own in both arms: only the linear layers differ."""
    import copy
    import torch.nn.functional as F
    import deepwell_b200 as dw

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU fallback for the product path")
    torch.cuda.set_device(0)
    vocab, hidden, heads, ffn, layers, batch, seq = 32000, 1024, 16, 4096, 12, 8, 2048
    torch.manual_seed(1234)
    base = build_decoder(vocab, hidden, heads, ffn, layers).cuda().bfloat16()
    arms = {"bf16_nn_linear": copy.deepcopy(base), "mxfp8_dwlinear": dw.optimize(copy.deepcopy(base), precision="mxfp8", verbose=False)}
    del base
    n_dw = sum(isinstance(m, dw.DWLinear) for m in arms["mxfp8_dwlinear"].modules())
    lin_params = sum(m.weight.numel() for m in arms["mxfp8_dwlinear"].modules() if isinstance(m, dw.DWLinear))
    ids_host = torch.randint(0, vocab, (args.steps + args.warmup, batch, seq), generator=torch.Generator().manual_seed(7)).pin_memory()
    out, losses = {}, {}
    sampler = ClockSampler(0)
    sampler.start()
    for name, net in arms.items():
        opt = torch.optim.AdamW(net.parameters(), lr=1e-4, fused=True)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = []
        for i in range(args.steps + args.warmup):
            if i == args.warmup:
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
        out[name] = ev0.elapsed_time(ev1) / args.steps
        losses[name] = cur
        del opt
        arms[name] = None
        torch.cuda.empty_cache()
    clocks = sampler.stop()
    tokens = batch * seq
    ms = out["mxfp8_dwlinear"]
    print(json.dumps({
        "metric": "decoder_train_tokens_per_s", "value": tokens / ms * 1e3, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "mxfp8 linears (e4m3+e8m0, fp32 accumulate), bf16 elsewhere", "data": "synthetic",
        "config": {"workload": "preln_decoder_12x1024_ffn4096_vocab32000_b8_s2048_train_step", "dwlinear_modules": n_dw,
                   "linear_tflop_per_step": 6.0 * lin_params * tokens / 1e12, "optimizer": "AdamW(fused)",
                   "l2": "activations and weights far larger than L2"},
        "bf16_nn_linear": {"ms_per_step": out["bf16_nn_linear"], "tokens_per_s": tokens / out["bf16_nn_linear"] * 1e3},
        "speedup_vs_bf16_nn_linear": out["bf16_nn_linear"] / ms,
        "loss_first_last": {k: [v[0], v[-1]] for k, v in losses.items()},
        "e2e": {"value": tokens / ms * 1e3, "unit": "tokens/s", "h2d_bytes_per_step": tokens * 8, "d2h_bytes_per_step": 4,
                "api": "deepwell_b200.optimize(model, precision='mxfp8'); ids host->device and loss.item() every step"},
        "clocks": clocks}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="deepwell_b200", choices=["deepwell_b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--variant", type=int, default=0, help="GEMM kernel variant (0 = automatic)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sweep-quantize", action="store_true",
                    help="quantise-only bandwidth sweep (K in {128,1024,4096,16384}, 2^20..2^32 elements, both directions)")
    ap.add_argument("--emulate-world", type=int, default=0,
                    help="tuning aid: on one GPU, run the shard sizes rank 0 would get in a job of this many GPUs")
    ap.add_argument("--serial", action="store_true", help="quantise and GEMM on one stream (no overlap between layers)")
    ap.add_argument("--profile-case", default=None, choices=["gemm", "quant_row", "quant_both", "quant_col"],
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
    if args.profile_case:
        run_profile_case(args)
        return
    if args.sweep_quantize:
        run_quantize_sweep(args)
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
    stream = torch.cuda.current_stream(dev)          # GEMMs (and the step timer) run here
    st = stream.cuda_stream
    # The four layers are independent problems, so the (HBM-bound) quantisation of layer i+1 runs on a
    # second stream underneath the (tensor-bound) GEMM of layer i.  --serial keeps everything on one stream.
    qstream = stream if args.serial else torch.cuda.Stream(dev)
    sq = qstream.cuda_stream
    for l in layers:
        l["quantised"] = torch.cuda.Event()            # operands of this layer are ready
        l["consumed"] = torch.cuda.Event()             # the GEMM that read them has finished
    gemm_events = []

    def step(record: bool):
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
            launches += 3
        return launches

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(warmup):
        step(False)
    nv.check_status(dev)

    sampler = ClockSampler(local_rank)
    barrier()
    sampler.start()
    t_start, t_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    qstream.wait_event(t_start)                       # nothing of the timed steps starts before the timer
    launches = 0
    for _ in range(args.steps):
        launches += step(True)
    t_stop.record(stream)                             # the last GEMM depends on every quantisation before it
    barrier()
    clocks = sampler.stop()
    nv.check_status(dev)
    elapsed_ms = t_start.elapsed_time(t_stop)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = total_flops() / (ms_per_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel (GEMM), live CUDA-event durations of this rank ----
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_events)
    gemm_flops = args.steps * sum(2.0 * M_TOKENS * l["n"] * l["k"] for l in layers)
    achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12
    peaks = measured_peaks()
    peak = 2.0 * peaks["bf16_tflops_sustained"]
    roofline = {"bound": "tensor", "kernel": "mx_gemm_kernel", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": GEMM_DRAM_TRAFFIC_BYTES if world == 1 else None,
                "traffic_note": "mean DRAM bytes per GEMM launch (ncu, N = 1); algorithmic mean A + B + D = 5.16e8",
                "peak_basis": f"2 x bf16_tflops_sustained of {peaks['source']} MEASURED_PEAKS (MXFP8 issues at twice the "
                              "bf16 tensor rate); nominal dense MXFP8 is 4500",
                "frac_of_nominal_4500": achieved / NOMINAL_MXFP8_TFLOPS,
                "gemm_ms_per_step": gemm_ms / args.steps, "launches_timed": len(gemm_events)}

    # the same GEMM launches with nothing else on the GPU (in the timed region the next layer's
    # quantisation runs underneath them and takes its share of power and issue slots)
    if not args.serial:
        torch.cuda.synchronize(dev)
        alone = []
        for _ in range(3):
            for l in layers:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                nv.check(L.dw_mxfp8_gemm(l["xc"].data_ptr(), l["xs"].data_ptr(), l["wc"].data_ptr(), l["ws"].data_ptr(),
                                         l["y"].data_ptr(), None, M_TOKENS, l["n"], l["k"], 1.0, 0.0, None, 0,
                                         status.data_ptr(), st), "gemm")
                e1.record(stream)
                alone.append((e0, e1))
        torch.cuda.synchronize(dev)
        alone_ms = sum(a.elapsed_time(b) for a, b in alone) / 3
        alone_tf = sum(2.0 * M_TOKENS * l["n"] * l["k"] for l in layers) / (alone_ms * 1e-3) / 1e12
        roofline["achieved_alone"] = alone_tf
        roofline["frac_alone"] = alone_tf / peak
        roofline["note"] = ("achieved/frac: live in the timed region, where the next layer's quantiser shares the GPU; "
                            "achieved_alone: the same four launches back to back with nothing else running")

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
    roofline_q = {"bound": "hbm", "kernel": "mx_quant_row_kernel", "achieved": q_gbs, "peak": peaks["hbm_gbs"],
                  "unit": "GB/s", "frac": q_gbs / peaks["hbm_gbs"], "frac_of_nominal_8000": q_gbs / 8000.0,
                  "shape": [M_TOKENS, big["k"]], "bytes_per_element": 3.03125}

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
            torch.cuda.synchronize(dev)

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        barrier()
        dt = (time.perf_counter() - t0) / args.e2e_steps
        if world > 1:
            t = torch.tensor([dt], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e = {"value": total_flops() / dt / 1e12, "unit": "TFLOP/s",
               # whole-job bytes per step: every row of every X crosses PCIe once (N > 1: each rank uploads its
               # slice, NVLink replicates it), every rank downloads its shard of every Y
               "h2d_bytes_per_step": int(sum(hx.numel() * 2 for hx in host_x)) * (1 if even_rows or world == 1 else world),
               "d2h_bytes_per_step": int(sum(hy.numel() * 2 for hy in host_y)) * world, "ms_per_step": dt * 1e3,
               "api": "deepwell_b200.cutlass_kernels.BlackwellGemmKernel.gemm, pinned host X in, pinned host Y out, "
                      "copies on their own streams" + ("; X uploaded as 1/N row slices and all-gathered over NVLink"
                                                       if even_rows else "")}
        nv.check_status(dev)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        use_all_host_threads()
        cpu_baseline, _ = time_cpu(steps=2, warmup=1)

    if rank == 0:
        bytes_step = sum(l["x"].numel() * 2 + l["w"].numel() * 2 + l["y"].numel() * 2 for l in layers)
        line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "mxfp8(e4m3+e8m0), fp32 accumulate, bf16 out", "data": "synthetic",
                "config": {"workload": WORKLOAD, "M": M_TOKENS, "layers": {n: [k, nn] for n, k, nn in LAYERS},
                           "parallelism": f"N-sharded x{world}, X replicated, no data-path collective",
                           "step": "per layer: quantise X, quantise W shard, block-scaled GEMM"
                                   + ("" if args.serial else "; quantisation of the next layer on a second stream"),
                           "l2": f"inputs larger than L2: {bytes_step / 1e9:.2f} GB touched per step per GPU",
                           "gemm_variant": args.variant,
                           **({"emulated_world": args.emulate_world,
                               "note": "TUNING RUN: one rank's shard on one GPU; value is not a job throughput"}
                              if args.emulate_world else {})},
                "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline,
                "roofline_quantize": roofline_q, "cpu_baseline": cpu_baseline}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
