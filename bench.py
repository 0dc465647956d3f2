#!/usr/bin/env python
"""Benchmark of the differential-attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|reference_triton|flash_composition]
                    [--workload NAME]

A step is one forward + backward over one batch of synthetic fp16 input.  The default workload is
B=4, H=16, N=4096, D=64 (v width 128), the shape the headline metric is quoted on.  With N>1 GPUs every rank
runs that shape on its own (batch*head) shard (weak scaling, no data-path collective); the d(lambda)
partials are summed on the host.  `value` is credited TFLOP/s (fwd 8 N^2 D + bwd 20 N^2 D per head) over all
ranks with inputs resident in HBM, timed with CUDA events, max over ranks.  `e2e` is the same metric through
the Python operator with HOST (pinned) inputs and outputs, copies inside the timed region.  Every line also
carries
  * `check`: outside the timed regions every rank compares one seeded head of its shard (y and the five
    gradients) and its d(lambda) partial with the fp32 oracle evaluated on its own GPU;
  * `config5`: the batch-sharded workload B=64, H=32, N=4096, D=64 split over the ranks (same total
    work at every N: strong scaling), d(lambda) partials summed on the host;
  * `sustained`: a second timed loop of at least one second when the K timed steps last under half a second.
`--impl reference` times the reference's own PyTorch path (`MultiheadDiffAttn`, src/layers.py:49-80) on the
host cores when `baseline/_ref` holds the reference modules (see baseline/ref_loader.py), else the CPU
restatement under oracle/, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

WORKLOADS = {
    # name: (B, H, N, D, input scale, lambda, lambda_init, rms_norm)
    "b4h16n4096d64": (4, 16, 4096, 64, 1.0, 0.5, 0.8, True),        # headline shape
    "b1h32n16384d64": (1, 32, 16384, 64, 0.5, 0.3, 0.8, True),      # long sequence
    "b8h8n8192d128": (8, 8, 8192, 128, 1.0, 0.7, 0.2, False),       # wide head, RMSNorm off
    "b8h32n4096d64": (8, 32, 4096, 64, 1.0, 0.5, 0.8, True),        # one eighth of B=64 H=32
    "b4h16n4096d32": (4, 16, 4096, 32, 0.5, 0.5, 0.8, True),        # the reference's benchmark point H=16 D=32 N=4096 (src/benchmark.py:19-25)
    "b1h4n4096d128": (1, 4, 4096, 128, 1.0, 0.7, 0.2, False),       # small wide-head case for profiler captures
}
DEFAULT_WORKLOAD = "b4h16n4096d64"
SPLIT = (64, 32, 4096, 64, 1.0, 0.5, 0.8, True)                     # batch-sharded workload, split over the ranks
CPU_SMALL = (2, 16, 512, 32, 1.0, 0.5, 0.8, True)                   # the CPU-runnable shape: B=2 H=16 N=512 D=32, fp32
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from an ncu capture of this workload (its summary, with
# the command, sits under profiles/); reported only for the workload and flags of that capture.
NCU_TRAFFIC = {"workload": DEFAULT_WORKLOAD, "source": "ncu --set full capture of the kernels of commit 99934c7, summarised under profiles/",
               "bytes": {"diffattn_fwd64_kernel": 306.9e6, "diffattn_bwd_pre_kernel": 255.9e6,
                         "diffattn_bwd_dkdv64_kernel": 380.0e6, "diffattn_bwd_dq64_kernel": 324.5e6}}
METRIC = "diff-attn fwd+bwd TFLOP/s (credited 28*B*H*N^2*D), fp16"
NOMINAL_TFLOPS = 2250.0


def flops(b, h, n, d):
    unit = float(b) * h * n * n * d
    return 8.0 * unit, 20.0 * unit


def measured_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            j = json.load(f)
        return {"burst": float(j["bf16_tflops"]), "sustained": float(j["bf16_tflops_sustained"]),
                "hbm_gbs": float(j["hbm_gbs"]), "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a timed region runs (read only)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        # "under load" = samples whose power draw is at least 60 % of the highest one seen
        load = [c for c, w in zip(sm, power) if w >= 0.6 * max(power)] if power else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "samples_under_load": len(load),
                "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------------------
# CPU arms
# ------------------------------------------------------------------------------------------------------------
def _reference_layers():
    """The reference's own `layers` module from baseline/_ref, or (None, why)."""
    try:
        from baseline import ref_loader
        if not ref_loader.installed():
            ref_loader.install()            # only succeeds where the reference checkout is present
        return ref_loader.load(), None
    except Exception as e:                  # not installed on this box, or an import failure inside the reference
        return None, f"{type(e).__name__}: {e}"


def _cpu_inputs(b, h, n, d, scale, seed):
    g = torch.Generator().manual_seed(seed)
    def draw(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(torch.float16).float()
    q1, q2, k1, k2 = (draw(b, h, n, d) for _ in range(4))
    v = draw(b, h, n, 2 * d)
    dy = torch.randn(b, h, n, 2 * d, generator=g, dtype=torch.float32).to(torch.float16).float()
    return q1, q2, k1, k2, v, dy


def cpu_time(shape, steps, warmup, threads=None):
    """Forward and forward+backward wall time of the CPU path (fp32) at `shape` = (b, h, n, d, scale, lam, lam_init, rms).
    The literal reference when installed (kind "reference"), else the oracle's restatement (kind "port")."""
    b, h, n, d, scale, lam, lam_init, rms = shape
    # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1 to every rank)
    torch.set_num_threads(threads or os.cpu_count() or 1)
    layers, why = _reference_layers()
    q1, q2, k1, k2, v, dy = _cpu_inputs(b, h, n, d, scale, 4321)
    lam_t = torch.tensor([lam], dtype=torch.float32)             # shape [1]: a 0-dim fp32 lambda breaks the reference's
                                                                 # fp16 matmul (src/layers.py:65-70)
    t_f, t_fb = [], []
    if layers is not None:
        kind = "reference"
        for i in range(warmup + steps):
            leaves = [t.clone().requires_grad_(True) for t in (q1, q2, k1, k2, v)]
            lam_leaf = lam_t.clone().requires_grad_(True)
            t0 = time.perf_counter()
            y = layers.MultiheadDiffAttn(*leaves, lambda_scale=lam_leaf, lambda_init=lam_init, rms_norm=rms)
            t1 = time.perf_counter()
            y.backward(dy)
            t2 = time.perf_counter()
            if i >= warmup:
                t_f.append(t1 - t0); t_fb.append(t2 - t0)
    else:
        from oracle import diffattn_oracle as oracle             # CPU-baseline leg: the restatement is timed as the baseline
        kind = "port"
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            oracle.forward(q1, q2, k1, k2, v, lam_t, lam_init, rms)
            t1 = time.perf_counter()
            oracle.forward_backward_autograd(q1, q2, k1, k2, v, lam_t, dy, lam_init, rms)
            t2 = time.perf_counter()
            if i >= warmup:
                t_f.append(t1 - t0); t_fb.append(t2 - t1)
    f, bk = flops(b, h, n, d)
    ms_f, ms_fb = 1e3 * statistics.median(t_f), 1e3 * statistics.median(t_fb)
    return {"kind": kind, "why_not_reference": why if kind == "port" else None, "fwd_ms": ms_f, "fwd_bwd_ms": ms_fb,
            "tflops": (f + bk) / (ms_fb * 1e-3) / 1e12, "threads": torch.get_num_threads(), "os_cpu_count": os.cpu_count(),
            "timed": len(t_fb), "warmup": warmup, "shape": f"B={b} H={h} N={n} D={d} fp32"}


def cpu_baseline_block(workload, steps, warmup, with_small=True):
    """`cpu_baseline`: a bounded sample of the workload (2 of its heads, all host threads) and, beside it, the
    complete CPU-runnable shape B=2 H=16 N=512 D=32 (3 warm-up, 7 timed, median)."""
    b, h, n, d, scale, lam, lam_init, rms = WORKLOADS[workload]
    heads = 1                 # the reference rounds P to fp16 on the CPU (src/layers.py:65,68): about 2 s per head at N=4096 on 8 cores
    r = cpu_time((1, heads, n, d, scale, lam, lam_init, rms), steps, warmup)
    block = {"value": r["tflops"], "unit": "TFLOP/s", "cores": r["threads"], "kind": r["kind"],
             "sample": f"{heads} of {b * h} heads of {workload} (B=1,H={heads},N={n},D={d}), fp32 forward + autograd backward, "
                       f"median of {r['timed']} timed passes after {warmup} warm-up",
             "ms_per_sample": r["fwd_bwd_ms"], "os_cpu_count": r["os_cpu_count"]}
    if r["why_not_reference"]:
        block["why_port"] = r["why_not_reference"]
    if with_small:
        c1 = cpu_time(CPU_SMALL, 7, 3)
        block["c1"] = {"shape": c1["shape"], "kind": c1["kind"], "fwd_ms": c1["fwd_ms"], "fwd_bwd_ms": c1["fwd_bwd_ms"],
                       "tflops": c1["tflops"], "threads": c1["threads"], "os_cpu_count": c1["os_cpu_count"],
                       "timed": c1["timed"], "warmup": c1["warmup"]}
    return block, r


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    b, h, n, d, *_ = WORKLOADS[args.workload]
    block, r = cpu_baseline_block(args.workload, max(args.steps, 1), args.warmup, with_small=not args.no_cpu_small)
    line = {
        "impl": "reference", "metric": METRIC, "value": block["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["fwd_bwd_ms"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: B={b} H={h} N={n} D={d} (v width {2 * d}), rms_norm, fwd+bwd",
                   "note": ("the reference's own MultiheadDiffAttn (src/layers.py:49-80) imported from baseline/_ref"
                            if block["kind"] == "reference" else
                            "CPU restatement of the reference's MultiheadDiffAttn (PyTorch ops, fp32): baseline/_ref is absent")},
        "cpu_baseline": block,
        "e2e": {"value": block["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ------------------------------------------------------------------------------------------------------------
# informational same-box GPU arms (library / reference code, not the product)
# ------------------------------------------------------------------------------------------------------------
def run_reference_triton(args):
    """The reference's own Triton kernel (`MultiheadDiffAttnKernel`, src/layers.py:10-26, src/kernel.py) under the
    image's Triton, one GPU: first at the reference's self-test shape (B2 H2 N256 D32, src/kernel.py:581-596), then at
    the workload.  Any failure prints the arm's `unavailable` line and stops."""
    layers, why = _reference_layers()
    if layers is None:
        emit({"impl": "reference_triton", "unavailable": f"baseline/_ref not installed: {why}"})
        return
    dev = torch.device("cuda", 0)
    try:
        def run(b, h, n, d, scale, lam, lam_init, rms, steps, warmup):
            g = torch.Generator(device=dev).manual_seed(7)
            def draw(*shape):
                return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale).to(torch.float16).requires_grad_(True)
            q1, q2, k1, k2 = (draw(b, h, n, d) for _ in range(4))
            v = draw(b, h, n, 2 * d)
            dy = torch.rand(b, h, n, 2 * d, generator=g, device=dev, dtype=torch.float32).to(torch.float16)
            lam_t = torch.tensor([lam], dtype=torch.float16, device=dev, requires_grad=True)
            def step():
                y = layers.MultiheadDiffAttnKernel(q1, q2, k1, k2, v, lam_t, lam_init, rms)
                y.backward(dy)
                for t in (q1, q2, k1, k2, v, lam_t):
                    t.grad = None
                return y
            for _ in range(warmup):
                step()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                y = step()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / steps, y
        ms_small, y_small = run(2, 2, 256, 32, 0.5, 0.5, 0.8, True, 3, 2)
        if not bool(torch.isfinite(y_small).all()):
            raise RuntimeError("non-finite output at the self-test shape")
        b, h, n, d, scale, lam, lam_init, rms = WORKLOADS[args.workload]
        ms, _ = run(b, h, n, d, scale, lam, lam_init, rms, max(args.steps, 3), max(args.warmup, 3))
        f, bk = flops(b, h, n, d)
        emit({"impl": "reference_triton", "metric": METRIC, "value": (f + bk) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
              "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "fp16",
              "data": "synthetic", "selftest_shape_ms": ms_small,
              "config": {"workload": args.workload, "note": "the reference's Triton kernel from baseline/_ref under this image's Triton; "
                         "informational same-box arm"}})
    except Exception as e:
        emit({"impl": "reference_triton", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"})


def run_reference_protocol_sweep(args):
    """The reference's runtime benchmark protocol (src/benchmark.py:19-25,83-148): H=16, D=32 (v width 64), fp16,
    forward and forward+backward, rms_norm on, N in {512,...,16384} with batch 16384/N; median of per-call CUDA-event
    times (the reference reports do_bench medians).  One JSON line per N; one GPU."""
    from triton_diff_attn_b200 import MultiheadDiffAttnKernel
    dev = torch.device("cuda", 0)
    h, d = 16, 32
    for n in (512, 1024, 2048, 4096, 8192, 16384):
        b = 16384 // n
        g = torch.Generator(device=dev).manual_seed(n)
        def draw(*shape):
            return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * 0.5).to(torch.float16).requires_grad_(True)
        q1, q2, k1, k2 = (draw(b, h, n, d) for _ in range(4))
        v = draw(b, h, n, 2 * d)
        dy = torch.rand(b, h, n, 2 * d, generator=g, device=dev, dtype=torch.float32).to(torch.float16)
        lam = torch.tensor([0.5], dtype=torch.float16, device=dev, requires_grad=True)

        def fwd_only():
            return MultiheadDiffAttnKernel(q1, q2, k1, k2, v, lam, 0.8, True)

        def fwd_bwd():
            fwd_only().backward(dy)
            for t in (q1, q2, k1, k2, v, lam):
                t.grad = None

        res = {}
        for name, fn in (("fwd", fwd_only), ("fwd_bwd", fwd_bwd)):
            for _ in range(max(args.warmup, 3)):
                fn()
            times = []
            for _ in range(max(args.steps, 10)):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); fn(); e1.record(); torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1))
            res[name] = statistics.median(times)
        # peak device memory of one call, as the reference's memory benchmark takes it (src/benchmark.py:181-250):
        # allocator peak in MiB after reset, inputs and dY included
        peak = {}
        for name in ("fwd", "fwd_bwd"):
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats(dev)
            y = fwd_only()
            if name == "fwd_bwd":
                y.backward(dy)
            torch.cuda.synchronize()
            peak[name] = torch.cuda.max_memory_allocated(dev) / 2**20
            del y
            for t in (q1, q2, k1, k2, v, lam):
                t.grad = None
        resident = sum(t.numel() * t.element_size() for t in (q1, q2, k1, k2, v, dy)) / 2**20
        f, bk = flops(b, h, n, d)
        emit({"protocol": "reference src/benchmark.py:19-25", "B": b, "H": h, "N": n, "D": d,
              "fwd_peak_mib": peak["fwd"], "fwd_bwd_peak_mib": peak["fwd_bwd"], "inputs_and_dy_mib": resident,
                          "fwd_ms_median": res["fwd"], "fwd_bwd_ms_median": res["fwd_bwd"],
                          "fwd_tflops": f / (res["fwd"] * 1e-3) / 1e12, "fwd_bwd_tflops": (f + bk) / (res["fwd_bwd"] * 1e-3) / 1e12})


def run_flash_composition(args):
    """Informational same-box LIBRARY baseline, not the product and not the reference arm: differential attention
    composed from FlashAttention-2 calls, the construction the reference compares its kernel with.  With
    baseline/_ref installed the reference's own `MultiheadFlashDiffAttn` (src/layers.py:104-148) is called; else
    the same construction written here against the flash_attn package of this image.  One GPU only."""
    from flash_attn import flash_attn_func
    b, h, n, d, scale, lam, lam_init, rms = WORKLOADS[args.workload]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1234)
    def draw(*shape):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale).to(torch.float16).requires_grad_(True)
    layers, _ = _reference_layers()
    literal = layers is not None and hasattr(layers, "MultiheadFlashDiffAttn") and not args.no_literal
    lam_t = torch.tensor([lam], dtype=torch.float16, device=dev, requires_grad=True)
    if literal:
        # the reference's function takes [B, H, N, D] like its other layers
        q1, q2, k1, k2 = (draw(b, h, n, d) for _ in range(4))
        v = draw(b, h, n, 2 * d)
        dy = torch.randn(b, h, n, 2 * d, generator=g, device=dev, dtype=torch.float32).to(torch.float16)
    else:
        q1, q2, k1, k2 = (draw(b, n, h, d) for _ in range(4))     # flash_attn wants [B, N, H, D]
        v = draw(b, n, h, 2 * d)
        dy = torch.randn(b, n, h, 2 * d, generator=g, device=dev, dtype=torch.float32).to(torch.float16)

    def step():
        if literal:
            a = layers.MultiheadFlashDiffAttn(q1, q2, k1, k2, v, lam_t, lam_init, rms)
        else:
            v1, v2 = v[..., :d], v[..., d:]
            a1 = torch.cat([flash_attn_func(q1, k1, v1), flash_attn_func(q1, k1, v2)], dim=-1)
            a2 = torch.cat([flash_attn_func(q2, k2, v1), flash_attn_func(q2, k2, v2)], dim=-1)
            a = a1 - lam_t * a2
            if rms:
                a = (1.0 - lam_init) * a * torch.rsqrt((a.float() ** 2).mean(-1, keepdim=True) + 1e-5).to(a.dtype)
        a.backward(dy.reshape(a.shape) if a.shape != dy.shape else dy)
        for t in (q1, q2, k1, k2, v, lam_t):
            t.grad = None

    try:
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    except Exception as e:
        emit({"impl": "flash_composition", "unavailable": f"{type(e).__name__}: {str(e)[:300]}", "literal_reference_layer": literal})
        return
    ms = e0.elapsed_time(e1) / args.steps
    f, bk = flops(b, h, n, d)
    emit({"impl": "flash_composition", "metric": METRIC, "value": (f + bk) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                      "dtype": "fp16", "data": "synthetic", "literal_reference_layer": literal,
                      "config": {"workload": args.workload, "note": "library baseline: FlashAttention-2 calls + torch ops; credited "
                                 "flops as for the product (the composition executes S twice per branch)"}})


_REAL_STDOUT = None


def _quiet_stdout():
    """Send everything libraries print on file descriptor 1 (NCCL's version banner, for one) to stderr and
    keep the real stdout for the result lines, so that a run prints exactly one JSON line there."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(obj):
    data = (json.dumps(obj) + "\n").encode()
    sys.stdout.flush()
    os.write(_REAL_STDOUT if _REAL_STDOUT is not None else 1, data)


# ------------------------------------------------------------------------------------------------------------
# the product arm
# ------------------------------------------------------------------------------------------------------------
class Problem:
    """Device tensors of one shape plus a filled DiffAttnParams; fwd()/bwd() call the C ABI directly."""

    def __init__(self, shape, dev, seed, io_dtype, causal=False, dropout=0.0, single_pass=False):
        from triton_diff_attn_b200 import _lib, layers
        self._lib = _lib
        b, h, n, d, scale, lam, lam_init, rms = shape
        self.shape, self.dev = shape, dev
        g = torch.Generator(device=dev).manual_seed(seed)

        def draw(*s):
            return (torch.randn(*s, generator=g, device=dev, dtype=torch.float32) * scale).to(io_dtype)

        self.q1, self.q2, self.k1, self.k2 = (draw(b, h, n, d) for _ in range(4))
        self.v = draw(b, h, n, 2 * d)
        self.dy = torch.randn(b, h, n, 2 * d, generator=g, device=dev, dtype=torch.float32).to(io_dtype)
        self.lam_t = torch.tensor([lam], dtype=torch.float32, device=dev)
        self.y, self.a2 = torch.empty_like(self.v), torch.empty_like(self.v)
        self.lse1 = torch.empty(b, h, n, dtype=torch.float32, device=dev)
        self.lse2, self.rstd = torch.empty_like(self.lse1), torch.empty_like(self.lse1)
        self.dq1, self.dq2, self.dk1, self.dk2 = (torch.empty_like(self.q1) for _ in range(4))
        self.dv = torch.empty_like(self.v)
        self.dlam = torch.zeros(1, dtype=torch.float32, device=dev)
        p = _lib.new_params()
        layers._fill_common(p, self.q1, self.q2, self.k1, self.k2, self.v, self.lam_t, lam_init, rms,
                            (self.y, self.a2, self.lse1, self.lse2, self.rstd), causal, layers.dropout_threshold(dropout),
                            20241125, single_pass=single_pass)
        self.ws_bytes = int(_lib.lib.diffattn_workspace_bytes(p))
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        p.dy = self.dy.data_ptr()
        p.dq1, p.dq2, p.dk1, p.dk2, p.dv = (t.data_ptr() for t in (self.dq1, self.dq2, self.dk1, self.dk2, self.dv))
        p.dlambda = self.dlam.data_ptr()
        p.workspace, p.workspace_bytes = self.ws.data_ptr(), self.ws_bytes
        self.p, self.pref = p, ctypes.byref(p)
        self.fused = bool(single_pass) and d <= 64
        L = _lib
        self.stage_list = ([("preprocess", L.STAGE_PRE), ("dkdv_dq_single_pass", L.STAGE_FUSED), ("dq_finish", L.STAGE_DQ_FINISH)]
                           if self.fused else [("preprocess", L.STAGE_PRE), ("dkdv", L.STAGE_DKDV), ("dq", L.STAGE_DQ)])

    def fwd(self):
        self._lib.check(self._lib.lib.diffattn_fwd(self.pref), "diffattn_fwd")

    def bwd(self, stages=None):
        if stages is None:
            self._lib.check(self._lib.lib.diffattn_bwd(self.pref), "diffattn_bwd")
        else:
            self._lib.check(self._lib.lib.diffattn_bwd_stages(self.pref, stages), "diffattn_bwd_stages")

    def step(self):
        self.fwd()
        self.dlam.zero_()
        self.bwd()

    def check_one_head(self, bi, hi, lam_init_rms=None):
        """y and the five gradients of head (bi, hi) against the fp32 oracle evaluated on this GPU (TF32 off)."""
        from oracle import diffattn_oracle as oracle        # checker only, outside every timed region
        b, h, n, d, scale, lam, lam_init, rms = self.shape
        sl = lambda t: t[bi:bi + 1, hi:hi + 1].contiguous()
        want = oracle.backward_closed_form(sl(self.q1), sl(self.q2), sl(self.k1), sl(self.k2), sl(self.v), torch.tensor([lam]),
                                           sl(self.dy), lam_init, rms, device=self.dev)
        worst_rel, worst_abs = 0.0, 0.0
        for nm, t in (("y", self.y), ("dq1", self.dq1), ("dq2", self.dq2), ("dk1", self.dk1), ("dk2", self.dk2), ("dv", self.dv)):
            m = oracle.error_metrics(sl(t), want[nm])
            worst_rel = max(worst_rel, m["rel_l2"])
            worst_abs = max(worst_abs, m["max_abs"] / max(1.0, float(want[nm].abs().max())))
        return worst_rel, worst_abs

    def dlambda_oracle(self):
        """-sum(E2) over every head of this problem, fp32 oracle on this GPU one head at a time, summed in fp64."""
        from oracle import diffattn_oracle as oracle
        b, h, n, d, scale, lam, lam_init, rms = self.shape
        total, mag = 0.0, 0.0
        for bi in range(b):
            for hi in range(h):
                sl = lambda t: t[bi:bi + 1, hi:hi + 1].contiguous()
                w = oracle.backward_closed_form(sl(self.q1), sl(self.q2), sl(self.k1), sl(self.k2), sl(self.v), torch.tensor([lam]),
                                                sl(self.dy), lam_init, rms, device=self.dev)
                total += float(w["dlambda"])
                mag += float(w["e2"].double().abs().sum())
        return total, mag


def host_overhead(args, dev):
    """Host microseconds per diffattn_fwd / diffattn_bwd call (CPU clock around enqueues only) at a small shape."""
    from triton_diff_attn_b200 import _lib
    out = {}
    for d in (64, 32, 128):
        pr = Problem((2, 4, 128, d, 1.0, 0.5, 0.8, True), dev, 1, torch.float16)
        for name, fn in (("fwd", pr.fwd), ("bwd", pr.bwd)):
            for _ in range(20):
                fn()
            torch.cuda.synchronize()
            tot = 0.0
            for _ in range(10):
                t0 = time.perf_counter()
                for _ in range(100):
                    fn()
                tot += time.perf_counter() - t0
                torch.cuda.synchronize()
            out[f"d{d}_{name}_us"] = tot / 1000 * 1e6
    emit({"host_us_per_call": out, "shape": "B=2 H=4 N=128, 1000 enqueues each, host clock around the calls only"})


def main():
    _quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference_triton", "flash_composition"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cpu-small", action="store_true", help="reference arm: skip the B=2 H=16 N=512 D=32 timing")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-split", action="store_true", help="skip the B=64 H=32 batch-sharded block")
    ap.add_argument("--no-check", action="store_true", help="skip the per-rank comparison with the oracle")
    ap.add_argument("--no-literal", action="store_true", help="flash_composition: do not call the reference's own layer")
    ap.add_argument("--single-pass", action="store_true", help="time the one-pass backward (atomic dQ partial sums; head dim <= 64)")
    ap.add_argument("--io-dtype", default="fp16", choices=["fp16", "bf16"],
                    help="16-bit type of the tensors: fp16 (the reference's and the headline) or bf16 (extension)")
    ap.add_argument("--dropout", type=float, default=0.0, help="attention dropout probability (extension); flops are "
                    "credited as without dropout")
    ap.add_argument("--causal", action="store_true", help="causal mask (extension); flops credited for the visible "
                    "N(N+1)/2 pairs only")
    ap.add_argument("--sweep-reference-protocol", action="store_true",
                    help="instead of the one-line benchmark: the reference's own sweep (src/benchmark.py:19-25): "
                         "H=16, D=32, fp16, rms_norm, N in 512..16384 with B = 16384/N; one JSON line per N")
    ap.add_argument("--host-overhead", action="store_true", help="instead of the benchmark: host microseconds per C-ABI call")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference(args)
        return
    if args.impl == "reference_triton":
        run_reference_triton(args)
        return
    if args.impl == "flash_composition":
        run_flash_composition(args)
        return
    if args.sweep_reference_protocol:
        run_reference_protocol_sweep(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    torch.backends.cuda.matmul.allow_tf32 = False            # the oracle's fp32 matmuls on this GPU stay fp32
    if args.host_overhead:
        host_overhead(args, dev)
        return
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from triton_diff_attn_b200 import _lib, MultiheadDiffAttnKernel, shard_batch, sum_dlambda_on_host, device_status

    shape = WORKLOADS[args.workload]
    b, h, n, d, scale, lam, lam_init, rms = shape
    io_dtype = torch.bfloat16 if args.io_dtype == "bf16" else torch.float16
    pr = Problem(shape, dev, 1234 + rank, io_dtype, args.causal, args.dropout, args.single_pass)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters):
        """CUDA events on the launching (current) stream, barrier + synchronize on both sides; max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / iters

    def all_sum(x):
        t = torch.tensor([float(x)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t)

    def all_max(x):
        t = torch.tensor([float(x)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        pr.step()
    device_status(local_rank)
    ms_step = timed(pr.step, args.steps)
    # per-kernel durations (each kernel alone, same resident inputs); the inputs are larger than L2
    ms_fwd = timed(pr.fwd, args.steps)
    ms_stage = {name: timed(lambda s=s: pr.bwd(s), args.steps) for name, s in pr.stage_list}
    ms_bwd = timed(pr.bwd, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    device_status(local_rank)

    f_fwd, f_bwd = flops(b, h, n, d)
    if args.causal:
        f_fwd, f_bwd = f_fwd * (n + 1) / (2.0 * n), f_bwd * (n + 1) / (2.0 * n)
    total_flops = (f_fwd + f_bwd) * world
    value = total_flops / (ms_step * 1e-3) / 1e12

    # ---- a longer loop when the timed region was short (boost clocks): at least one second
    sustained = None
    if args.steps * ms_step < 500.0:
        n_long = int(math.ceil(1000.0 / ms_step))
        s2 = ClockSampler(local_rank)
        if rank == 0:
            s2.start()
        ms_long = timed(pr.step, n_long)
        sustained = {"steps": n_long, "ms_per_step": ms_long, "value": total_flops / (ms_long * 1e-3) / 1e12, "unit": "TFLOP/s",
                     "clocks": s2.stop() if rank == 0 else None}

    # ---- correctness on every rank, outside the timed regions: one seeded head and the rank's d(lambda) partial
    check = None
    pr.dlam.zero_(); pr.fwd(); pr.bwd()
    dl_rank = float(pr.dlam.cpu())
    dl_total = sum_dlambda_on_host(pr.dlam)
    if not args.no_check and not args.causal and not args.dropout:
        gsel = torch.Generator().manual_seed(99 + rank)
        bi, hi = int(torch.randint(0, b, (1,), generator=gsel)), int(torch.randint(0, h, (1,), generator=gsel))
        rel, mabs = pr.check_one_head(bi, hi)
        dl_want, dl_mag = pr.dlambda_oracle()
        loosen = 8.0 if args.io_dtype == "bf16" else 1.0
        dl_tol = loosen * max(1e-2 * abs(dl_want), 1e-4 * dl_mag)
        ok = (rel <= loosen * 1e-3) and (mabs <= loosen * 2e-2) and (abs(dl_rank - dl_want) <= dl_tol)
        check = {"ranks_ok": int(all_sum(1.0 if ok else 0.0)), "ranks": world, "worst_rel_l2": all_max(rel),
                 "worst_max_abs_scaled": all_max(mabs), "dlambda_rel": all_max(abs(dl_rank - dl_want) / max(abs(dl_want), 1e-30)),
                 "dlambda_err_over_sum_abs_e2": all_max(abs(dl_rank - dl_want) / max(dl_mag, 1e-30)),
                 "tolerance": "rel-L2 <= 1e-3, max-abs <= 2e-2 (x max|ref| above 1); d(lambda) within max(1e-2 |dl|, 1e-4 sum|E2|)",
                 "how": "fp32 oracle on each rank's own GPU (TF32 off): one seeded head for y and 5 gradients, every head for d(lambda)"}

    # ---- end to end through the Python operator with host buffers
    e2e = None
    if not args.no_e2e:
        host_in = [t.cpu().pin_memory() for t in (pr.q1, pr.q2, pr.k1, pr.k2, pr.v, pr.dy)]
        host_out = [torch.empty_like(t, device="cpu").pin_memory() for t in (pr.y, pr.dq1, pr.dq2, pr.dk1, pr.dk2, pr.dv)]
        host_dl = torch.empty(1, dtype=torch.float32).pin_memory()
        h2d = sum(t.numel() * t.element_size() for t in host_in)
        d2h = sum(t.numel() * t.element_size() for t in host_out) + 4

        from triton_diff_attn_b200 import HostStepPipeline
        pipe = HostStepPipeline(dev)

        def e2e_run(iters):
            """iters steps through the host pipeline: every step copies its inputs from pinned host memory and
            its y / gradients / d(lambda) back; copies of neighbouring steps overlap with the kernels."""
            pipe.begin()
            for _ in range(iters):
                pipe.submit(host_in, host_out, host_dl, pr.lam_t, lam_init, rms, args.causal)
            pipe.end()

        # enough steps for the steady state to dominate the pipeline's fill and drain, about a second in all
        e2e_steps = max(10, min(100, int(1000.0 / (2.0 * ms_step))))
        e2e_run(3)
        ms_e2e = timed(lambda: e2e_run(e2e_steps), 1) / e2e_steps
        # each leg alone, a few steps: which of them bounds the overlapped figure
        dev_in = [torch.empty_like(t, device=dev) for t in host_in]
        def leg_h2d():
            for dst, src in zip(dev_in, host_in):
                dst.copy_(src, non_blocking=True)
        dev_out = [pr.y, pr.dq1, pr.dq2, pr.dk1, pr.dk2, pr.dv]
        def leg_d2h():
            for dst, src in zip(host_out, dev_out):
                dst.copy_(src, non_blocking=True)
        leaves = [t.detach().requires_grad_(True) for t in dev_in[:5]]
        def leg_kernels():
            lam_leaf = pr.lam_t.detach().clone().requires_grad_(True)
            MultiheadDiffAttnKernel(*leaves, lam_leaf, lam_init, rms, args.causal).backward(dev_in[5])
            for t in leaves:
                t.grad = None
        leg_h2d(); leg_kernels(); leg_d2h()
        ms_h2d, ms_d2h, ms_k = timed(leg_h2d, 5), timed(leg_d2h, 5), timed(leg_kernels, 5)
        e2e = {"value": total_flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "steps": e2e_steps,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "breakdown": {"h2d_ms": ms_h2d, "d2h_ms": ms_d2h, "kernels_ms": ms_k, "overlapped_ms": ms_e2e,
                             "h2d_gbs": h2d / ms_h2d / 1e6, "d2h_gbs": d2h / ms_d2h / 1e6,
                             "host_gbs_all_ranks_overlapped": world * (h2d + d2h) / ms_e2e / 1e6,
                             "bound": max((("h2d", ms_h2d), ("d2h", ms_d2h), ("kernels", ms_k)), key=lambda kv: kv[1])[0],
                             "note": "each leg timed alone (max over ranks); the pipeline can at best reach the longest leg"},
               "how": "HostStepPipeline: H2D, diffattn_fwd + diffattn_bwd and D2H of consecutive steps on three streams; two ring slots of preallocated device buffers, no allocator call per step"}
        del host_in, host_out, dev_in, leaves

    # ---- B=64 H=32 N=4096 D=64 split over the ranks along the batch (same total work at every N)
    split = None
    if not args.no_split and not args.causal and not args.dropout and args.workload == DEFAULT_WORKLOAD:
        sb, sh, sn, sd, sscale, slam, slam_init, srms = SPLIT
        lo, hi_ = shard_batch(sb, sh, rank, world)
        ps = Problem((hi_ - lo, sh, sn, sd, sscale, slam, slam_init, srms), dev, 5550 + lo, io_dtype, single_pass=args.single_pass)
        for _ in range(3):
            ps.step()
        split_steps = 5
        ms_split = timed(ps.step, split_steps)
        ps.dlam.zero_(); ps.fwd(); ps.bwd()
        device_status(local_rank)
        dl_split = sum_dlambda_on_host(ps.dlam)
        sf, sbk = flops(sb, sh, sn, sd)
        split = {"workload": f"B={sb} H={sh} N={sn} D={sd} split along the batch: {hi_ - lo} batches x {sh} heads per rank",
                 "scaling": "strong", "ms_per_step": ms_split, "steps": split_steps, "value": (sf + sbk) / (ms_split * 1e-3) / 1e12,
                 "unit": "TFLOP/s", "per_gpu_tflops": (sf + sbk) / (ms_split * 1e-3) / 1e12 / world,
                 "dlambda_host_sum": dl_split,
                 "efficiency_note": "strong-scaling efficiency = ms_per_step(1 GPU) / (N x ms_per_step(N GPUs)), from the 1-GPU line"}
        if not args.no_check:
            gsel = torch.Generator().manual_seed(199 + rank)
            bi, hi2 = int(torch.randint(0, hi_ - lo, (1,), generator=gsel)), int(torch.randint(0, sh, (1,), generator=gsel))
            rel, mabs = ps.check_one_head(bi, hi2)
            loosen = 8.0 if args.io_dtype == "bf16" else 1.0
            ok = rel <= loosen * 1e-3 and mabs <= loosen * 2e-2
            split["check"] = {"ranks_ok": int(all_sum(1.0 if ok else 0.0)), "ranks": world, "worst_rel_l2": all_max(rel),
                              "worst_max_abs_scaled": all_max(mabs)}
        del ps
        torch.cuda.empty_cache()

    failed = (check is not None and check["ranks_ok"] != world) or \
             (split is not None and "check" in split and split["check"]["ranks_ok"] != world)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        if failed:
            sys.exit(1)
        return

    peaks = measured_peaks()
    # executed MMA flops per unit B*H*N^2*D.  D<=64: fwd 12 (S 4 + two P V 8); single-pass backward 20; two-kernel form
    # dK/dV 16 + dQ 12 (S and dP recomputed).  D=128: fwd 12 (one CTA per branch, clusters of two), dV + dK kernels 24, dQ kernel 16.
    unit = f_fwd / 8.0
    fwd_name = "diffattn_fwd128_branch_kernel" if d == 128 else "diffattn_fwd64_kernel"
    kernels = {fwd_name: {"ms": ms_fwd, "credited_flops": f_fwd, "executed_mma_flops": unit * 12.0}}
    if pr.fused:
        kernels["diffattn_bwd_pre_kernel"] = {"ms": ms_stage["preprocess"], "credited_flops": 0.0, "executed_mma_flops": 0.0}
        kernels["diffattn_bwd_fused64_kernel"] = {"ms": ms_stage["dkdv_dq_single_pass"], "credited_flops": f_bwd, "executed_mma_flops": unit * 20.0}
        kernels["diffattn_bwd_dq_finish_kernel"] = {"ms": ms_stage["dq_finish"], "credited_flops": 0.0, "executed_mma_flops": 0.0}
    else:
        ex = {"dkdv": 24.0, "dq": 16.0} if d == 128 else {"dkdv": 16.0, "dq": 12.0}
        dkdv_name = "diffattn_bwd_dv128_kernel + diffattn_bwd_side128_kernel<K side>" if d == 128 else "diffattn_bwd_dkdv64_kernel"
        dq_name = "diffattn_bwd_side128_kernel<Q side>" if d == 128 else "diffattn_bwd_dq64_kernel"
        kernels["diffattn_bwd_pre_kernel"] = {"ms": ms_stage["preprocess"], "credited_flops": 0.0, "executed_mma_flops": 0.0}
        kernels[dkdv_name] = {"ms": ms_stage["dkdv"], "credited_flops": f_bwd * 16 / 20, "executed_mma_flops": unit * ex["dkdv"]}
        kernels[dq_name] = {"ms": ms_stage["dq"], "credited_flops": f_bwd * 4 / 20, "executed_mma_flops": unit * ex["dq"]}
    for kinfo in kernels.values():
        kinfo["credited_tflops"] = kinfo["credited_flops"] / (kinfo["ms"] * 1e-3) / 1e12
        kinfo["executed_tflops"] = kinfo["executed_mma_flops"] / (kinfo["ms"] * 1e-3) / 1e12
    dom = max(kernels, key=lambda k: kernels[k]["ms"])
    achieved = kernels[dom]["credited_tflops"]
    plain = (args.workload == NCU_TRAFFIC["workload"] and not args.causal and not args.dropout and args.io_dtype == "fp16"
             and not args.single_pass)
    traffic = NCU_TRAFFIC["bytes"].get(dom) if plain else None
    roofline = {
        "bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["burst"], "unit": "TFLOP/s",
        "frac": achieved / peaks["burst"], "peak_kind": f"cuBLAS bf16 burst, {peaks['source']} (kernel timed alone)",
        "executed_tflops": kernels[dom]["executed_tflops"], "executed_frac": kernels[dom]["executed_tflops"] / peaks["burst"],
        "traffic": traffic, "traffic_source": NCU_TRAFFIC["source"] if traffic is not None else None,
        "whole_step": {"achieved": value / world, "frac_of_measured_sustained": value / world / peaks["sustained"],
                       "frac_of_nominal_2250": value / world / NOMINAL_TFLOPS},
    }
    ours_per_step = 1 + len(pr.stage_list) + (1 if d == 128 else 0)       # forward + backward kernels (D=128: dV, dK side, dQ side)
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.io_dtype,
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: B={b} H={h} N={n} D={d} (v width {2 * d}) per GPU, rms_norm={rms}, "
                               f"lambda={lam}, lambda_init={lam_init}, fwd+bwd" + (", causal" if args.causal else "")
                               + (f", dropout {int(round(args.dropout * 256))}/256" if args.dropout else "")
                               + (", single-pass backward" if args.single_pass else ""),
                   "sharding": f"(batch*head) shards, {world} rank(s), no data-path collective; d(lambda) summed on host",
                   "l2": "inputs+outputs per step (~0.8 GB) exceed the 126 MB L2; no explicit flush"},
        "fwd": {"ms": ms_fwd, "tflops": f_fwd / (ms_fwd * 1e-3) / 1e12, "frac_nominal": f_fwd / (ms_fwd * 1e-3) / 1e12 / NOMINAL_TFLOPS},
        "bwd": {"ms": ms_bwd, "tflops": f_bwd / (ms_bwd * 1e-3) / 1e12, "frac_nominal": f_bwd / (ms_bwd * 1e-3) / 1e12 / NOMINAL_TFLOPS},
        "fwd_bwd_frac_nominal": value / world / NOMINAL_TFLOPS,
        "kernels": kernels, "roofline": roofline, "clocks": clocks,
        "gpu_launches": ours_per_step * args.steps,
        "gpu_launches_note": f"{ours_per_step} kernels of this library per step (forward, " + ", ".join(nm for nm, _ in pr.stage_list)
                             + "); torch's one-element fill that zeroes d(lambda) is not counted",
        "dlambda_host_sum": dl_total,
    }
    if sustained:
        line["sustained"] = sustained
    if check:
        line["check"] = check
    if split:
        line["config5"] = split
    if e2e:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"], _ = cpu_baseline_block(args.workload, 3, 1)
    emit(line)
    if world > 1:
        dist.destroy_process_group()
    if failed:
        sys.exit(1)


if __name__ == "__main__":
    main()
