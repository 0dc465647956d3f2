#!/usr/bin/env python
"""Benchmark of the differential-attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c3|c4|c5shard|ref_d32]

A step is one forward + backward over one batch of synthetic fp16 input.  At N=1 the workload is
BASELINE config 2 (B=4, H=16, N=4096, D=64).  With N>1 every rank runs the same shape on its own
(batch*head) shard (weak scaling, no data-path collective); the d(lambda) partials are summed on
the host.  `value` is credited TFLOP/s (fwd 8 N^2 D + bwd 20 N^2 D per head) over all ranks with inputs
resident in HBM, timed with CUDA events, max over ranks.  `e2e` is the same metric through the Python
operator with HOST (pinned) inputs and outputs, copies inside the timed region.
`--impl reference` times the CPU restatement of the reference's PyTorch path (oracle/) on the host
cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
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
    "c2": (4, 16, 4096, 64, 1.0, 0.5, 0.8, True),        # BASELINE config 2 (headline)
    "c3": (1, 32, 16384, 64, 0.5, 0.3, 0.8, True),       # BASELINE config 3
    "c4": (8, 8, 8192, 128, 1.0, 0.7, 0.2, False),       # BASELINE config 4 (wide head, RMSNorm off)
    "c5shard": (8, 32, 4096, 64, 1.0, 0.5, 0.8, True),   # BASELINE config 5 split over 8 GPUs
    "ref_d32": (4, 16, 4096, 32, 0.5, 0.5, 0.8, True),   # the reference's benchmark point H=16 D=32 N=4096 (src/benchmark.py:19-25)
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised in
# profiles/c2_kernels_ncu_full.md (workload c2); other workloads report null.
NCU_TRAFFIC_BYTES = {"c2": {"diffattn_fwd64_kernel": 309.9e6, "diffattn_bwd_pre_kernel": 257.1e6,
                            "diffattn_bwd_dkdv64_kernel": 383.2e6, "diffattn_bwd_dq64_kernel": 326.0e6}}
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


def cpu_sample(workload, heads, steps, warmup, threads=None):
    """Times the oracle's forward + autograd backward (CPU fp32) on `heads` heads of the workload."""
    from oracle import diffattn_oracle as oracle
    b, h, n, d, scale, lam, lam_init, rms = WORKLOADS[workload]
    # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1 to every rank)
    torch.set_num_threads(threads or os.cpu_count() or 1)
    q1, q2, k1, k2, v, dy = oracle.make_inputs(1, heads, n, d, seed=4321, scale=scale)
    lam_t = torch.tensor([lam])
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.forward_backward_autograd(q1, q2, k1, k2, v, lam_t, dy, lam_init, rms)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    f, bk = flops(1, heads, n, d)
    total = sum(times)
    return {"tflops": (f + bk) * len(times) / total / 1e12, "ms_per_step": 1e3 * total / len(times),
            "cores": torch.get_num_threads(),
            "sample": f"{heads} of {b * h} heads of {workload} (B=1,H={heads},N={n},D={d}), fp32 forward + autograd backward, "
                      f"{len(times)} timed passes after {warmup} warm-up"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    b, h, n, d, *_ = WORKLOADS[args.workload]
    r = cpu_sample(args.workload, heads=2, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["tflops"], "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: B={b} H={h} N={n} D={d} (v width {2 * d}), rms_norm, fwd+bwd",
                   "note": "CPU restatement of the reference's MultiheadDiffAttn (PyTorch ops, fp32); the reference "
                           "checkout itself does not travel to the GPU box"},
        "cpu_baseline": {"value": r["tflops"], "unit": "TFLOP/s", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": r["tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


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
    """Informational same-box LIBRARY baseline, not the product and not the reference arm: differential
    attention composed from four FlashAttention-2 calls (each branch against the two halves of V), the
    construction the reference compares its kernel with (reference src/layers.py:104-148), written here
    against the flash_attn package of this image, RMSNorm in plain torch ops.  One GPU only."""
    import math
    from flash_attn import flash_attn_func
    b, h, n, d, scale, lam, lam_init, rms = WORKLOADS[args.workload]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1234)
    def draw(*shape):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale).to(torch.float16).requires_grad_(True)
    # flash_attn wants [B, N, H, D]
    q1, q2, k1, k2 = (draw(b, n, h, d) for _ in range(4))
    v = draw(b, n, h, 2 * d)
    dy = torch.randn(b, n, h, 2 * d, generator=g, device=dev, dtype=torch.float32).to(torch.float16)
    lam_t = torch.tensor([lam], dtype=torch.float16, device=dev, requires_grad=True)

    def step():
        v1, v2 = v[..., :d], v[..., d:]
        a1 = torch.cat([flash_attn_func(q1, k1, v1), flash_attn_func(q1, k1, v2)], dim=-1)
        a2 = torch.cat([flash_attn_func(q2, k2, v1), flash_attn_func(q2, k2, v2)], dim=-1)
        a = a1 - lam_t * a2
        if rms:
            a = (1.0 - lam_init) * a * torch.rsqrt((a.float() ** 2).mean(-1, keepdim=True) + 1e-5).to(a.dtype)
        a.backward(dy)
        for t in (q1, q2, k1, k2, v, lam_t):
            t.grad = None

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    f, bk = flops(b, h, n, d)
    emit({"impl": "flash_composition", "metric": METRIC, "value": (f + bk) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                      "dtype": "fp16", "data": "synthetic",
                      "config": {"workload": args.workload, "note": "library baseline: 4x flash_attn_func + torch ops; credited "
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


def main():
    _quiet_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "flash_composition"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--io-dtype", default="fp16", choices=["fp16", "bf16"],
                    help="16-bit type of the tensors: fp16 (the reference's and the headline) or bf16 (extension)")
    ap.add_argument("--dropout", type=float, default=0.0, help="attention dropout probability (extension); flops are "
                    "credited as without dropout")
    ap.add_argument("--causal", action="store_true", help="causal mask (extension); flops credited for the visible "
                    "N(N+1)/2 pairs only")
    ap.add_argument("--sweep-reference-protocol", action="store_true",
                    help="instead of the one-line benchmark: the reference's own sweep (src/benchmark.py:19-25): "
                         "H=16, D=32, fp16, rms_norm, N in 512..16384 with B = 16384/N; one JSON line per N")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference(args)
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
    import torch.distributed as dist
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ["NCCL_DEBUG"] = "WARN"      # keep NCCL's version banner off stdout: rank 0 prints ONE JSON line
        dist.init_process_group("nccl", device_id=dev)

    from triton_diff_attn_b200 import _lib, layers, MultiheadDiffAttnKernel, sum_dlambda_on_host, device_status

    b, h, n, d, scale, lam, lam_init, rms = WORKLOADS[args.workload]
    g = torch.Generator(device=dev).manual_seed(1234 + rank)

    io_dtype = torch.bfloat16 if args.io_dtype == "bf16" else torch.float16

    def draw(*shape):
        return (torch.randn(*shape, generator=g, device=dev, dtype=torch.float32) * scale).to(io_dtype)

    q1, q2, k1, k2 = (draw(b, h, n, d) for _ in range(4))
    v = draw(b, h, n, 2 * d)
    dy = torch.randn(b, h, n, 2 * d, generator=g, device=dev, dtype=torch.float32).to(io_dtype)
    lam_t = torch.tensor([lam], dtype=torch.float32, device=dev)

    y = torch.empty_like(v); a2 = torch.empty_like(v)
    lse1 = torch.empty(b, h, n, dtype=torch.float32, device=dev); lse2 = torch.empty_like(lse1); rstd = torch.empty_like(lse1)
    dq1, dq2, dk1, dk2 = (torch.empty_like(q1) for _ in range(4))
    dv = torch.empty_like(v)
    dlam = torch.zeros(1, dtype=torch.float32, device=dev)
    p = _lib.new_params()
    layers._fill_common(p, q1, q2, k1, k2, v, lam_t, lam_init, rms, (y, a2, lse1, lse2, rstd), args.causal,
                        layers.dropout_threshold(args.dropout), 20241125)
    ws_bytes = int(_lib.lib.diffattn_workspace_bytes(p))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    p.dy = dy.data_ptr()
    p.dq1, p.dq2, p.dk1, p.dk2, p.dv = (t.data_ptr() for t in (dq1, dq2, dk1, dk2, dv))
    p.dlambda = dlam.data_ptr()
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws_bytes
    pref = ctypes.byref(p)

    def fwd():
        _lib.check(_lib.lib.diffattn_fwd(pref), "diffattn_fwd")

    def bwd(stages=_lib.STAGE_ALL):
        _lib.check(_lib.lib.diffattn_bwd_stages(pref, stages), "diffattn_bwd")

    def step():
        fwd()
        dlam.zero_()
        bwd()

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

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        step()
    device_status(local_rank)
    ms_step = timed(step, args.steps)
    # per-kernel durations (each kernel alone, same resident inputs); L2 is smaller than the inputs
    ms_fwd = timed(fwd, args.steps)
    ms_pre = timed(lambda: bwd(_lib.STAGE_PRE), args.steps)
    ms_dkdv = timed(lambda: bwd(_lib.STAGE_DKDV), args.steps)
    ms_dq = timed(lambda: bwd(_lib.STAGE_DQ), args.steps)
    ms_bwd = timed(bwd, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    device_status(local_rank)
    dlam.zero_(); bwd()
    dl_total = sum_dlambda_on_host(dlam)

    f_fwd, f_bwd = flops(b, h, n, d)
    if args.causal:
        f_fwd, f_bwd = f_fwd * (n + 1) / (2.0 * n), f_bwd * (n + 1) / (2.0 * n)
    total_flops = (f_fwd + f_bwd) * world
    value = total_flops / (ms_step * 1e-3) / 1e12

    # ---- end to end through the Python operator with host buffers
    e2e = None
    if not args.no_e2e:
        host_in = [t.cpu().pin_memory() for t in (q1, q2, k1, k2, v, dy)]
        host_out = [torch.empty_like(t, device="cpu").pin_memory() for t in (y, dq1, dq2, dk1, dk2, dv)]
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
                pipe.submit(host_in, host_out, host_dl, lam_t, lam_init, rms, args.causal)
            pipe.end()

        e2e_run(3)
        ms_e2e = timed(lambda: e2e_run(args.steps), 1) / args.steps
        e2e = {"value": total_flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "how": "HostStepPipeline: H2D, kernels and D2H of consecutive steps on three streams, double-buffered staging"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = measured_peaks()
    # executed MMA flops per unit B*H*N^2*D: D<=64: fwd 12 (S 4 + two P V 8), dK/dV 16, dQ 12 (S and dP recomputed);
    # D=128: fwd 16 (S in both value-column passes), dV + dK kernels 24, dQ kernel 16
    unit = f_fwd / 8.0
    ex = {"fwd": 16.0, "dkdv": 24.0, "dq": 16.0} if d == 128 else {"fwd": 12.0, "dkdv": 16.0, "dq": 12.0}
    tag = "128" if d == 128 else "64"
    dkdv_name = "diffattn_bwd_dv128_kernel + diffattn_bwd_side128_kernel<K side>" if d == 128 else "diffattn_bwd_dkdv64_kernel"
    dq_name = "diffattn_bwd_side128_kernel<Q side>" if d == 128 else "diffattn_bwd_dq64_kernel"
    kernels = {
        f"diffattn_fwd{tag}_kernel": {"ms": ms_fwd, "credited_flops": f_fwd, "executed_mma_flops": unit * ex["fwd"]},
        "diffattn_bwd_pre_kernel": {"ms": ms_pre, "credited_flops": 0.0, "executed_mma_flops": 0.0},
        dkdv_name: {"ms": ms_dkdv, "credited_flops": f_bwd * 16 / 20, "executed_mma_flops": unit * ex["dkdv"]},
        dq_name: {"ms": ms_dq, "credited_flops": f_bwd * 4 / 20, "executed_mma_flops": unit * ex["dq"]},
    }
    for kinfo in kernels.values():
        kinfo["credited_tflops"] = kinfo["credited_flops"] / (kinfo["ms"] * 1e-3) / 1e12
        kinfo["executed_tflops"] = kinfo["executed_mma_flops"] / (kinfo["ms"] * 1e-3) / 1e12
    dom = max(kernels, key=lambda k: kernels[k]["ms"])
    achieved = kernels[dom]["credited_tflops"]
    roofline = {
        "bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peaks["burst"], "unit": "TFLOP/s",
        "frac": achieved / peaks["burst"], "peak_kind": f"cuBLAS bf16 burst, {peaks['source']} (kernel timed alone)",
        "executed_tflops": kernels[dom]["executed_tflops"], "executed_frac": kernels[dom]["executed_tflops"] / peaks["burst"],
        "traffic": NCU_TRAFFIC_BYTES.get(args.workload, {}).get(dom),
        "whole_step": {"achieved": value / world, "frac_of_measured_sustained": value / world / peaks["sustained"],
                       "frac_of_nominal_2250": value / world / NOMINAL_TFLOPS},
    }
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.io_dtype,
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: B={b} H={h} N={n} D={d} (v width {2 * d}) per GPU, rms_norm={rms}, "
                               f"lambda={lam}, lambda_init={lam_init}, fwd+bwd" + (", causal" if args.causal else "")
                               + (f", dropout {layers.dropout_threshold(args.dropout)}/256" if args.dropout else ""),
                   "sharding": f"(batch*head) shards, {world} rank(s), no data-path collective; d(lambda) summed on host",
                   "l2": "inputs+outputs per step (~0.8 GB) exceed the 126 MB L2; no explicit flush"},
        "fwd": {"ms": ms_fwd, "tflops": f_fwd / (ms_fwd * 1e-3) / 1e12, "frac_nominal": f_fwd / (ms_fwd * 1e-3) / 1e12 / NOMINAL_TFLOPS},
        "bwd": {"ms": ms_bwd, "tflops": f_bwd / (ms_bwd * 1e-3) / 1e12, "frac_nominal": f_bwd / (ms_bwd * 1e-3) / 1e12 / NOMINAL_TFLOPS},
        "fwd_bwd_frac_nominal": value / world / NOMINAL_TFLOPS,
        "kernels": kernels, "roofline": roofline, "clocks": clocks, "gpu_launches": (5 if d == 128 else 4) * args.steps,   # fwd, pre, then dK/dV + dQ (D<=64) or dV + dK + dQ (D=128)
        "dlambda_host_sum": dl_total,
    }
    if e2e:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        c = cpu_sample(args.workload, heads=2, steps=3, warmup=1)
        line["cpu_baseline"] = {"value": c["tflops"], "unit": "TFLOP/s", "cores": c["cores"], "kind": "port",
                                "sample": c["sample"], "ms_per_sample": c["ms_per_step"]}
    emit(line)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
