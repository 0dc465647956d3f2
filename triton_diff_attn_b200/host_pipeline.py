"""Forward + backward on HOST-resident tensors, with the copies overlapped with the kernels.

A caller whose q/k/v and upstream gradient live in (pinned) host memory pays two PCIe transfers per
step that together take longer than the kernels.  `HostStepPipeline` runs the three phases of
consecutive steps on three CUDA streams -- host->device copies, the operator (`MultiheadDiffAttnKernel`
forward and backward), device->host copies of y and the six gradients -- with double-buffered device
staging, so that in steady state a step costs max(copy in, kernels, copy out) instead of their sum.
The reference has no such path (its benchmark keeps everything on the device, src/benchmark.py:115-131).
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .layers import MultiheadDiffAttnKernel


class HostStepPipeline:
    def __init__(self, device: torch.device, depth: int = 2):
        self.device = device
        self.depth = depth
        self.s_in = torch.cuda.Stream(device)
        self.s_run = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self.staging: List[List[torch.Tensor]] = []
        self.run_done = [torch.cuda.Event() for _ in range(depth)]
        self.in_done = [torch.cuda.Event() for _ in range(depth)]
        self.count = 0

    def begin(self) -> None:
        """Order the pipeline's streams after everything already queued on the current stream."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)

    def submit(self, host_in: Sequence[torch.Tensor], host_out: Sequence[torch.Tensor], host_dlambda: torch.Tensor,
               lambda_scale: torch.Tensor, lambda_init: float, rms_norm: bool, causal: bool = False) -> None:
        """host_in = (q1, q2, k1, k2, v, dy) pinned; host_out = (y, dq1, dq2, dk1, dk2, dv) pinned."""
        slot = self.count % self.depth
        if len(self.staging) <= slot:
            self.staging.append([torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_in])
        bufs = self.staging[slot]
        with torch.cuda.stream(self.s_in):
            if self.count >= self.depth:
                self.s_in.wait_event(self.run_done[slot])      # the kernels of step count-depth have read this slot
            for dst, src in zip(bufs, host_in):
                dst.copy_(src, non_blocking=True)
            self.in_done[slot].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.in_done[slot])
            leaves = [b.detach().requires_grad_(True) for b in bufs[:5]]
            lam = lambda_scale.detach().clone().requires_grad_(True)
            y = MultiheadDiffAttnKernel(*leaves, lam, lambda_init, rms_norm, causal)
            y.backward(bufs[5])
            self.run_done[slot].record(self.s_run)
            results = [y.detach()] + [t.grad for t in leaves] + [lam.grad]
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.run_done[slot])
            for dst, src in zip(list(host_out) + [host_dlambda], results):
                src.record_stream(self.s_out)
                dst.copy_(src.reshape(dst.shape) if src.numel() == dst.numel() else src, non_blocking=True)
        self.count += 1

    def end(self) -> None:
        """Make the current stream wait for everything the pipeline has queued."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)
