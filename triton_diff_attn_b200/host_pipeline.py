"""Forward + backward on HOST-resident tensors, with the copies overlapped with the kernels.

A caller whose q/k/v and upstream gradient live in (pinned) host memory pays two PCIe transfers per
step that together take longer than the kernels.  `HostStepPipeline` runs the three phases of
consecutive steps on three CUDA streams -- host->device copies, the operator's forward and backward
(`diffattn_fwd` / `diffattn_bwd` of the C ABI), device->host copies of y and the six gradients -- so that
in steady state a step costs max(copy in, kernels, copy out) instead of their sum.
Every device buffer (staged inputs, outputs, saved statistics, gradients, workspace) is allocated once per
ring slot and reused: in steady state a step makes no allocator call at all (an allocation that has to go
to cudaMalloc synchronises the device and would serialise the three streams).
The reference has no such path (its benchmark keeps everything on the device, src/benchmark.py:115-131).
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

import torch

from . import _lib
from .layers import _check_inputs, _fill_common


class _Slot:
    """Device buffers and the filled parameter block of one ring slot."""

    def __init__(self, host_in, lambda_scale, lambda_init, rms_norm, causal, device, stream):
        q1, q2, k1, k2, v, dy = host_in
        mk = lambda t: torch.empty(t.shape, dtype=t.dtype, device=device)
        self.inputs = [mk(t) for t in host_in]
        dq1, dq2, dk1, dk2, dv_, ddy = self.inputs
        b, h, n, d = q1.shape
        self.y, self.a2 = mk(v), mk(v)
        self.lse1 = torch.empty((b, h, n), dtype=torch.float32, device=device)
        self.lse2, self.rstd = torch.empty_like(self.lse1), torch.empty_like(self.lse1)
        self.grads = [mk(q1), mk(q1), mk(q1), mk(q1), mk(v)]
        self.dlam = torch.zeros(1, dtype=torch.float32, device=device)
        self.lam = lambda_scale.detach().to(device).clone()
        _check_inputs(dq1, dq2, dk1, dk2, dv_, self.lam)
        p = _lib.new_params()
        with torch.cuda.stream(stream):          # the parameter block records the stream the kernels are enqueued on
            _fill_common(p, dq1, dq2, dk1, dk2, dv_, self.lam, lambda_init, rms_norm,
                         (self.y, self.a2, self.lse1, self.lse2, self.rstd), causal)
        nbytes = int(_lib.lib.diffattn_workspace_bytes(p))
        self.ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        p.dy = ddy.data_ptr()
        p.dq1, p.dq2, p.dk1, p.dk2, p.dv = (t.data_ptr() for t in self.grads)
        p.dlambda = self.dlam.data_ptr()
        p.workspace, p.workspace_bytes = self.ws.data_ptr(), nbytes
        self.p = p
        self.key = (tuple(q1.shape), q1.dtype, float(lambda_init), bool(rms_norm), bool(causal))
        self.outputs = [self.y] + self.grads + [self.dlam]


class HostStepPipeline:
    def __init__(self, device: torch.device, depth: int = 2):
        self.device = device
        self.depth = depth
        self.s_in = torch.cuda.Stream(device)
        self.s_run = torch.cuda.Stream(device)
        self.s_out = torch.cuda.Stream(device)
        self.slots: List[_Slot] = []
        self.in_done = [torch.cuda.Event() for _ in range(depth)]
        self.run_done = [torch.cuda.Event() for _ in range(depth)]
        self.out_done = [torch.cuda.Event() for _ in range(depth)]
        self.count = 0

    def begin(self) -> None:
        """Order the pipeline's streams after everything already queued on the current stream."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)

    def submit(self, host_in: Sequence[torch.Tensor], host_out: Sequence[torch.Tensor], host_dlambda: torch.Tensor,
               lambda_scale: torch.Tensor, lambda_init: float, rms_norm: bool, causal: bool = False) -> None:
        """host_in = (q1, q2, k1, k2, v, dy) pinned; host_out = (y, dq1, dq2, dk1, dk2, dv) pinned; host_dlambda: one
        pinned fp32 element that receives d(lambda)."""
        slot_i = self.count % self.depth
        key = (tuple(host_in[0].shape), host_in[0].dtype, float(lambda_init), bool(rms_norm), bool(causal))
        if len(self.slots) <= slot_i:
            self.slots.append(_Slot(host_in, lambda_scale, lambda_init, rms_norm, causal, self.device, self.s_run))
        elif self.slots[slot_i].key != key:
            torch.cuda.synchronize(self.device)          # shapes changed: nothing of the old slot may be in flight
            self.slots[slot_i] = _Slot(host_in, lambda_scale, lambda_init, rms_norm, causal, self.device, self.s_run)
        slot = self.slots[slot_i]
        reuse = self.count >= self.depth
        with torch.cuda.stream(self.s_in):
            if reuse:
                self.s_in.wait_event(self.run_done[slot_i])      # the kernels of step count-depth have read this slot's inputs
            for dst, src in zip(slot.inputs, host_in):
                dst.copy_(src, non_blocking=True)
            slot.lam.copy_(lambda_scale.detach().reshape(slot.lam.shape), non_blocking=True)
            self.in_done[slot_i].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.in_done[slot_i])
            if reuse:
                self.s_run.wait_event(self.out_done[slot_i])     # the copies of step count-depth have read this slot's outputs
            slot.dlam.zero_()
            _lib.check(_lib.lib.diffattn_fwd(ctypes.byref(slot.p)), "diffattn_fwd")
            _lib.check(_lib.lib.diffattn_bwd(ctypes.byref(slot.p)), "diffattn_bwd")
            self.run_done[slot_i].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.run_done[slot_i])
            for dst, src in zip(list(host_out) + [host_dlambda], slot.outputs):
                dst.copy_(src.reshape(dst.shape), non_blocking=True)
            self.out_done[slot_i].record(self.s_out)
        self.count += 1

    def end(self) -> None:
        """Make the current stream wait for everything the pipeline has queued."""
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)
