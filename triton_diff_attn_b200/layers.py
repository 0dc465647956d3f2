"""Drop-in for the reference's `MultiheadDiffAttnKernel` (reference src/layers.py:10-26) and its
autograd function `_diff_attention` (reference src/kernel.py:461-575).

Host side only: argument checks, output allocation through torch, and two calls into the C ABI
(`diffattn_fwd`, `diffattn_bwd`).  All arithmetic runs in the hand-written sm_100a kernels of
libdiffattn.so.  Differences from the reference's host code, on purpose:
  * no host synchronisation in the backward (the reference calls `.item()`, src/kernel.py:573):
    d(lambda) is accumulated on the device and returned as a tensor of lambda_scale's shape/dtype;
  * the backward keeps logsumexp per branch, rstd and A2 = P2 V instead of O1 and O2
    (src/kernel.py:505);
  * no global autotune state (src/kernel.py:511-512).
"""
from __future__ import annotations

import math

import torch

from . import _lib

EPS = 1e-5   # reference src/kernel.py:50


def _check_inputs(q1, q2, k1, k2, v, lambda_scale):
    if not torch.is_tensor(lambda_scale):
        raise TypeError("lambda_scale must be a 1-element CUDA tensor (the reference loads it from a "
                        "device pointer, src/kernel.py:138)")
    for name, t in (("q1", q1), ("q2", q2), ("k1", k1), ("k2", k2), ("v", v)):
        if not torch.is_tensor(t):
            raise TypeError(f"{name} must be a tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor: this operator has no CPU path")
        if t.dtype not in (torch.float16, torch.bfloat16):
            raise ValueError(f"{name} must be float16 (the reference's type: it computes P in fp16, "
                             f"src/kernel.py:175-176) or bfloat16 (extension), got {t.dtype}")
        if t.dtype != q1.dtype:
            raise ValueError(f"{name} is {t.dtype} but q1 is {q1.dtype}: q1, q2, k1, k2 and v must share one dtype")
        if t.dim() != 4:
            raise ValueError(f"{name} must be [B, H, N, D]")
    if lambda_scale.numel() != 1 or lambda_scale.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise ValueError("lambda_scale must hold one float16, bfloat16 or float32 element")
    if lambda_scale.device != q1.device:
        raise RuntimeError("lambda_scale must live on the same device as q1")
    b, h, n, d = q1.shape
    for name, t in (("q2", q2), ("k1", k1), ("k2", k2)):
        if tuple(t.shape) != (b, h, n, d):
            raise ValueError(f"{name} shape {tuple(t.shape)} != q1 shape {(b, h, n, d)}")
        if t.device != q1.device:
            raise RuntimeError(f"{name} is on {t.device}, q1 on {q1.device}")
    if tuple(v.shape) != (b, h, n, 2 * d):
        raise ValueError(f"v shape {tuple(v.shape)} != {(b, h, n, 2 * d)}")
    if v.device != q1.device:
        raise RuntimeError("v is on another device")


def _tma_ready(t):
    """A tensor the TMA descriptors can address as it lies: unit stride in the last dimension, every other
    stride a positive multiple of 8 elements (16 bytes), base pointer 16-byte aligned.  Anything else the
    reference's pointer arithmetic would accept (expanded tensors with stride 0, odd slices of a packed
    buffer) is copied into a dense tensor first."""
    if t.data_ptr() % 16 != 0:
        return t.clone(memory_format=torch.contiguous_format)      # a fresh allocation is aligned
    if t.stride(-1) != 1 or any(stride <= 0 or stride % 8 != 0 for stride in t.stride()[:-1]):
        return t.contiguous()
    return t


def _same_layout(ts):
    """q1,q2,k1,k2 must share strides (the reference reads them from Q1 only, src/kernel.py:487-490)."""
    ts = [_tma_ready(t) for t in ts]
    if any(t.stride() != ts[0].stride() for t in ts):
        ts = [t.contiguous() for t in ts]
    return ts


def dropout_threshold(dropout_p: float) -> int:
    """The kernels drop a probability when a hash byte is below round(256 p): p is quantised to 1/256 steps
    (0 below 1/512) and must stay below 255.5/256."""
    if not 0.0 <= float(dropout_p) < 1.0:
        raise ValueError(f"dropout_p must be in [0, 1), got {dropout_p}")
    t = int(round(float(dropout_p) * 256.0))
    if t > 255:
        raise ValueError(f"dropout_p {dropout_p} is too close to 1 (largest supported: 255/256)")
    return t


def _fill_common(p, q1, q2, k1, k2, v, lam, lambda_init, rms_norm, saved, causal=False, drop_threshold=0, drop_seed=0,
                 gain=None, y_gained=None, single_pass=False):
    b, h, n, d = q1.shape
    p.device = q1.device.index if q1.device.index is not None else torch.cuda.current_device()
    p.stream = torch.cuda.current_stream(q1.device).cuda_stream
    p.B, p.H, p.N, p.D = b, h, n, d
    p.qk_stride_b, p.qk_stride_h, p.qk_stride_n = q1.stride(0), q1.stride(1), q1.stride(2)
    p.v_stride_b, p.v_stride_h, p.v_stride_n = v.stride(0), v.stride(1), v.stride(2)
    p.q1, p.q2, p.k1, p.k2, p.v = (t.data_ptr() for t in (q1, q2, k1, k2, v))
    p.lambda_scale = lam.data_ptr()
    p.lambda_dtype = {torch.float16: _lib.LAMBDA_F16, torch.bfloat16: _lib.LAMBDA_BF16}.get(lam.dtype, _lib.LAMBDA_F32)
    p.io_dtype = _lib.IO_BF16 if q1.dtype == torch.bfloat16 else _lib.IO_F16
    p.rms_norm = 1 if rms_norm else 0
    p.causal = 1 if causal else 0
    p.dropout_threshold = int(drop_threshold)
    p.dropout_seed = int(drop_seed) & 0xFFFFFFFFFFFFFFFF
    p.single_pass = 1 if single_pass else 0
    if gain is not None:
        p.gain, p.y_gained = gain.data_ptr(), y_gained.data_ptr()
    p.sm_scale = 1.0 / math.sqrt(d)          # reference src/layers.py:20-22 (D, not 2D)
    p.lambda_init = float(lambda_init)
    p.eps = EPS
    y, a2, lse1, lse2, rstd = saved
    p.y, p.a2, p.lse1, p.lse2, p.rstd = (t.data_ptr() for t in (y, a2, lse1, lse2, rstd))


class DiffAttnFunction(torch.autograd.Function):
    """forward/backward pair bound to the C ABI; counterpart of `_diff_attention`
    (reference src/kernel.py:461-575)."""

    @staticmethod
    def forward(ctx, q1, q2, k1, k2, v, lambda_scale, lambda_init, rms_norm, causal=False, drop_threshold=0, drop_seed=0,
                gain=None, single_pass=False):
        _check_inputs(q1, q2, k1, k2, v, lambda_scale)
        if gain is not None:
            if not torch.is_tensor(gain) or gain.device != q1.device or tuple(gain.shape) != (v.shape[-1],):
                raise ValueError("gain must be a tensor of shape [2*D] on the inputs' device")
        q1, q2, k1, k2 = _same_layout([q1, q2, k1, k2])
        v = _tma_ready(v)
        b, h, n, d = q1.shape
        dev = q1.device
        with torch.cuda.device(dev):
            y = torch.empty((b, h, n, 2 * d), dtype=v.dtype, device=dev)
            a2 = torch.empty_like(y)
            lse1 = torch.empty((b, h, n), dtype=torch.float32, device=dev)
            lse2 = torch.empty_like(lse1)
            rstd = torch.empty_like(lse1)
            gain32 = gain.detach().to(torch.float32).contiguous() if gain is not None else None
            y_gained = torch.empty_like(y) if gain is not None else None
            p = _lib.new_params()
            _fill_common(p, q1, q2, k1, k2, v, lambda_scale, lambda_init, rms_norm, (y, a2, lse1, lse2, rstd), causal,
                         drop_threshold, drop_seed, gain32, y_gained)
            _lib.check(_lib.lib.diffattn_fwd(p), "diffattn_fwd")
        ctx.save_for_backward(q1, q2, k1, k2, v, lambda_scale, y, a2, lse1, lse2, rstd)
        ctx.gain32 = gain32
        ctx.gain_dtype = gain.dtype if gain is not None else None
        ctx.lambda_init = float(lambda_init)
        ctx.rms_norm = bool(rms_norm)
        ctx.causal = bool(causal)
        ctx.drop = (int(drop_threshold), int(drop_seed))
        ctx.single_pass = bool(single_pass)
        return y_gained if gain is not None else y

    @staticmethod
    def backward(ctx, dy):
        q1, q2, k1, k2, v, lam, y, a2, lse1, lse2, rstd = ctx.saved_tensors
        b, h, n, d = q1.shape
        dev = q1.device
        dy = dy.to(v.dtype).contiguous()   # the kernels index dY densely (as src/kernel.py:278-280)
        with torch.cuda.device(dev):
            dq1 = torch.empty((b, h, n, d), dtype=q1.dtype, device=dev)
            dq2, dk1, dk2 = torch.empty_like(dq1), torch.empty_like(dq1), torch.empty_like(dq1)
            dv = torch.empty((b, h, n, 2 * d), dtype=v.dtype, device=dev)
            dlam = torch.zeros(1, dtype=torch.float32, device=dev)
            p = _lib.new_params()
            dgain = torch.zeros(2 * d, dtype=torch.float32, device=dev) if ctx.gain32 is not None else None
            _fill_common(p, q1, q2, k1, k2, v, lam, ctx.lambda_init, ctx.rms_norm, (y, a2, lse1, lse2, rstd), ctx.causal,
                         *ctx.drop, ctx.gain32, y, ctx.single_pass)     # y_gained is not read by the backward
            if dgain is not None:
                p.dgain = dgain.data_ptr()
            nbytes = int(_lib.lib.diffattn_workspace_bytes(p))
            ws = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=dev)
            p.dy = dy.data_ptr()
            p.dq1, p.dq2, p.dk1, p.dk2, p.dv = (t.data_ptr() for t in (dq1, dq2, dk1, dk2, dv))
            p.dlambda = dlam.data_ptr()
            p.workspace, p.workspace_bytes = ws.data_ptr(), nbytes
            _lib.check(_lib.lib.diffattn_bwd(p), "diffattn_bwd")
        # fp32 partial kept for callers that shard (batch*head) and sum partials themselves
        DiffAttnFunction.last_dlambda_fp32 = dlam
        dlam_out = dlam.to(lam.dtype).reshape(lam.shape) if ctx.needs_input_grad[5] else None
        dgain_out = dgain.to(ctx.gain_dtype) if (dgain is not None and ctx.needs_input_grad[11]) else None
        return dq1, dq2, dk1, dk2, dv, dlam_out, None, None, None, None, None, dgain_out, None

    last_dlambda_fp32 = None


def MultiheadDiffAttnKernel(q1, q2, k1, k2, v, lambda_scale=-0.5, lambda_init: float = 0.8, rms_norm: bool = False,
                            causal: bool = False, dropout_p: float = 0.0, dropout_seed=None, gain=None,
                            single_pass: bool = False):
    """Fused differential attention, same signature as the reference (src/layers.py:10-26).

    q1,q2,k1,k2: fp16 CUDA [B,H,N,D]; v: fp16 CUDA [B,H,N,2D]; lambda_scale: 1-element fp16/fp32
    CUDA tensor (the reference's float default cannot be loaded by its kernel either,
    src/layers.py:16 vs src/kernel.py:138).  Returns fp16 [B,H,N,2D].  The softmax scale is
    1/sqrt(D) (src/layers.py:20-22); (1 - lambda_init) is applied only with rms_norm
    (src/layers.py:74-78).  Any sequence length N >= 1 is accepted (key columns past N are masked in the last
    tile); the reference needs N to be a multiple of its block sizes (src/kernel.py:148,527).
    `causal=True` (keyword, after the reference's eight parameters) restricts query i to keys j <= i; the
    reference has no masking (README.md:2).
    `dropout_p` > 0 (keyword; the reference has no dropout either) drops attention probabilities after the
    softmax, independently in the two branches, and scales the kept ones by 1/(1-p); p is quantised to 1/256
    steps (`dropout_threshold`).  The mask is a pure function of `dropout_seed` and the position, so the backward
    recomputes it; without a seed one is drawn from torch's CPU generator (no device synchronisation).
    `gain` (keyword, a [2D] tensor, normally a learnable parameter): the output is multiplied column-wise by it
    inside the forward epilogue and its gradient comes out of the backward's preprocess kernel -- the weight of
    the output norm in the layer the reference adapts (src/layers.py:114), which the reference's own norm
    (elementwise_affine=False, src/layers.py:75) does not have.
    `single_pass=True` (keyword; head dims 32 and 64) selects the backward that visits every score tile once and
    sums each key block's share of dq1/dq2 with fp32 atomic adds, so those two gradients can differ in the last
    bit from run to run.  The default backward is two tensor-core kernels whose second recomputes the scores per
    query block, as the reference's second loop does (src/kernel.py:426-436); it is bit-reproducible and, on
    B200, the faster of the two.

    A device-side wait that gives up (a kernel bug or a broken GPU, never a property of the inputs) leaves the
    outputs undefined without raising here; `device_status()` synchronises and raises in that case.
    """
    thresh = dropout_threshold(dropout_p)
    seed = 0
    if thresh:
        seed = int(torch.randint(0, 2 ** 62, (1,)).item()) if dropout_seed is None else int(dropout_seed)
    return DiffAttnFunction.apply(q1, q2, k1, k2, v, lambda_scale, lambda_init, rms_norm, causal, thresh, seed, gain,
                                  single_pass)


def lambda_from_reparam(lambda_q1, lambda_k1, lambda_q2, lambda_k2, lambda_init: float):
    """lambda = exp(<lambda_q1, lambda_k1>) - exp(<lambda_q2, lambda_k2>) + lambda_init as a 1-element fp32
    tensor on the parameters' device: the re-parameterisation of the layer the reference adapts
    (src/layers.py:114; the reference itself takes lambda_scale ready-made, src/layers.py:16).  Plain device-side
    torch ops, differentiable, no host synchronisation: together with the operator's device-side d(lambda) the
    whole layer runs without a sync (the reference's backward calls .item(), src/kernel.py:573)."""
    l1 = torch.exp(torch.sum(lambda_q1.float() * lambda_k1.float()))
    l2 = torch.exp(torch.sum(lambda_q2.float() * lambda_k2.float()))
    return (l1 - l2 + float(lambda_init)).reshape(1)


class DiffAttnCore(torch.nn.Module):
    """The attention core of a differential-attention layer around the operator: owns the four lambda vectors
    and the output norm's gain, forms lambda on the device and calls `MultiheadDiffAttnKernel` with rms_norm on.
    Projections and head reshapes stay with the caller."""

    def __init__(self, head_dim: int, lambda_init: float = 0.8, causal: bool = False, dropout_p: float = 0.0,
                 device=None, dtype=torch.float32):
        super().__init__()
        mk = lambda: torch.nn.Parameter(torch.zeros(head_dim, device=device, dtype=dtype).normal_(mean=0.0, std=0.1))
        self.lambda_q1, self.lambda_k1, self.lambda_q2, self.lambda_k2 = mk(), mk(), mk(), mk()
        self.gain = torch.nn.Parameter(torch.ones(2 * head_dim, device=device, dtype=dtype))
        self.lambda_init, self.causal, self.dropout_p = float(lambda_init), bool(causal), float(dropout_p)

    def forward(self, q1, q2, k1, k2, v):
        lam = lambda_from_reparam(self.lambda_q1, self.lambda_k1, self.lambda_q2, self.lambda_k2, self.lambda_init)
        return MultiheadDiffAttnKernel(q1, q2, k1, k2, v, lam, self.lambda_init, True, causal=self.causal,
                                       dropout_p=self.dropout_p if self.training else 0.0, gain=self.gain)


def device_status(device=None) -> None:
    """Synchronise and raise RuntimeError if a device-side bounded wait gave up in any kernel."""
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    _lib.check(_lib.lib.diffattn_status(int(dev)), "diffattn_status")
