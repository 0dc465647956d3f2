"""CPU oracle for differential attention (forward and backward).

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA path is compared with; it is
never imported by the shipped package.  Only the tests, the smoke entry and the CPU-baseline leg of
the benchmark may use it.

Parity status: PINNED.  `tests/golden/*.npz` were produced by importing the reference's own
`MultiheadDiffAttn` (src/layers.py:49-80) with a stand-in for the un-vendored third-party
`apex.normalization.FusedRMSNorm` (apex==0.1, requirements.txt:1; arithmetic restated from the
reference's own kernel, src/kernel.py:196-198, eps from src/kernel.py:50), see
`tests/golden/make_golden.py`.  `tests/test_oracle.py` checks this restatement against them.

Algorithm restated (per batch b, head h; s = 1/sqrt(D), c = 1 - lambda_init, Dv = 2 D):

    S_b = s Q_b K_b^T                      src/layers.py:64,67   (sm_scale from D, layers.py:60-62)
    P_b = softmax_rows(S_b)                src/layers.py:65,68
    A   = (P_1 - lam P_2) V                src/layers.py:70-72
    Y   = c A rsqrt(mean(A^2) + eps)       src/layers.py:74-78, src/kernel.py:196-198
    Y   = A            when rms_norm off   src/layers.py:74,80   (lambda_init unused then)

The reference rounds P_b to fp16 with a hard-coded `.half()` (layers.py:65,68).  `round_p_half=True`
mirrors that literally (used to pin the oracle to the golden vectors); the default keeps P in the
compute dtype, which is the fp32 parity target of the CUDA kernels.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

EPS = 1e-5  # src/kernel.py:50


def _lam(lambda_scale, dtype, device="cpu") -> torch.Tensor:
    if not torch.is_tensor(lambda_scale):
        lambda_scale = torch.tensor([float(lambda_scale)])
    return lambda_scale.detach().reshape(-1)[0].to(dtype=dtype, device=device)


def _mix32(h: np.ndarray) -> np.ndarray:
    """Two-multiply xorshift finaliser on uint32 arrays (wrap-around arithmetic), as in csrc/sm100.cuh."""
    h = h.astype(np.uint32)
    h = h ^ (h >> np.uint32(16))
    h = (h * np.uint32(0x7feb352d)).astype(np.uint32)
    h = h ^ (h >> np.uint32(15))
    h = (h * np.uint32(0x846ca68b)).astype(np.uint32)
    h = h ^ (h >> np.uint32(16))
    return h


def dropout_keep_mask(seed: int, bh: int, branch: int, n: int, threshold: int) -> np.ndarray:
    """Keep decisions [n, n] (query row, key column) of attention dropout for one (batch*head, branch).

    Restates the device rule (extension; the reference has no dropout, README.md:2): one 32-bit hash per 2x2
    block, h = mix32(((row>>1)<<16 | (col>>1)) ^ key), key = mix32(seed_lo ^ mix32(seed_hi + 0x9E3779B9 (2 bh +
    branch + 1))); position (row, col) is kept iff byte 2 (row&1) + (col&1) of h is >= threshold."""
    with np.errstate(over="ignore"):
        lo, hi = np.uint32(seed & 0xffffffff), np.uint32((seed >> 32) & 0xffffffff)
        inner = np.array([(int(hi) + 0x9E3779B9 * (2 * bh + branch + 1)) & 0xffffffff], dtype=np.uint32)
        key = _mix32(lo ^ _mix32(inner))[0]
        r = np.arange(n, dtype=np.uint32)[:, None]
        c = np.arange(n, dtype=np.uint32)[None, :]
        h = _mix32((((r >> np.uint32(1)) << np.uint32(16)) | (c >> np.uint32(1))) ^ key)
        byte = (np.uint32(2) * (r & np.uint32(1)) + (c & np.uint32(1))) * np.uint32(8)
        return ((h >> byte) & np.uint32(0xff)) >= np.uint32(threshold)


def dropout_multipliers(b: int, h: int, n: int, threshold: int, seed: int, dtype, device):
    """(m1, m2): [b, h, n, n] tensors holding 0 (dropped) or 256/(256 - threshold) (kept) per branch."""
    scale = 256.0 / (256 - threshold)
    out = []
    for br in (0, 1):
        m = np.stack([dropout_keep_mask(seed, i, br, n, threshold) for i in range(b * h)]).reshape(b, h, n, n)
        out.append(torch.from_numpy(m).to(device=device, dtype=dtype) * scale)
    return out


def forward(q1, q2, k1, k2, v, lambda_scale, lambda_init: float = 0.8, rms_norm: bool = False,
            dtype=torch.float32, round_p_half: bool = False, eps: float = EPS, device="cpu",
            causal: bool = False, dropout_threshold: int = 0, dropout_seed: int = 0, gain=None) -> Dict[str, torch.Tensor]:
    """Forward pass; returns Y and the intermediates the backward kernels save (src/layers.py:60-80).

    Keys: y, a (pre-norm), a1, a2 (per-branch P_b V), lse1, lse2 (natural-log logsumexp of S_b,
    the quantity the reference kernel stores as M1/M2, src/kernel.py:188-189), rstd.

    `device` selects where torch evaluates the same restatement (default CPU).  Tests of sequence lengths
    whose N x N matrices are too slow on the host pass a CUDA device and get the identical fp32 arithmetic
    there (TF32 off); the baseline timing always uses the CPU.
    """
    q1, q2, k1, k2, v = (t.detach().to(device, dtype) for t in (q1, q2, k1, k2, v))
    lam = _lam(lambda_scale, dtype, device)
    d = q1.shape[-1]
    s = 1.0 / math.sqrt(d)                                             # layers.py:60-62
    s1 = torch.matmul(q1, k1.transpose(2, 3)) * s                      # layers.py:64
    s2 = torch.matmul(q2, k2.transpose(2, 3)) * s                      # layers.py:67
    if causal:
        # extension (the reference has no masking, README.md:2): key j is visible to query i iff j <= i
        n = s1.shape[-1]
        hidden = torch.ones(n, n, dtype=torch.bool, device=s1.device).triu(1)
        s1 = s1.masked_fill(hidden, float("-inf"))
        s2 = s2.masked_fill(hidden, float("-inf"))
    lse1 = torch.logsumexp(s1, dim=-1)
    lse2 = torch.logsumexp(s2, dim=-1)
    p1 = torch.softmax(s1, dim=-1)                                     # layers.py:65
    p2 = torch.softmax(s2, dim=-1)                                     # layers.py:68
    if round_p_half:
        p1 = p1.half().to(dtype)
        p2 = p2.half().to(dtype)
    m1 = m2 = None
    pd1, pd2 = p1, p2
    if dropout_threshold:
        # extension: P_b -> P_b * keep_b / (1 - p), after the softmax (its denominator sees every key)
        m1, m2 = dropout_multipliers(q1.shape[0], q1.shape[1], q1.shape[2], dropout_threshold, dropout_seed, dtype, s1.device)
        pd1, pd2 = p1 * m1, p2 * m2
    a1 = torch.matmul(pd1, v)
    a2 = torch.matmul(pd2, v)
    a = torch.matmul(pd1 - lam * pd2, v)                               # layers.py:70-72
    rstd = torch.rsqrt((a * a).mean(dim=-1) + eps)                     # kernel.py:196-197
    if rms_norm:
        y = (1.0 - lambda_init) * a * rstd[..., None]                  # layers.py:75-78
    else:
        y = a                                                          # layers.py:80
    out = {"y": y, "a": a, "a1": a1, "a2": a2, "lse1": lse1, "lse2": lse2, "rstd": rstd,
           "p1": p1, "p2": p2, "m1": m1, "m2": m2}
    if gain is not None:
        # extension: learnable column gain of the output norm; "y" stays the un-gained value the backward keeps
        out["y_gained"] = y * gain.detach().to(y.device, dtype)
    return out


def backward_closed_form(q1, q2, k1, k2, v, lambda_scale, dy, lambda_init: float = 0.8,
                         rms_norm: bool = False, dtype=torch.float32,
                         eps: float = EPS, device="cpu", causal: bool = False,
                         dropout_threshold: int = 0, dropout_seed: int = 0, gain=None) -> Dict[str, torch.Tensor]:
    """Closed-form gradients (no autograd).  With `gain`, dy is the gradient of y * gain.  Same quantities the reference's backward kernel forms
    (src/kernel.py:283-299 preprocess, :410-436 main loop), with the division-free d(lambda).

        dA   = c (r dY - r^3 A (dY.A)/Dv)     (rms on; kernel.py:283-290)   |  dA = dY (rms off)
        dP   = dA V^T
        E_b  = rowsum(dA * A_b)               (= the reference's D1, and D2 / (-lambda); kernel.py:295-296)
        dV   = (P_1 - lam P_2)^T dA           (kernel.py:416)
        dS_1 = P_1 * (dP - E_1),  dS_2 = -lam P_2 * (dP - E_2)       (kernel.py:420-421)
        dQ_b = s dS_b K_b,  dK_b = s dS_b^T Q_b                       (kernel.py:423-424,435-436)
        dlam = - sum E_2
    """
    f = forward(q1, q2, k1, k2, v, lambda_scale, lambda_init, rms_norm, dtype=dtype, eps=eps, device=device, causal=causal,
                dropout_threshold=dropout_threshold, dropout_seed=dropout_seed, gain=gain)
    q1, q2, k1, k2, v, dy = (t.detach().to(device, dtype) for t in (q1, q2, k1, k2, v, dy))
    dgain = None
    if gain is not None:
        dgain = (dy * f["y"]).sum(dim=(0, 1, 2))
        dy = dy * gain.detach().to(device, dtype)
    lam = _lam(lambda_scale, dtype, device)
    d = q1.shape[-1]
    dv_dim = v.shape[-1]
    s = 1.0 / math.sqrt(d)
    a, r = f["a"], f["rstd"][..., None]
    if rms_norm:
        c = 1.0 - lambda_init
        da = c * (r * dy - r ** 3 * a * (dy * a).sum(-1, keepdim=True) / dv_dim)
    else:
        da = dy
    dp = torch.matmul(da, v.transpose(2, 3))
    e1 = (da * f["a1"]).sum(-1, keepdim=True)
    e2 = (da * f["a2"]).sum(-1, keepdim=True)
    # with dropout (multipliers m_b = keep_b / (1 - p)): P_b m_b feeds A_b and dV, and dP reaches S_b through m_b
    m1 = f["m1"] if f["m1"] is not None else 1.0
    m2 = f["m2"] if f["m2"] is not None else 1.0
    dvv = torch.matmul((f["p1"] * m1 - lam * f["p2"] * m2).transpose(2, 3), da)
    ds1 = f["p1"] * (m1 * dp - e1)
    ds2 = -lam * f["p2"] * (m2 * dp - e2)
    out = {
        "dq1": s * torch.matmul(ds1, k1), "dq2": s * torch.matmul(ds2, k2),
        "dk1": s * torch.matmul(ds1.transpose(2, 3), q1), "dk2": s * torch.matmul(ds2.transpose(2, 3), q2),
        "dv": dvv, "dlambda": -e2.sum(), "da": da, "e1": e1[..., 0], "e2": e2[..., 0],
    }
    out.update({k: f[k] for k in ("y", "lse1", "lse2", "rstd", "a2")})
    if gain is not None:
        out["dgain"], out["y_gained"] = dgain, f["y_gained"]
    return out


def forward_backward_autograd(q1, q2, k1, k2, v, lambda_scale, dy, lambda_init: float = 0.8,
                              rms_norm: bool = False, dtype=torch.float32, round_p_half: bool = False,
                              eps: float = EPS, num_threads: Optional[int] = None, causal: bool = False,
                              dropout_threshold: int = 0, dropout_seed: int = 0, gain=None) -> Dict[str, torch.Tensor]:
    """Forward + autograd backward of the literal op sequence of src/layers.py:60-80.

    This is the independent check of `backward_closed_form` and the function the CPU baseline times.
    """
    if num_threads:
        torch.set_num_threads(num_threads)
    leaves = [t.detach().to("cpu", dtype).clone().requires_grad_(True) for t in (q1, q2, k1, k2, v)]
    lam = _lam(lambda_scale, dtype).reshape(1).clone().requires_grad_(True)
    lq1, lq2, lk1, lk2, lv = leaves
    d = lq1.shape[-1]
    s = 1.0 / math.sqrt(d)
    sc1 = torch.matmul(lq1, lk1.transpose(2, 3)) * s
    sc2 = torch.matmul(lq2, lk2.transpose(2, 3)) * s
    if causal:
        n = sc1.shape[-1]
        hidden = torch.ones(n, n, dtype=torch.bool).triu(1)
        sc1 = sc1.masked_fill(hidden, float("-inf"))
        sc2 = sc2.masked_fill(hidden, float("-inf"))
    p1 = torch.softmax(sc1, dim=-1)
    p2 = torch.softmax(sc2, dim=-1)
    if round_p_half:
        # straight-through is NOT used by the reference: .half() is differentiable as a cast
        p1 = p1.half().to(dtype)
        p2 = p2.half().to(dtype)
    if dropout_threshold:
        m1, m2 = dropout_multipliers(lq1.shape[0], lq1.shape[1], lq1.shape[2], dropout_threshold, dropout_seed, dtype, "cpu")
        p1, p2 = p1 * m1, p2 * m2
    a = torch.matmul(p1 - lam * p2, lv)
    if rms_norm:
        y = (1.0 - lambda_init) * a * torch.rsqrt((a * a).mean(-1, keepdim=True) + eps)
    else:
        y = a
    gl = None
    if gain is not None:
        gl = gain.detach().to("cpu", dtype).clone().requires_grad_(True)
        y = y * gl
    y.backward(dy.detach().to("cpu", dtype))
    out = {"y": y.detach(), "dq1": lq1.grad, "dq2": lq2.grad, "dk1": lk1.grad, "dk2": lk2.grad,
           "dv": lv.grad, "dlambda": lam.grad.reshape(())}
    if gl is not None:
        out["dgain"] = gl.grad
    return out


def error_metrics(got: torch.Tensor, want: torch.Tensor) -> Dict[str, float]:
    """max-abs and relative-L2 error of `got` against `want`, both taken in fp64."""
    g = got.detach().to("cpu", torch.float64)
    w = want.detach().to("cpu", torch.float64)
    diff = g - w
    denom = float(w.norm())
    return {"max_abs": float(diff.abs().max()) if diff.numel() else 0.0,
            "rel_l2": float(diff.norm()) / denom if denom > 0 else float(diff.norm())}


def make_inputs(b: int, h: int, n: int, d: int, seed: int, scale: float = 1.0, dtype=torch.float16,
                dy_uniform: bool = False):
    """Seeded synthetic inputs: i.i.d. N(0,1)*scale drawn in fp32 on the CPU, then cast.

    dy_uniform=True reproduces the reference self-test's `rand_like` upstream gradient
    (src/kernel.py:596).  Returns (q1, q2, k1, k2, v, dy).
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    def draw(*shape):
        return (torch.randn(*shape, generator=g, dtype=torch.float32) * scale).to(dtype)
    q1, q2, k1, k2 = (draw(b, h, n, d) for _ in range(4))
    v = draw(b, h, n, 2 * d)
    if dy_uniform:
        dy = torch.rand(b, h, n, 2 * d, generator=g, dtype=torch.float32).to(dtype)
    else:
        dy = torch.randn(b, h, n, 2 * d, generator=g, dtype=torch.float32).to(dtype)
    return q1, q2, k1, k2, v, dy
