"""Generate golden vectors by running the reference's own PyTorch differential-attention path.

Run once, in a container that has the reference checkout (path given by --reference, default
$DIFFATTN_REFERENCE or ../reference next to the repo); the produced `tests/golden/*.npz` are
committed and are what travels.  Nothing at test time imports the reference.

The reference module `src/layers.py` imports `apex.normalization.FusedRMSNorm` (third party,
apex==0.1, not vendored) and `flash_attn`.  Both are replaced by stand-ins before import:
the RMSNorm stand-in computes x * rsqrt(mean(x^2, -1) + 1e-5), the arithmetic the reference's own
kernel uses for the same step (src/kernel.py:196-198, eps at src/kernel.py:50); flash_attn is never
called on this path.  `kernel.py` needs triton only to define the Triton kernels; it is stubbed too
when triton cannot be imported.

Inputs: seeded N(0,1)*scale fp32 -> (optionally) rounded to fp16 -> handed to the reference as fp32.
The reference path `MultiheadDiffAttn` (src/layers.py:49-80) rounds P to fp16 internally.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)

from oracle import diffattn_oracle as oracle  # noqa: E402

CASES = [
    # name, B, H, N, D, scale, lambda, lambda_init, rms_norm, dy_uniform, seed
    ("c1_b2h16n512d32", 2, 16, 512, 32, 1.0, 0.5, 0.8, True, False, 1234),     # the CPU-runnable benchmark shape (fp32 on the host)
    ("selftest_b2h2n256d32", 2, 2, 256, 32, 0.5, 0.5, 0.8, True, True, 77),    # src/kernel.py:581-596
    ("small_d64_rms", 1, 2, 256, 64, 1.0, 0.5, 0.8, True, False, 5),
    ("small_d64_norms_neg", 1, 2, 128, 64, 1.0, -0.5, 0.2, False, False, 6),
    ("small_d128_norms", 1, 1, 128, 128, 1.0, 0.7, 0.2, False, False, 7),
]


def import_reference(ref_root):
    src = os.path.join(ref_root, "src")
    if not os.path.isdir(src):
        raise SystemExit(f"reference checkout not found at {ref_root}")

    class _RMSNorm(torch.nn.Module):
        def __init__(self, normalized_shape, elementwise_affine=False, eps=1e-5):
            super().__init__()
            self.eps = eps

        def forward(self, x):
            return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + self.eps)

    apex = types.ModuleType("apex")
    apex_norm = types.ModuleType("apex.normalization")
    apex_norm.FusedRMSNorm = _RMSNorm
    apex.normalization = apex_norm
    sys.modules["apex"] = apex
    sys.modules["apex.normalization"] = apex_norm
    fa = types.ModuleType("flash_attn")
    fa.flash_attn_func = None
    sys.modules["flash_attn"] = fa
    sys.path.insert(0, src)
    import layers  # the reference module
    return layers


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DIFFATTN_REFERENCE",
                                                          os.path.join(os.path.dirname(REPO), "reference")))
    args = ap.parse_args()
    layers = import_reference(args.reference)
    for name, b, h, n, d, scale, lam, lam_init, rms, dyu, seed in CASES:
        q1, q2, k1, k2, v, dy = oracle.make_inputs(b, h, n, d, seed, scale, torch.float16, dyu)
        leaves = [t.float().clone().requires_grad_(True) for t in (q1, q2, k1, k2, v)]
        lam_t = torch.tensor([lam], dtype=torch.float32, requires_grad=True)   # shape [1], README.md:17
        y = layers.MultiheadDiffAttn(*leaves, lambda_scale=lam_t, lambda_init=lam_init, rms_norm=rms)
        y.backward(dy.float())
        out = {
            "meta": np.array([b, h, n, d, seed], dtype=np.int64),
            "fmeta": np.array([scale, lam, lam_init, float(rms), float(dyu)], dtype=np.float64),
            "y": y.detach().numpy(),
            "dlambda": lam_t.grad.numpy(),
        }
        for nm, t in zip(("dq1", "dq2", "dk1", "dk2", "dv"), leaves):
            out[nm] = t.grad.numpy()
        # keep a strided sample of sequence rows so the fixtures stay small in git
        step = 16 if n * b * h > 4096 else 4
        for k in ("y", "dq1", "dq2", "dk1", "dk2", "dv"):
            out[k] = np.ascontiguousarray(out[k][:, :, ::step, :])
        out["row_step"] = np.array([step])
        for k in ("y", "dq1", "dq2", "dk1", "dk2", "dv"):
            out[k] = out[k].astype(np.float32)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **out)
        print(name, "->", path, os.path.getsize(path) // 1024, "KiB", "dlambda", float(lam_t.grad))


if __name__ == "__main__":
    main()
