"""Install and import the UNMODIFIED reference (aharbi/triton-diff-attn) for the benchmark's reference arm.

`install()` copies the reference's two hot-path modules, `src/layers.py` and `src/kernel.py`, from a checkout
into `baseline/_ref/`, a git-ignored folder (the copies never enter the repository's history; like the built
shared library they travel to the GPU box with the working tree).  The reference has no setup.py or
pyproject.toml -- it is four scripts -- so there is nothing to pip-install.

`load()` imports `layers` from there.  Its two third-party imports are replaced by stand-ins first:
  * `apex.normalization.FusedRMSNorm` (apex==0.1, not installed, not vendored): x * rsqrt(mean(x^2, -1) + 1e-5),
    the arithmetic the reference's own kernel uses for the same step (src/kernel.py:196-198, eps :50);
  * `flash_attn` when it cannot be imported (only the comparison layers use it).
`triton` is imported by the reference's kernel module; the image has it.  Nothing in the shipped package
imports this file; `bench.py --impl reference` and `--impl reference_triton` do.
"""
from __future__ import annotations

import os
import shutil
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = ("layers.py", "kernel.py")


def default_checkout() -> str:
    return os.environ.get("DIFFATTN_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def installed() -> bool:
    return all(os.path.exists(os.path.join(REF_DIR, f)) for f in FILES)


def install(checkout: str | None = None) -> bool:
    """Copy the reference modules into baseline/_ref/.  Returns False (and changes nothing) when the checkout
    is not present, as on the GPU box."""
    src = os.path.join(checkout or default_checkout(), "src")
    if not all(os.path.exists(os.path.join(src, f)) for f in FILES):
        return False
    os.makedirs(REF_DIR, exist_ok=True)
    for f in FILES:
        shutil.copyfile(os.path.join(src, f), os.path.join(REF_DIR, f))
    return True


def load():
    """Import the reference's `layers` module from baseline/_ref/ (raises ImportError when not installed)."""
    if not installed():
        raise ImportError(f"{REF_DIR} does not hold the reference modules; run baseline/ref_loader.py where the "
                          "reference checkout is present")
    import torch

    class _RMSNorm(torch.nn.Module):
        def __init__(self, normalized_shape, elementwise_affine=False, eps=1e-5):
            super().__init__()
            self.eps = eps

        def forward(self, x):
            return x * torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + self.eps)

    if "apex" not in sys.modules:
        apex = types.ModuleType("apex")
        apex_norm = types.ModuleType("apex.normalization")
        apex_norm.FusedRMSNorm = _RMSNorm
        apex.normalization = apex_norm
        sys.modules["apex"] = apex
        sys.modules["apex.normalization"] = apex_norm
    try:
        import flash_attn  # noqa: F401
    except Exception:
        fa = types.ModuleType("flash_attn")
        fa.flash_attn_func = None
        sys.modules["flash_attn"] = fa
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import layers  # the reference module
    return layers


if __name__ == "__main__":
    ok = install(sys.argv[1] if len(sys.argv) > 1 else None)
    print("installed" if ok else "reference checkout not found; nothing installed", REF_DIR)
