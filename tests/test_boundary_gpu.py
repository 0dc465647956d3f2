"""GPU tests of the C-ABI boundary's device handling: a tensor pointer that is not device memory of the named
device is refused before any launch, and every entry point leaves the caller's current device as it found it."""
import ctypes

import pytest
import torch

from oracle import diffattn_oracle as oracle

pytestmark = pytest.mark.gpu


def _problem(dev, b=1, h=2, n=256, d=64, seed=7):
    from triton_diff_attn_b200 import _lib, layers
    q1, q2, k1, k2, v, dy = (t.to(dev) for t in oracle.make_inputs(b, h, n, d, seed))
    lam = torch.tensor([0.5], dtype=torch.float32, device=dev)
    y, a2 = torch.empty_like(v), torch.empty_like(v)
    lse1 = torch.empty(b, h, n, dtype=torch.float32, device=dev)
    lse2, rstd = torch.empty_like(lse1), torch.empty_like(lse1)
    p = _lib.new_params()
    layers._fill_common(p, q1, q2, k1, k2, v, lam, 0.8, True, (y, a2, lse1, lse2, rstd))
    return _lib, p, (q1, q2, k1, k2, v, dy, lam, y, a2, lse1, lse2, rstd)


def test_host_pointer_is_refused():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda", 0)
    _lib, p, keep = _problem(dev)
    pinned = torch.zeros(keep[0].shape, dtype=torch.float16).pin_memory()      # host memory the GPU could even reach
    p.k2 = pinned.data_ptr()
    assert _lib.lib.diffattn_fwd(ctypes.byref(p)) == -11
    assert "k2" in _lib.last_error() and "not device memory" in _lib.last_error()
    with pytest.raises(ValueError, match="WRONG_DEVICE"):
        _lib.check(_lib.lib.diffattn_fwd(ctypes.byref(p)), "diffattn_fwd")
    p.k2 = keep[3].data_ptr()
    assert _lib.lib.diffattn_fwd(ctypes.byref(p)) == 0
    _lib.check(_lib.lib.diffattn_status(0), "diffattn_status")


def test_other_gpus_pointer_is_refused_and_current_device_is_kept():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    dev1 = torch.device("cuda", 1)
    _lib, p, keep = _problem(dev1)
    torch.cuda.set_device(0)
    # a call that names device 1 while device 0 is current: runs there and leaves device 0 current
    assert _lib.lib.diffattn_fwd(ctypes.byref(p)) == 0
    assert torch.cuda.current_device() == 0
    _lib.check(_lib.lib.diffattn_status(1), "diffattn_status")
    assert torch.cuda.current_device() == 0
    want = oracle.forward(*(t.cpu() for t in keep[:5]), torch.tensor([0.5]), 0.8, True)
    assert oracle.error_metrics(keep[7].cpu(), want["y"])["rel_l2"] <= 1e-3
    # a tensor of device 0 handed to a call that names device 1
    foreign = torch.zeros_like(keep[4], device=torch.device("cuda", 0))
    p.v = foreign.data_ptr()
    assert _lib.lib.diffattn_fwd(ctypes.byref(p)) == -11
    assert "device 0" in _lib.last_error() and "device 1" in _lib.last_error()
    assert torch.cuda.current_device() == 0
