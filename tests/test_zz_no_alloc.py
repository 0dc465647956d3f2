"""GPU test of `diffattn_bwd_static`, the backward entry point for hosts that cannot allocate.

Some users of the C ABI have no device allocator in their step loop: they were handed a fixed set of
buffers, or they avoid cudaMalloc there because it synchronises the device.  For them the library
carries its backward scratch inside its own image (32 MiB per GPU).  This test drives that entry
point through ctypes exactly as such a host would, several times in a row with different upstream
gradients and shapes (the scratch keeps the previous call's contents, so a stale read would show), and
compares every gradient with what the ordinary `diffattn_bwd` (caller workspace) produces for the same
inputs.  Both entry points run the same kernels, so the comparison is exact wherever the kernels are
bit-reproducible: everything in the default form, and everything but dq1/dq2 (fp32 atomic sums, compared
at the parity tolerance) with single_pass = 1.
The file name sorts last so that a run stopping at the first failure has already run everything else.
"""
import ctypes

import pytest
import torch

from oracle import diffattn_oracle as oracle

pytestmark = pytest.mark.gpu

GRADS = ("dq1", "dq2", "dk1", "dk2", "dv")


def _setup(b, h, n, d, seed, single_pass):
    from triton_diff_attn_b200 import _lib, layers
    dev = torch.device("cuda", 0)
    q1, q2, k1, k2, v, dy = (t.to(dev) for t in oracle.make_inputs(b, h, n, d, seed))
    lam = torch.tensor([0.5], dtype=torch.float32, device=dev)
    y, a2 = torch.empty_like(v), torch.empty_like(v)
    lse1 = torch.empty(b, h, n, dtype=torch.float32, device=dev)
    lse2, rstd = torch.empty_like(lse1), torch.empty_like(lse1)
    p = _lib.new_params()
    layers._fill_common(p, q1, q2, k1, k2, v, lam, 0.8, True, (y, a2, lse1, lse2, rstd), single_pass=single_pass)
    _lib.check(_lib.lib.diffattn_fwd(ctypes.byref(p)), "diffattn_fwd")
    keep = (q1, q2, k1, k2, v, lam, y, a2, lse1, lse2, rstd)
    return _lib, p, keep, dy


def _grads_into(p, shapes_like, dev):
    q1, v = shapes_like
    out = {k: torch.zeros_like(q1) for k in GRADS[:4]}
    out["dv"] = torch.zeros_like(v)
    out["dlambda"] = torch.zeros(1, dtype=torch.float32, device=dev)
    p.dq1, p.dq2, p.dk1, p.dk2, p.dv = (out[k].data_ptr() for k in GRADS)
    p.dlambda = out["dlambda"].data_ptr()
    return out


@pytest.mark.parametrize("single_pass", [False, True])
def test_static_scratch_backward_matches_workspace_backward(single_pass):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda", 0)
    # three calls in a row on the shared array: two upstream gradients at one shape, then a ragged, wider shape whose
    # statistics rows and dA tail land on what the earlier calls left behind
    calls = [((2, 2, 256, 64), 41, 0), ((2, 2, 256, 64), 41, 1), ((1, 3, 200, 32 if single_pass else 128), 43, 0)]
    for call, (shape, seed, which_dy) in enumerate(calls):
        _lib, p, keep, dy = _setup(*shape, seed=seed, single_pass=single_pass)
        q1, v = keep[0], keep[4]
        if which_dy:
            g = torch.Generator(device="cpu").manual_seed(42)
            dy = torch.randn(dy.shape, generator=g).to(torch.float16).to(dev)
        p.dy = dy.data_ptr()
        # the ordinary entry point, with a workspace the caller (torch here) allocated
        want = _grads_into(p, (q1, v), dev)
        nbytes = int(_lib.lib.diffattn_workspace_bytes(ctypes.byref(p)))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        p.workspace, p.workspace_bytes = ws.data_ptr(), nbytes
        _lib.check(_lib.lib.diffattn_bwd(ctypes.byref(p)), "diffattn_bwd")
        torch.cuda.synchronize()
        # the allocation-free entry point: no workspace handed over, and the device's free memory must not move
        got = _grads_into(p, (q1, v), dev)
        p.workspace, p.workspace_bytes = None, 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        _lib.check(_lib.lib.diffattn_bwd_static(ctypes.byref(p)), "diffattn_bwd_static")
        _lib.check(_lib.lib.diffattn_status(0), "diffattn_status")
        assert torch.cuda.mem_get_info(dev)[0] == free_before, "diffattn_bwd_static changed the free device memory"
        for k in GRADS:
            assert float(want[k].abs().max()) > 0, k
            if k in ("dq1", "dq2") and single_pass and shape[3] <= 64:
                m = oracle.error_metrics(got[k].cpu(), want[k].cpu().float())
                assert m["max_abs"] <= 2e-2 and m["rel_l2"] <= 1e-3, (call, k, m)
            else:
                assert torch.equal(got[k], want[k]), (call, k)
        a, b = float(got["dlambda"].cpu()), float(want["dlambda"].cpu())
        assert abs(a - b) <= 1e-2 * max(abs(b), 1e-3), (call, a, b)


def test_static_scratch_rejects_shapes_beyond_its_size():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from triton_diff_attn_b200 import _lib
    p = _lib.new_params()
    p.B, p.H, p.N, p.D = 4, 16, 4096, 64          # needs far more scratch than 32 MiB
    assert _lib.lib.diffattn_workspace_bytes(ctypes.byref(p)) > _lib.STATIC_SCRATCH_BYTES
    assert _lib.lib.diffattn_bwd_static(ctypes.byref(p)) == -8
    assert "built-in array" in _lib.last_error()
    p.B = 0                                        # an empty shape is fine and touches nothing
    assert _lib.lib.diffattn_bwd_static(ctypes.byref(p)) == 0
