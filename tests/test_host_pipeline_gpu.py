"""GPU test of HostStepPipeline: steps fed from pinned host memory through three overlapped streams
return exactly what the plain operator call returns for the same inputs."""
import pytest
import torch

from oracle import diffattn_oracle as oracle

pytestmark = pytest.mark.gpu


def test_pipeline_matches_direct_call():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import triton_diff_attn_b200 as pkg
    dev = torch.device("cuda", 0)
    b, h, n, d = 2, 4, 512, 64
    steps = 5
    sets = [oracle.make_inputs(b, h, n, d, seed=900 + i) for i in range(steps)]
    lam = torch.tensor([0.5], device=dev)
    want = []
    for ins in sets:
        leaves = [t.to(dev).requires_grad_(True) for t in ins[:5]]
        lam_l = lam.clone().requires_grad_(True)
        y = pkg.MultiheadDiffAttnKernel(*leaves, lam_l, 0.8, True)
        y.backward(ins[5].to(dev))
        want.append([y.detach().cpu()] + [t.grad.cpu() for t in leaves] + [lam_l.grad.cpu()])
    pipe = pkg.HostStepPipeline(dev)
    outs = []
    pipe.begin()
    for ins in sets:
        host_in = [t.pin_memory() for t in ins]
        host_out = [torch.empty_like(t).pin_memory() for t in (ins[4], ins[0], ins[1], ins[2], ins[3], ins[4])]
        host_dl = torch.empty(1, dtype=torch.float32).pin_memory()
        pipe.submit(host_in, host_out, host_dl, lam, 0.8, True)
        outs.append((host_in, host_out, host_dl))
    pipe.end()
    torch.cuda.synchronize()
    pkg.device_status(0)
    for (_, host_out, host_dl), w in zip(outs, want):
        for got, ref in zip(host_out, w[:6]):
            assert torch.equal(got, ref)
        assert abs(float(host_dl) - float(w[6])) <= 1e-3 * max(1.0, abs(float(w[6])))
