"""The forward and backward C-ABI calls inside a CUDA graph: they allocate nothing, never synchronise and take the
stream from the caller, so a serving or training loop can capture them once and replay.  (Tensor maps are encoded
on the host at capture time: the graph is tied to the buffers it was captured with.)"""
import pytest
import torch

from oracle import diffattn_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,causal", [(64, False), (128, True)])
def test_capture_and_replay(d, causal):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from triton_diff_attn_b200 import _lib, layers
    dev = torch.device("cuda", 0)
    b, h, n = 2, 2, 384
    q1, q2, k1, k2, v, dy = (t.to(dev) for t in oracle.make_inputs(b, h, n, d, 31))
    lam = torch.tensor([0.5], device=dev)
    y, a2 = torch.empty_like(v), torch.empty_like(v)
    l1 = torch.empty(b, h, n, device=dev); l2 = torch.empty_like(l1); rs = torch.empty_like(l1)
    grads = [torch.empty_like(q1) for _ in range(4)] + [torch.empty_like(v)]
    dl = torch.zeros(1, device=dev)

    def params(stream):
        p = _lib.new_params()
        layers._fill_common(p, q1, q2, k1, k2, v, lam, 0.8, True, (y, a2, l1, l2, rs), causal)
        p.stream = stream
        p.dy = dy.data_ptr()
        p.dq1, p.dq2, p.dk1, p.dk2, p.dv = (t.data_ptr() for t in grads)
        p.dlambda = dl.data_ptr()
        return p

    p0 = params(torch.cuda.current_stream().cuda_stream)
    nb = int(_lib.lib.diffattn_workspace_bytes(p0))
    ws = torch.empty(nb, dtype=torch.uint8, device=dev)
    p0.workspace, p0.workspace_bytes = ws.data_ptr(), nb

    def eager():
        dl.zero_()
        _lib.check(_lib.lib.diffattn_fwd(p0), "fwd")
        _lib.check(_lib.lib.diffattn_bwd(p0), "bwd")
        torch.cuda.synchronize()
        return [t.clone() for t in [y] + grads], float(dl)

    want, want_dl = eager()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        p1 = params(torch.cuda.current_stream().cuda_stream)
        p1.workspace, p1.workspace_bytes = ws.data_ptr(), nb
        dl.zero_()
        _lib.check(_lib.lib.diffattn_fwd(p1), "fwd in capture")
        _lib.check(_lib.lib.diffattn_bwd(p1), "bwd in capture")
    for _rep in range(2):
        for t in [y] + grads:
            t.zero_()
        g.replay()
        torch.cuda.synchronize()
        for a, w in zip([y] + grads, want):
            assert torch.equal(a, w)                    # the kernels are deterministic; d(lambda) sums by atomics
        assert abs(float(dl) - want_dl) <= 1e-4 * max(1.0, abs(want_dl))
        # new contents in the captured buffers, then the eager result for the next replay to match
        q1.copy_(q1.flip(2)); v.copy_(v * 0.5)
        want, want_dl = eager()
    _lib.check(_lib.lib.diffattn_status(0), "status")
