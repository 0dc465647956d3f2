"""CPU tests of the C-ABI boundary: the library loads, exports what include/diffattn.h declares, and
rejects bad arguments with the documented codes before touching the device."""
import ctypes
import os
import re

import pytest
import torch

from oracle import diffattn_oracle as oracle

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from triton_diff_attn_b200 import _lib
    return _lib


def _good(L, n=256, d=64):
    p = L.new_params()
    p.B, p.H, p.N, p.D = 2, 2, n, d
    p.qk_stride_n, p.qk_stride_h, p.qk_stride_b = d, n * d, 2 * n * d
    p.v_stride_n, p.v_stride_h, p.v_stride_b = 2 * d, 2 * n * d, 4 * n * d
    fake = 0x10000   # never dereferenced: every check below fails before a launch
    for f in ("q1", "q2", "k1", "k2", "v", "lambda_scale", "y", "a2", "lse1", "lse2", "rstd"):
        setattr(p, f, fake)
    p.lambda_dtype = L.LAMBDA_F32
    p.sm_scale, p.lambda_init, p.eps = d ** -0.5, 0.8, 1e-5
    return p


def test_exports_match_header(L):
    hdr = open(os.path.join(REPO, "include", "diffattn.h")).read()
    declared = set(re.findall(r"\b(diffattn_[a-z_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    assert declared == set(L.EXPORTS)
    raw = ctypes.CDLL(L.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), name
    assert L.lib.diffattn_version() == 2
    assert "DIFFATTN_ERR_WRONG_DEVICE = -11" in hdr and L.ERR_NAMES[-11] == "WRONG_DEVICE"


def test_supports(L):
    assert L.lib.diffattn_supports(64, 0) == 1 and L.lib.diffattn_supports(64, 1) == 1
    assert L.lib.diffattn_supports(32, 0) == 1 and L.lib.diffattn_supports(32, 1) == 1
    assert L.lib.diffattn_supports(128, 0) == 1 and L.lib.diffattn_supports(128, 1) == 1
    assert L.lib.diffattn_supports(48, 0) == 0 and L.lib.diffattn_supports(256, 0) == 0
    assert L.lib.diffattn_supports(64, 2) == 0          # directions are 0 (forward) and 1 (backward)


def test_null_and_struct(L):
    assert L.lib.diffattn_fwd(None) == -1
    p = _good(L)
    p.struct_size = 8
    assert L.lib.diffattn_fwd(p) == -2
    assert "struct_size" in L.last_error()


@pytest.mark.parametrize("mutate,code", [
    (lambda p: setattr(p, "N", -128), -3),
    (lambda p: setattr(p, "D", 48), -4),
    (lambda p: setattr(p, "qk_stride_n", 60), -5),
    (lambda p: setattr(p, "v_stride_h", 12), -5),
    (lambda p: setattr(p, "v_stride_n", 64), -5),
    (lambda p: setattr(p, "q2", 0), -1),
    (lambda p: setattr(p, "k1", 0x10008), -6),
    (lambda p: setattr(p, "lambda_dtype", 9), -7),
    (lambda p: setattr(p, "io_dtype", 2), -7),
    (lambda p: setattr(p, "dropout_threshold", 256), -3),
    (lambda p: (setattr(p, "dropout_threshold", 26), setattr(p, "N", 131200)), -3),
    (lambda p: setattr(p, "B", 70000), -3),
])
def test_fwd_rejects(L, mutate, code):
    p = _good(L)
    mutate(p)
    assert L.lib.diffattn_fwd(p) == code
    assert L.last_error()


def test_bwd_rejects_missing_workspace_and_grads(L):
    p = _good(L)
    assert L.lib.diffattn_bwd(p) == -1             # dy NULL
    for f in ("dy", "dq1", "dq2", "dk1", "dk2", "dv", "dlambda"):
        setattr(p, f, 0x10000)
    assert L.lib.diffattn_bwd(p) == -8             # no workspace
    need = L.lib.diffattn_workspace_bytes(p)
    rows = 2 * 2 * 256
    assert need == rows * 128 * 2 + rows * 16        # dA + statistics
    p.single_pass = 1                                # + fp32 partial sums of dQ1, dQ2: [2][B*H][N_pad][64]
    assert L.lib.diffattn_workspace_bytes(p) == rows * 128 * 2 + rows * 16 + 2 * rows * 64 * 4
    p.single_pass = 0
    q = _good(L, n=200)      # ragged length: the statistics rows are padded to a multiple of 128 per (batch, head)
    assert L.lib.diffattn_workspace_bytes(q) == 2 * 2 * 200 * 128 * 2 + 2 * 2 * 256 * 16
    q.single_pass = 1
    assert L.lib.diffattn_workspace_bytes(q) == 2 * 2 * 200 * 128 * 2 + 2 * 2 * 256 * 16 + 2 * 2 * 2 * 256 * 64 * 4
    q128 = _good(L, n=256, d=128)
    q128.single_pass = 1
    assert L.lib.diffattn_workspace_bytes(q128) == rows * 256 * 2 + rows * 16      # head dim 128 has no single-pass form
    p.workspace, p.workspace_bytes = 0x10010, need
    assert L.lib.diffattn_bwd_stages(p, L.STAGE_PRE) == -6   # workspace not 256-byte aligned
    p.workspace, p.workspace_bytes = 0x10100, need - 1
    assert L.lib.diffattn_bwd(p) == -8
    # a stage that does not belong to the call's form is refused before anything touches the device
    p.workspace_bytes = need
    assert L.lib.diffattn_bwd_stages(p, L.STAGE_FUSED | L.STAGE_PRE) == -3 and "form" in L.last_error()
    p.single_pass = 1
    p.workspace_bytes = L.lib.diffattn_workspace_bytes(p)
    assert L.lib.diffattn_bwd_stages(p, L.STAGE_DQ) == -3


def test_empty_is_ok_without_device(L):
    p = _good(L)
    p.B = 0
    assert L.lib.diffattn_fwd(p) == 0
    assert L.lib.diffattn_workspace_bytes(p) == 0
    assert L.lib.diffattn_bwd(p) == 0 and L.lib.diffattn_bwd_static(p) == 0


def test_python_wrapper_has_no_cpu_path():
    import triton_diff_attn_b200 as pkg
    q = torch.zeros(1, 1, 128, 64, dtype=torch.float16)
    v = torch.zeros(1, 1, 128, 128, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pkg.MultiheadDiffAttnKernel(q, q, q, q, v, torch.tensor([0.5]))
    with pytest.raises(TypeError):
        pkg.MultiheadDiffAttnKernel(q, q, q, q, v, 0.5)


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    """Importing the binding without the shared object raises ImportError (no fallback)."""
    import importlib.util
    src = os.path.join(REPO, "triton_diff_attn_b200", "_lib.py")
    dst = tmp_path / "_lib_copy.py"
    dst.write_text(open(src).read())
    spec = importlib.util.spec_from_file_location("_lib_copy", dst)
    mod = importlib.util.module_from_spec(spec)
    with pytest.raises(ImportError, match="no CPU or PyTorch fallback"):
        spec.loader.exec_module(mod)


def test_preprocess_formula_matches_oracle():
    """The row preprocess reconstructs A from Y and rstd: dA = r (c dY - Y (dY.Y)/(c Dv)); checked here
    in fp64 against the oracle's dA (host-side restatement of the kernel's arithmetic)."""
    q1, q2, k1, k2, v, dy = oracle.make_inputs(1, 2, 64, 16, seed=31, dtype=torch.float64)
    lam = torch.tensor([0.4], dtype=torch.float64)
    c = 1 - 0.8
    w = oracle.backward_closed_form(q1, q2, k1, k2, v, lam, dy, 0.8, True, dtype=torch.float64)
    y, r = w["y"], w["rstd"][..., None]
    t = (dy * y).sum(-1, keepdim=True)
    da = r * (c * dy - y * t / (c * y.shape[-1]))
    assert torch.allclose(da, w["da"], rtol=1e-10, atol=1e-12)
    a = y / (c * r)
    e2 = (da * w["a2"]).sum(-1)
    e1 = (da * a).sum(-1) + 0.4 * e2
    assert torch.allclose(e1, w["e1"], rtol=1e-9, atol=1e-11)


def test_dropout_probability_quantisation():
    from triton_diff_attn_b200.layers import dropout_threshold
    assert dropout_threshold(0.0) == 0 and dropout_threshold(0.25) == 64 and dropout_threshold(0.1) == 26
    assert dropout_threshold(0.001) == 0            # below 1/512: off
    for bad in (-0.1, 1.0, 0.999):
        with pytest.raises(ValueError):
            dropout_threshold(bad)
