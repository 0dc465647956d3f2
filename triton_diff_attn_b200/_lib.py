"""ctypes binding of the C ABI declared in include/diffattn.h.

There is no fallback: if the shared library is missing the import of this module raises, and every
operator in the package fails with it.
"""
from __future__ import annotations

import ctypes as C
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# DIFFATTN_LIBRARY names another build of the same library (for instance one compiled with other tuning macros)
LIB_PATH = os.environ.get("DIFFATTN_LIBRARY") or os.path.join(PKG_DIR, "libdiffattn.so")

EXPORTS = ("diffattn_fwd", "diffattn_bwd", "diffattn_bwd_stages", "diffattn_bwd_static", "diffattn_workspace_bytes", "diffattn_status",
           "diffattn_last_error", "diffattn_version", "diffattn_supports")

ERR_NAMES = {
    0: "OK", -1: "NULL_PTR", -2: "BAD_STRUCT", -3: "BAD_SHAPE", -4: "UNSUPPORTED_D", -5: "BAD_STRIDE",
    -6: "MISALIGNED", -7: "BAD_DTYPE", -8: "WORKSPACE", -9: "CUDA", -10: "TIMEOUT", -11: "WRONG_DEVICE",
}
VALUE_ERRORS = (-1, -2, -3, -4, -5, -6, -7, -8, -11)   # caller mistakes -> ValueError; the rest RuntimeError

LAMBDA_F16, LAMBDA_F32, LAMBDA_BF16 = 0, 1, 2
IO_F16, IO_BF16 = 0, 1
STAGE_PRE, STAGE_DKDV, STAGE_DQ, STAGE_FUSED, STAGE_DQ_FINISH = 1, 2, 4, 8, 16
STATIC_SCRATCH_BYTES = 32 << 20


class DiffAttnParams(C.Structure):
    """Mirror of `struct DiffAttnParams` (include/diffattn.h); field order and types must match."""
    _fields_ = [
        ("struct_size", C.c_uint32), ("device", C.c_int32), ("stream", C.c_void_p),
        ("B", C.c_int32), ("H", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("qk_stride_b", C.c_int64), ("qk_stride_h", C.c_int64), ("qk_stride_n", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64), ("v_stride_n", C.c_int64),
        ("q1", C.c_void_p), ("q2", C.c_void_p), ("k1", C.c_void_p), ("k2", C.c_void_p), ("v", C.c_void_p),
        ("lambda_scale", C.c_void_p), ("lambda_dtype", C.c_int32), ("rms_norm", C.c_int32),
        ("sm_scale", C.c_float), ("lambda_init", C.c_float), ("eps", C.c_float), ("causal", C.c_int32),
        ("y", C.c_void_p), ("a2", C.c_void_p), ("lse1", C.c_void_p), ("lse2", C.c_void_p), ("rstd", C.c_void_p),
        ("dy", C.c_void_p),
        ("dq1", C.c_void_p), ("dq2", C.c_void_p), ("dk1", C.c_void_p), ("dk2", C.c_void_p), ("dv", C.c_void_p),
        ("dlambda", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_uint64),
        ("io_dtype", C.c_int32), ("dropout_threshold", C.c_uint32), ("dropout_seed", C.c_uint64),
        ("gain", C.c_void_p), ("y_gained", C.c_void_p), ("dgain", C.c_void_p),
        ("single_pass", C.c_int32),
    ]


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python triton_diff_attn_b200/build.py` "
            "(needs nvcc with sm_100a support). There is no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    lib.diffattn_fwd.argtypes = [C.POINTER(DiffAttnParams)]
    lib.diffattn_fwd.restype = C.c_int
    lib.diffattn_bwd.argtypes = [C.POINTER(DiffAttnParams)]
    lib.diffattn_bwd.restype = C.c_int
    lib.diffattn_bwd_stages.argtypes = [C.POINTER(DiffAttnParams), C.c_int32]
    lib.diffattn_bwd_stages.restype = C.c_int
    lib.diffattn_bwd_static.argtypes = [C.POINTER(DiffAttnParams)]
    lib.diffattn_bwd_static.restype = C.c_int
    lib.diffattn_workspace_bytes.argtypes = [C.POINTER(DiffAttnParams)]
    lib.diffattn_workspace_bytes.restype = C.c_uint64
    lib.diffattn_status.argtypes = [C.c_int32]
    lib.diffattn_status.restype = C.c_int
    lib.diffattn_last_error.argtypes = []
    lib.diffattn_last_error.restype = C.c_char_p
    lib.diffattn_version.argtypes = []
    lib.diffattn_version.restype = C.c_int
    lib.diffattn_supports.argtypes = [C.c_int32, C.c_int32]
    lib.diffattn_supports.restype = C.c_int
    return lib


lib = _load()


def last_error() -> str:
    return lib.diffattn_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = f"{what}: DIFFATTN_ERR_{ERR_NAMES.get(rc, rc)}: {last_error()}"
    raise (ValueError if rc in VALUE_ERRORS else RuntimeError)(msg)


def new_params() -> DiffAttnParams:
    p = DiffAttnParams()
    p.struct_size = C.sizeof(DiffAttnParams)
    return p
