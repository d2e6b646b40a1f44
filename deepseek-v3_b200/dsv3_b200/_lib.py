"""ctypes binding of libdsv3_b200.so (the C ABI declared in include/dsv3_b200.h).

The library is built in-tree by ``deepseek-v3_b200/build.py``.  There is no other
implementation behind these functions: if the shared object is missing the import
fails, and tensors that are not on a CUDA device are rejected.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libdsv3_b200.so")

OK = 0
ERR_INVALID_ARGUMENT = -1
ERR_UNSUPPORTED = -2
ERR_CUDA = -3
ERR_WORKSPACE = -4
ERR_DEVICE_TIMEOUT = -5
WORKSPACE_HEADER_BYTES = 16384

EXPORTS = (
    "dsv3_version", "dsv3_strerror", "dsv3_last_error", "dsv3_act_quant", "dsv3_weight_dequant",
    "dsv3_fp8_gemm_workspace_bytes", "dsv3_fp8_gemm", "dsv3_set_gemm_policy", "dsv3_weight_quant",
    "dsv3_check_device_status", "dsv3_fp8_gemm_static", "dsv3_fp8_gemm_static_scratch_bytes",
    "dsv3_group_table_bytes", "dsv3_group_table_build", "dsv3_fp8_gemm_grouped", "dsv3_moe_combine", "dsv3_moe_route",
    "dsv3_fp8_linear", "dsv3_swiglu_quant", "dsv3_selftest_bounded_wait", "dsv3_p2p_handle_bytes", "dsv3_p2p_create", "dsv3_p2p_connect", "dsv3_p2p_connect_local", "dsv3_p2p_base",
    "dsv3_allreduce_oneshot", "dsv3_allreduce_oneshot_pair_on_one_gpu", "dsv3_p2p_destroy", "dsv3_set_num_sms",
)


class Dsv3Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python deepseek-v3_b200/build.py` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    i64, vp, ci, sz = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.dsv3_version.restype = ci
    lib.dsv3_strerror.argtypes = [ci]
    lib.dsv3_strerror.restype = ctypes.c_char_p
    lib.dsv3_last_error.restype = ctypes.c_char_p
    lib.dsv3_act_quant.argtypes = [vp, i64, i64, ci, ci, vp, vp, vp]
    lib.dsv3_selftest_bounded_wait.argtypes = [ctypes.c_uint64, vp]
    lib.dsv3_swiglu_quant.argtypes = [vp, vp, i64, i64, ci, vp, vp, vp]
    lib.dsv3_weight_dequant.argtypes = [vp, vp, i64, i64, ci, vp, vp]
    lib.dsv3_fp8_gemm_workspace_bytes.argtypes = [i64, i64, i64]
    lib.dsv3_fp8_gemm_workspace_bytes.restype = sz
    lib.dsv3_fp8_gemm.argtypes = [vp, vp, vp, vp, i64, i64, i64, vp, vp, sz, vp]
    u64 = ctypes.c_uint64
    lib.dsv3_p2p_handle_bytes.restype = sz
    lib.dsv3_p2p_create.argtypes = [ci, ci, sz, ctypes.POINTER(vp), vp]
    lib.dsv3_p2p_connect.argtypes = [vp, vp]
    lib.dsv3_p2p_connect_local.argtypes = [vp, vp]
    lib.dsv3_p2p_base.argtypes = [vp]
    lib.dsv3_p2p_base.restype = vp
    lib.dsv3_allreduce_oneshot.argtypes = [vp, vp, vp, i64, u64, vp]
    lib.dsv3_allreduce_oneshot_pair_on_one_gpu.argtypes = [vp, vp, vp, vp, vp, vp, i64, u64, vp]
    lib.dsv3_p2p_destroy.argtypes = [vp]
    lib.dsv3_fp8_linear.argtypes = [vp, i64, i64, vp, vp, i64, ci, vp, vp]
    lib.dsv3_fp8_linear.restype = ci
    lib.dsv3_fp8_gemm_static.argtypes = [vp, vp, vp, vp, i64, i64, i64, vp, vp]
    lib.dsv3_fp8_gemm_static.restype = ci
    lib.dsv3_fp8_gemm_static_scratch_bytes.restype = sz
    lib.dsv3_group_table_bytes.argtypes = [ci]
    lib.dsv3_group_table_bytes.restype = sz
    lib.dsv3_group_table_build.argtypes = [vp, vp, vp, ci, i64, i64, vp]
    lib.dsv3_group_table_build.restype = ci
    lib.dsv3_fp8_gemm_grouped.argtypes = [vp, ci, vp, vp, vp, i64, i64, i64, i64, vp, vp]
    lib.dsv3_fp8_gemm_grouped.restype = ci
    lib.dsv3_moe_combine.argtypes = [vp, vp, vp, i64, ci, i64, vp, vp]
    lib.dsv3_moe_combine.restype = ci
    lib.dsv3_moe_route.argtypes = [vp, vp, i64, ci, ci, ci, vp, vp, vp, vp, vp, vp]
    lib.dsv3_moe_route.restype = ci
    lib.dsv3_set_gemm_policy.argtypes = [ci, ci]
    lib.dsv3_set_num_sms.argtypes = [ci]
    lib.dsv3_set_num_sms.restype = ci
    lib.dsv3_weight_quant.argtypes = [vp, i64, i64, vp, vp, vp]
    lib.dsv3_check_device_status.argtypes = [vp, ctypes.POINTER(ctypes.c_uint32 * 4)]
    for name in ("dsv3_act_quant", "dsv3_weight_dequant", "dsv3_fp8_gemm", "dsv3_set_gemm_policy",
                 "dsv3_weight_quant", "dsv3_check_device_status"):
        getattr(lib, name).restype = ci
    return lib


lib = _load()


def check(status: int) -> None:
    if status != OK:
        detail = lib.dsv3_last_error().decode(errors="replace")
        raise Dsv3Error(status, f"{lib.dsv3_strerror(status).decode()} ({status}): {detail}")
