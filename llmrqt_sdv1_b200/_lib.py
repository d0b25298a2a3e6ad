"""ctypes binding of the C ABI declared in include/awq_b200.h.

The shared library is built in-tree by `setup_runtime.py`.  There is no CPU or
pure-torch fallback: if the library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
# AWQ_B200_LIBRARY points the binding at another build of the same ABI (e.g. a diagnostic build).
LIB_PATH = os.environ.get("AWQ_B200_LIBRARY") or os.path.join(_HERE, "libawq_b200.so")

# name -> (restype, argtypes); mirrors include/awq_b200.h one to one.
_P, _I, _Z = C.c_void_p, C.c_int, C.c_size_t
_COMPUTE = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _Z, _P]
SIGNATURES = {
    "awq_b200_version": (_I, []),
    "awq_b200_status_string": (C.c_char_p, [_I]),
    "awq_b200_last_cuda_error": (_I, []),
    "awq_b200_set_device": (_I, [_I]),
    "awq_b200_packed_bytes": (_Z, [_I, _I]),
    "awq_b200_repack": (_I, [_P, _P, _I, _I, _P]),
    "awq_b200_unpack": (_I, [_P, _P, _I, _I, _P]),
    "awq_b200_dequant": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "awq_b200_dequant_packed": (_I, [_P, _P, _P, _P, _I, _I, _I, _P]),
    "awq_b200_gemv_workspace_bytes": (_Z, [_I, _I, _I]),
    "awq_b200_gemv_counter_bytes": (_Z, [_I]),
    "awq_b200_gemv": (_I, _COMPUTE),
    "awq_b200_gemv_ex": (_I, _COMPUTE + [C.c_uint]),
    "awq_b200_linear_ex": (_I, _COMPUTE + [C.c_uint]),
    "awq_b200_gemv_static_scratch_bytes": (_Z, []),
    "awq_b200_gemv_static": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "awq_b200_gemv_static_status": (_I, [_P, _P]),
    "awq_b200_gemv_workspace_bytes_max": (_Z, [_I, _I, _I]),
    "awq_b200_gemv_plan": (_I, _COMPUTE + [_I, _I, _I, C.c_uint]),
    "awq_b200_gemm_workspace_bytes": (_Z, [_I, _I, _I]),
    "awq_b200_gemm": (_I, _COMPUTE),
    "awq_b200_gemm_smem": (_I, _COMPUTE),
    "awq_b200_gemm_wtm": (_I, _COMPUTE),
    "awq_b200_gemm_wtm_tile": (_I, _COMPUTE + [_I]),
    "awq_b200_skinny_workspace_bytes": (_Z, [_I, _I, _I]),
    "awq_b200_skinny": (_I, _COMPUTE + [C.c_uint]),
    "awq_b200_decode_workspace_bytes": (_Z, [_I, _I, _I]),
    "awq_b200_decode_i8": (_I, _COMPUTE + [C.c_uint]),
    "awq_b200_decode_i8_push": (_I, _COMPUTE[:-1] + [_P, _P, _Z, _I, _I, _P, C.c_uint]),
    "awq_b200_peer_allreduce_flag_bytes": (_Z, []),
    "awq_b200_peer_allreduce": (_I, [_P, _P, _P, _P, _Z, _I, _I, _I, _P]),
    "awq_b200_peer_allreduce_push": (_I, [_P, _P, _P, _P, _P, _Z, _I, _Z, _I, _I, _P]),
    "awq_b200_gemv_max_rows": (_I, []),
    "awq_b200_linear_workspace_bytes": (_Z, [_I, _I, _I]),
    "awq_b200_linear": (_I, _COMPUTE),
    "awq_b200_linear_fused": (_I, _COMPUTE + [C.c_uint]),   # 5th argument: const awq_b200_epilogue*
    "awq_b200_interleave_columns": (_I, [_P, _P, _P, _I, _I, _P]),
    "awq_b200_qk_norm_rope_cache": (_I, [_P, _P, _P, C.c_float, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "awq_b200_attn_workspace_bytes": (_Z, [_I, _I]),
    "awq_b200_attn_decode": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, C.c_float, _P, _Z, _P]),
    "awq_b200_rmsnorm": (_I, [_P, _P, C.c_float, _P, _I, _I, _P]),
    "awq_b200_attn_step": (_I, [_P, _P, _P, C.c_float, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, C.c_float, _P, _Z, _P]),
    "awq_b200_q8_splits": (_I, [_I, _I, _I]),
    "awq_b200_fp8_gemm_tensorwise": (_I, [_P, _I, _P, _I, _P, _I, _P, _I, _I, _I, C.c_float, _P, _P, C.c_float, _I, C.c_uint, _P, _P]),
    "awq_b200_fp8_gemm_rowwise": (_I, [_P, _I, _I, _P, _I, _P, _I, _P, _P, _P, _I, _I, _I, C.c_uint, _P, _P]),
    "awq_b200_int8_gemm_tensorwise": (_I, [_P, _I, _P, _I, _P, _I, _P, _I, _I, _I, C.c_float, _P, _P, C.c_float, _I, C.c_uint, _P, _P]),
    "awq_b200_q8_quantize": (_I, [_P, _I, _I, _I, _I, _P, C.c_float, _P, _P, _P, _P]),
}


class Epilogue(C.Structure):
    """awq_b200_epilogue."""
    _fields_ = [("bias", C.c_void_p), ("residual", C.c_void_p), ("gated", C.c_int)]


class AWQKernelError(RuntimeError):
    """A C-ABI call returned a non-zero status for a reason other than bad arguments."""


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build the CUDA extension first (python setup_runtime.py). "
            "This package has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)   # AttributeError here = header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()

OVERLAP_PREVIOUS = 1
NO_CLUSTER = 2
GEMV_STREAM = 4
GEMV_PER_SPLIT = 8
GEMM_SMEM = 16
ONE_KERNEL_BELOW_8 = 32
ERR_NULL, ERR_SHAPE, ERR_ALIGN, ERR_GROUP, ERR_WORKSPACE, ERR_CUDA, ERR_ARCH, ERR_TOO_LARGE = range(1, 9)
_VALUE_ERRORS = {ERR_NULL, ERR_SHAPE, ERR_ALIGN, ERR_GROUP, ERR_TOO_LARGE}


def check(status: int, what: str) -> None:
    """Raise the Python exception matching a C status: ValueError for argument
    errors (as the reference's std::invalid_argument surfaces,
    LLMQRT/runtime_refact/csrc/awq/gemm_db.cu:702-727), RuntimeError otherwise."""
    if status == 0:
        return
    msg = f"{what}: {lib.awq_b200_status_string(status).decode()} (status {status})"
    if status == ERR_CUDA:
        msg += f", cudaError {lib.awq_b200_last_cuda_error()}"
    if status in _VALUE_ERRORS:
        raise ValueError(msg)
    raise AWQKernelError(msg)


_tls = threading.local()


def set_device(index: int) -> None:
    """Make `index` current inside the library's CUDA runtime for this thread."""
    if getattr(_tls, "device", None) != index:
        check(lib.awq_b200_set_device(index), "awq_b200_set_device")
        _tls.device = index
