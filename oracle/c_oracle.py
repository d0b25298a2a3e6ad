"""ctypes access to the C restatement (oracle/awq_oracle.c).  Test and benchmark
infrastructure only.  The library is rebuilt on the machine that runs it, so
its instruction-set flags always match the host."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libawq_oracle.so")
_lib = None


def load(rebuild: bool = False):
    global _lib
    if _lib is not None and not rebuild:
        return _lib
    if rebuild:
        subprocess.run(["make", "-s", "-C", _HERE, "clean"], check=True)
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    lib = C.CDLL(_LIB)
    P, I = C.c_void_p, C.c_int
    lib.awq_oracle_threads.restype = I
    lib.awq_oracle_set_threads.argtypes = [I]
    lib.awq_oracle_set_threads.restype = I
    lib.awq_oracle_dequant.argtypes = [P, P, P, P, I, I, I]
    lib.awq_oracle_matmul.argtypes = [P, P, P, P, I, I, I]
    lib.awq_oracle_linear.argtypes = [P, P, P, P, P, P, I, I, I, I]
    lib.awq_oracle_linear.restype = I
    _lib = lib
    return lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def threads() -> int:
    return load().awq_oracle_threads()


def use_all_cores() -> int:
    """Run the OpenMP loops on every core this process may use, whatever OMP_NUM_THREADS says (launchers
    of multi-process jobs set it to 1).  Returns the thread count now in effect."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return load().awq_oracle_set_threads(max(n, 1))


def dequantize(qweight, qzeros, scales, group_size) -> np.ndarray:
    K, N = qweight.shape[0], qweight.shape[1] * 8
    W = np.empty((K, N), dtype=np.float16)
    load().awq_oracle_dequant(_p(np.ascontiguousarray(qweight)), _p(np.ascontiguousarray(qzeros)),
                              _p(np.ascontiguousarray(scales)), _p(W), K, N, group_size)
    return W


def linear_forward(x, qweight, qzeros, scales, group_size, bias=None) -> np.ndarray:
    K, N = qweight.shape[0], qweight.shape[1] * 8
    x2 = np.ascontiguousarray(x.reshape(-1, K))
    y = np.empty((x2.shape[0], N), dtype=np.float16)
    rc = load().awq_oracle_linear(_p(x2), _p(np.ascontiguousarray(qweight)), _p(np.ascontiguousarray(qzeros)),
                                  _p(np.ascontiguousarray(scales)), _p(bias), _p(y), x2.shape[0], K, N, group_size)
    if rc != 0:
        raise MemoryError("awq_oracle_linear could not allocate the fp16 weight")
    return y.reshape(x.shape[:-1] + (N,))
