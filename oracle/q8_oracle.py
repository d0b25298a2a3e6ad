"""ctypes access to the C restatement of the 8-bit quantized linears (oracle/q8_oracle.c).  Test and benchmark
infrastructure only: the shipped package never imports this.

Arrays are numpy: fp8 / int8 operands as uint8 / int8 byte arrays, 16-bit floats as uint16 bit patterns for bf16
(numpy has no bfloat16) and float16 for fp16.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_build", "libq8_oracle.so")
_lib = None

KIND_E4M3, KIND_INT8, KIND_X_E5M2 = 0, 1, 2
QUANT_FP8_PER_TENSOR, QUANT_FP8_PER_TOKEN, QUANT_FP8_STATIC, QUANT_INT8_PER_TENSOR = range(4)


def load():
    global _lib
    if _lib is not None:
        return _lib
    subprocess.run(["make", "-s", "-C", _HERE, "_build/libq8_oracle.so"], check=True)
    lib = C.CDLL(_LIB)
    P, I, F = C.c_void_p, C.c_int, C.c_float
    lib.q8_oracle_e4m3_to_f32.argtypes = [C.c_uint8]
    lib.q8_oracle_e4m3_to_f32.restype = F
    lib.q8_oracle_e5m2_to_f32.argtypes = [C.c_uint8]
    lib.q8_oracle_e5m2_to_f32.restype = F
    lib.q8_oracle_f32_to_e4m3.argtypes = [F]
    lib.q8_oracle_f32_to_e4m3.restype = C.c_uint8
    lib.q8_oracle_threads.restype = I
    lib.q8_oracle_set_threads.argtypes = [I]
    lib.q8_oracle_set_threads.restype = I
    lib.q8_oracle_gemm_acc.argtypes = [P, I, P, I, I, I, I, I, P]
    lib.q8_oracle_gemm_abs.argtypes = [P, I, P, I, I, I, I, I, P]
    lib.q8_oracle_epilogue_tensorwise.argtypes = [P, P, I, F, F, I, P, I, I]
    lib.q8_oracle_epilogue_rowwise.argtypes = [P, P, I, P, P, P, I, I]
    lib.q8_oracle_quantize.argtypes = [P, I, I, I, I, F, F, I, P, P]
    _lib = lib
    return lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def use_all_cores() -> int:
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return load().q8_oracle_set_threads(max(n, 1))


def e4m3_table() -> np.ndarray:
    lib = load()
    return np.array([lib.q8_oracle_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)


def e5m2_table() -> np.ndarray:
    lib = load()
    return np.array([lib.q8_oracle_e5m2_to_f32(i) for i in range(256)], dtype=np.float32)


def f32_to_e4m3(values: np.ndarray) -> np.ndarray:
    lib = load()
    flat = np.asarray(values, dtype=np.float32).ravel()
    return np.array([lib.q8_oracle_f32_to_e4m3(float(v)) for v in flat], dtype=np.uint8).reshape(np.shape(values))


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _bytes(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view(np.uint8) if a.dtype != np.uint8 else a


def _bias(bias):
    """bias: None, (uint16 bits, 'bf16'), float16 array or float32 array -> (array, kind)."""
    if bias is None:
        return None, 0
    if isinstance(bias, tuple):
        return np.ascontiguousarray(bias[0], dtype=np.uint16), 1
    if bias.dtype == np.float16:
        return np.ascontiguousarray(bias), 2
    if bias.dtype == np.float32:
        return np.ascontiguousarray(bias), 3
    raise TypeError(bias.dtype)


def gemm_acc(xq: np.ndarray, wq: np.ndarray, kind: int) -> np.ndarray:
    """xq [M, K] bytes, wq [N, K] bytes -> the accumulator as the epilogue sees it, fp32 [M, N]."""
    xq, wq = _bytes(xq), _bytes(wq)
    M, K = xq.shape
    N = wq.shape[0]
    assert wq.shape[1] == K
    acc = np.empty((M, N), dtype=np.float32)
    load().q8_oracle_gemm_acc(_p(xq), K, _p(wq), K, M, N, K, kind, _p(acc))
    return acc


def gemm_abs(xq: np.ndarray, wq: np.ndarray, kind: int) -> np.ndarray:
    xq, wq = _bytes(xq), _bytes(wq)
    M, K = xq.shape
    N = wq.shape[0]
    out = np.empty((M, N), dtype=np.float32)
    load().q8_oracle_gemm_abs(_p(xq), K, _p(wq), K, M, N, K, kind, _p(out))
    return out


def tensorwise(xq, wq, bias, alpha: float, beta: float, out_bf16: bool, kind: int = KIND_E4M3, acc=None) -> np.ndarray:
    """-> uint16 bit patterns [M, N] of the bf16 / fp16 result."""
    acc = gemm_acc(xq, wq, kind) if acc is None else acc
    M, N = acc.shape
    b, bk = _bias(bias)
    y = np.empty((M, N), dtype=np.uint16)
    load().q8_oracle_epilogue_tensorwise(_p(acc), _p(b), bk, float(np.float32(alpha)), float(np.float32(beta)),
                                         1 if out_bf16 else 0, _p(y), M, N)
    return y


def rowwise(xq, wq, bias, x_scale, w_scale, kind: int = KIND_E4M3, acc=None) -> np.ndarray:
    """-> uint16 bf16 bit patterns [M, N]."""
    acc = gemm_acc(xq, wq, kind) if acc is None else acc
    M, N = acc.shape
    b, bk = _bias(bias)
    xs = np.ascontiguousarray(x_scale, dtype=np.float32).reshape(M)
    ws = np.ascontiguousarray(w_scale, dtype=np.float32).reshape(N)
    y = np.empty((M, N), dtype=np.uint16)
    load().q8_oracle_epilogue_rowwise(_p(acc), _p(b), bk, _p(xs), _p(ws), _p(y), M, N)
    return y


def quantize(x_bits: np.ndarray, x_bf16: bool, mode: int, static_scale: float = 1.0, weight_scale: float = 1.0,
             host_scalar_reciprocal: bool = True):
    """x_bits [M, K] uint16 bit patterns (or a float16 array when not x_bf16) -> (bytes [M, K], fp32 scales)."""
    x_bits = np.ascontiguousarray(x_bits)
    if x_bits.dtype == np.float16:
        x_bits = x_bits.view(np.uint16)
    assert x_bits.dtype == np.uint16 and x_bits.ndim == 2
    M, K = x_bits.shape
    xq = np.empty((M, K), dtype=np.uint8)
    scales = np.zeros({0: 1, 1: M, 2: 1, 3: 2}[mode], dtype=np.float32)
    load().q8_oracle_quantize(_p(x_bits), 1 if x_bf16 else 0, M, K, mode, float(np.float32(static_scale)),
                              float(np.float32(weight_scale)), 1 if host_scalar_reciprocal else 0, _p(xq), _p(scales))
    return xq, scales
